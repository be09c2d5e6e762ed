"""bin/trace_run as a user runs it: a subprocess fed JSON lines step by step,
its <step>.f32 files compared with the plain implementation, for the three ways
of cutting the same requests, in float32 and bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama
import traces
from conftest import assert_within_bf16_noise

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def run_trace(folder, dtype, steps, out_dir, max_tokens):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_trace_run_three_cuts(tiny_folders, tmp_path, name, dtype):
    folder = tiny_folders[name]
    p, cfg = plain_llama.load_folder(folder)
    V = cfg["vocab_size"]
    reqs = traces.make_requests(V, [40, 3, 77, 64, 33], seed=21)
    ref, emu = {}, {}
    for rid, toks in reqs.items():
        logits = plain_llama.forward(toks, p, cfg)
        rounded = plain_llama.forward(toks, p, cfg, act=torch.bfloat16)       # the noise of bfloat16 on this model
        for j in range(len(toks) - traces.tail_of(toks), len(toks)):
            ref[(rid, j)] = logits[j]
            emu[(rid, j)] = rounded[j]
    results = {}
    for cut, steps in (("whole", traces.whole(reqs)), ("stepped", traces.stepped(reqs)), ("batched", traces.batched(reqs, 3))):
        out_dir = str(tmp_path / cut)
        run_trace(folder, dtype, steps, out_dir, traces.peak_tokens(steps))
        outputs = {}
        for st in steps:
            f = os.path.join(out_dir, f"{st['step']}.f32")
            wanted = sum(len(e["want"]) for e in st["entries"])
            assert os.path.exists(f) == (wanted > 0)
            if wanted:
                a = np.fromfile(f, dtype="<f4")
                assert a.size == wanted * V
                outputs[st["step"]] = a.reshape(wanted, V)
        rows = traces.collect(steps, outputs, V)
        assert set(rows) == set(ref)
        for key in sorted(ref):
            got, where = torch.from_numpy(rows[key].copy()), f"{cut}: request {key[0]}, token {key[1]}"
            if dtype == "float32":
                torch.testing.assert_close(got, ref[key], rtol=1e-4, atol=2e-5, msg=lambda m, where=where: f"{where}\n{m}")
            else:
                assert_within_bf16_noise(got, ref[key], emu[key], where)
        results[cut] = rows
    if dtype == "float32":
        for key in ref:
            for cut in ("stepped", "batched"):
                np.testing.assert_allclose(results[cut][key], results["whole"][key], rtol=1e-5, atol=2e-6)
