"""Trace replay: feed given token ids through a model step by step and write
the logits.  Nothing is sampled.

The program drives the library's own loader, model, step function, cache and
kernels (the ones generation uses); it has no forward pass of its own.  gpt-fast
has nothing like it; the nearest is eval.py:134-148, which runs one whole
sequence and returns all logits.

Input, one JSON object per line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries`: for each request its next tokens and `want`, the places among these
tokens whose logits are asked for.  A request's first appearance gives it a
cache slot; `end` lists requests that are finished after the step and give
back what they hold.  For a step in which something is wanted the logits at
the wanted places (in the order of the entries and of `want`) are written to
`<out>/<step>.f32` as little-endian float32 [wanted, vocab].  After every step
`done <step>` is printed and flushed.
"""
import argparse
import json
import os
import sys
from typing import Dict, IO, Optional

import numpy as np
import torch

from ..cache.paged import DEFAULT_PAGE_SIZE
from .load import load
from .step import Stepper


class Replayer:
    def __init__(self, model, max_tokens: int, out_dir: Optional[str]):
        self.model = model
        page = DEFAULT_PAGE_SIZE
        n_pages = -(-max_tokens // page)
        self.cache = model.new_cache(max_tokens=n_pages * page, max_seqs=n_pages,
                                     max_seq_len=min(n_pages * page, model.spec.max_position or n_pages * page))
        self.stepper = Stepper(model, self.cache)
        self.slot_of: Dict[str, int] = {}
        self.out_dir = out_dir
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)

    def run_step(self, rec: dict) -> Optional[np.ndarray]:
        entries = rec.get("entries", [])
        logits = None
        if entries:
            ids = [str(e["id"]) for e in entries]
            fresh = [i for i in ids if i not in self.slot_of]
            if fresh:
                for i, s in zip(fresh, self.cache.begin(len(fresh))):
                    self.slot_of[i] = s
            slots = [self.slot_of[i] for i in ids]
            tokens = [e["tokens"] for e in entries]
            want = [e.get("want", []) for e in entries]
            out = self.stepper.step(slots, tokens, want)
            self.stepper.check()
            if out.shape[0]:
                logits = out.cpu().numpy().astype("<f4", copy=False)
                if self.out_dir:
                    logits.tofile(os.path.join(self.out_dir, f"{rec['step']}.f32"))
        ended = [str(i) for i in rec.get("end", [])]
        if ended:
            unknown = [i for i in ended if i not in self.slot_of]
            if unknown:
                raise KeyError(f"step {rec.get('step')}: 'end' names requests that are not live: {unknown}")
            self.cache.end([self.slot_of.pop(i) for i in ended])
        return logits


def run(model_dir: str, dtype: str, out_dir: str, max_tokens: int, stream: IO[str] = sys.stdin,
        echo: IO[str] = sys.stdout, device: str = "cuda") -> int:
    with torch.no_grad():
        model = load(model_dir, dtype=dtype, device=device)
        rp = Replayer(model, max_tokens, out_dir)
        for line in stream:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            rp.run_step(rec)
            echo.write(f"done {rec['step']}\n")
            echo.flush()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="Replay token traces through the model and write logits.")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="the most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    a = ap.parse_args(argv)
    return run(a.model, a.dtype, a.out, a.max_tokens)
