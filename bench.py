"""Benchmark of the library's flagship step: decoding with Llama-3.1-8B sizes,
random bfloat16 weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 (a step
is one decode step of the whole batch, timed on the device with CUDA events
around K graph replays after W warm-up steps).  The weights a step streams
(15 GB) are far larger than L2, so nothing is flushed between steps.  Also
reported: `e2e` (the same through the Python entry point `generate`, host token
lists in and out, host clock), `prefill` (one prompt of 2,048 tokens),
`roofline` (bytes a decode step must read / its time, against the measured
copy bandwidth), `points` (decode at batch 1 and 64), `clocks` (sampled with
nvidia-smi during the timed region) and `gpu_launches` (this library's kernel
launches inside the timed region).  gpt-fast prints tokens/s and model-bytes x
tokens/s per sample (generate.py:418-424); the README number for this model is
93.89 tok/s at batch 1 on an A100 (README.md:98).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_NAME = "llama-3.1-8b"
BATCH, PROMPT_LEN, CONTEXT, PREFILL_TOKENS = 8, 128, 8192, 2048
README_B1_TOK_S = 93.89            # gpt-fast README.md:98, A100, batch 1


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def count_launches(kernels):
    """Wrap the kernel object's launcher so that every launch is counted."""
    counter = {"n": 0}
    inner = kernels._call

    def counted(*a):
        counter["n"] += 1
        return inner(*a)
    kernels._call = counted
    return counter


def decode_bench(gf, torch, model, batch, prompt_len, context, steps, warmup, counter):
    """Device-timed decode steps of `batch` sequences after prompts of prompt_len tokens."""
    from gpt_fast_b200.engine.generate import _Sampler
    from gpt_fast_b200.sampling import SamplingParams
    cache = model.new_cache(max_tokens=batch * context, max_seqs=batch, max_seq_len=context)
    stepper = gf.Stepper(model, cache)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, model.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(batch)]
    slots = cache.begin(batch)
    for s in slots:
        cache.reserve(s, prompt_len + warmup + steps + 4)
    logits = stepper.step(slots, prompts, "last")
    sampler = _Sampler(SamplingParams(0.8, 200, 1234), list(range(batch)), model.device)
    dec = gf.DecodeBatch(stepper, slots, True, sampler)
    gf.sample(logits, 0.8, 200, seed=1234, out=dec.tokens)
    for _ in range(max(warmup, 3)):
        dec.run()
    torch.cuda.synchronize()
    before = counter["n"]
    counter["per_step"] = None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        dec.run()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    stepper.check()
    ctx_len = prompt_len + max(warmup, 3) + steps // 2
    kv_bytes = batch * ctx_len * cache.kv_bytes_per_token()
    cache.end(slots)
    del dec, cache
    torch.cuda.empty_cache()
    return ms, kv_bytes


def prefill_bench(gf, torch, model, tokens, repeats=3):
    cache = model.new_cache(max_tokens=tokens + 64, max_seqs=1, max_seq_len=tokens + 64)
    stepper = gf.Stepper(model, cache)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, model.vocab_size, (tokens,), generator=g).tolist()
    best = None
    for i in range(repeats + 1):
        slot = cache.begin(1)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        stepper.step(slot, [prompt], "last")
        stop.record()
        torch.cuda.synchronize()
        cache.end(slot)
        if i > 0:
            ms = start.elapsed_time(stop)
            best = ms if best is None else min(best, ms)
    stepper.check()
    del cache
    torch.cuda.empty_cache()
    return best


def prefill_flops(args, n_layers, T):
    D, H, G, d, I, V = args.dim, args.n_head, args.n_local_heads, args.head_dim, args.intermediate_size, args.vocab_size
    per_token = 2 * (D * (H + 2 * G) * d + H * d * D + 3 * D * I)
    attn = 2 * 2 * H * d * (T * (T + 1) / 2)          # causal QK^T and PV
    return n_layers * (per_token * T + attn) + 2 * D * V      # logits at one place


def reference_arm():
    ref = os.path.join(ROOT, "baseline", "_ref")
    has_code = os.path.isdir(ref) and any(f.endswith(".py") for _, _, fs in os.walk(ref) for f in fs)
    why = ("gpt-fast's setup.py installs no modules (find_packages() over a flat source tree): "
           "baseline/_ref holds only package metadata, so there is no installed reference code to run")
    if has_code:
        why = "the installed reference needs a downloaded checkpoint and tokenizer.model (generate.py:290-293); none offline"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="build fewer layers than the named size has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (quicker)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm()
    if a.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {a.gpus} is not supported")
        return 2

    import torch
    import gpt_fast_b200 as gf
    from gpt_fast_b200 import ops
    from gpt_fast_b200.config.registry import config_from_name

    pk = peaks()
    full_layers = config_from_name(MODEL_NAME)["num_hidden_layers"]
    n_layers = a.layers or full_layers
    torch.cuda.set_device(0)
    t0 = time.time()
    model = gf.load(MODEL_NAME, dtype="bfloat16", device="cuda:0", random_weights=True, seed=0,
                    n_layers=None if n_layers == full_layers else n_layers)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    counter = count_launches(ops.kernels())
    weight_bytes = model.weight_bytes()

    with ClockSampler() as clocks:
        ms, kv_bytes = decode_bench(gf, torch, model, BATCH, PROMPT_LEN, CONTEXT, a.steps, a.warmup, counter)
    # kernels per step: count one eager step's launches
    cache = model.new_cache(max_tokens=256, max_seqs=1)
    st = gf.Stepper(model, cache)
    slot = cache.begin(1)
    st.step(slot, [[1, 2, 3]], "last")
    n0 = counter["n"]
    st.step(slot, [[4]], "last")
    launches_per_step = counter["n"] - n0 + 1          # + the sampling kernel
    cache.end(slot)
    del cache, st

    value = BATCH * 1000.0 / ms
    step_bytes = weight_bytes + kv_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9

    pre_ms = prefill_bench(gf, torch, model, PREFILL_TOKENS)
    flops = prefill_flops(model.args, n_layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

    points = {}
    if not a.skip_points:
        for b in (1, 64):
            pms, _ = decode_bench(gf, torch, model, b, PROMPT_LEN, CONTEXT,
                                  max(8, a.steps // 2), a.warmup, counter)
            points[f"decode_b{b}"] = b * 1000.0 / pms

    # end to end: host token lists in, host token lists out, through generate()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, model.vocab_size, (PROMPT_LEN,), generator=g).tolist() for _ in range(BATCH)]
    n_new = max(a.steps, 128) + 1          # long enough that the host clock is not measuring noise
    d2h = {"bytes": 0}

    def read_back(request_ids, tokens):
        d2h["bytes"] += len(tokens.tolist()) * 4          # device -> host read of every step's result

    # warm-up with the same token budget: the model keeps the cache it sizes for this call, and the cache keeps the
    # captured decode step, so the timed call below is what every later call of a serving process looks like
    for warm in range(2):      # the first call sizes cache and graphs, the second settles the allocator's pools
        gf.generate(model, prompts, n_new, temperature=0.8, top_k=200, seed=1, callback=read_back)
    d2h["bytes"] = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    seqs, stats = gf.generate(model, prompts, n_new, temperature=0.8, top_k=200, seed=2, callback=read_back)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_steps = stats.decode_steps + 1
    e2e = {"value": stats.generated_tokens / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": (BATCH * PROMPT_LEN * 4 + (3 * BATCH + 1 + BATCH * PROMPT_LEN) * 4) / e2e_steps,
           "d2h_bytes_per_step": d2h["bytes"] / e2e_steps, "includes": "prefill of the prompts, sampling, host copies",
           "decode_only_tokens_per_s": stats.decode_tokens / max(stats.decode_seconds, 1e-9)}

    ma = model.args
    out = {
        "metric": "Llama-3.1-8B bf16 decode tok/s @ batch 8 (points: batch 1/64; prefill tok/s @ 2,048 tok)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": max(a.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids",
        "config": {"model": MODEL_NAME, "global_batch": BATCH, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
                   "parallelism": "single-gpu", "layers": n_layers, "layers_full": full_layers, "dim": ma.dim,
                   "n_head": ma.n_head, "n_kv_head": ma.n_local_heads, "head_dim": ma.head_dim,
                   "intermediate_size": ma.intermediate_size, "vocab_size": ma.vocab_size,
                   "rope_theta": ma.rope_base, "norm_eps": ma.norm_eps, "page_size": 64,
                   "l2": "inputs larger than L2: each step streams all weights", "sampling": "temperature 0.8, top_k 200"},
        "e2e": e2e, "gpu_launches": launches_per_step * a.steps, "launches_per_step": launches_per_step,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": step_bytes, "peaks": pk["source"]},
        "points": points, "clocks": clocks.summary(),
        "vs_readme_a100_b1": (points.get("decode_b1") / README_B1_TOK_S) if points.get("decode_b1") else None,
        "load_seconds": load_s,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
