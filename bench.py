"""Benchmark of the library's flagship step: decoding with Llama-3.1-8B sizes,
random bfloat16 weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]
                    [--skip-points] [--skip-configs] [--skip-shares]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 (a step
is one decode step of the whole batch, timed on the device with CUDA events
around K graph replays after W warm-up steps).  The weights a step streams
(15 GB) are far larger than L2, so nothing is flushed between steps.  Also
reported: `e2e` (the same through the Python entry point `generate`, host token
lists in and out, host clock), `prefill` (one prompt of 2,048 tokens),
`roofline` (bytes a decode step must read / its time, against the measured
copy bandwidth), `points` (decode at batch 1 and 64), `kernel_shares` (where a
decode step's and the prefill's time goes, from events around every launch of an
eager step), `reference_style` (gpt-fast's own two numbers: model bytes x
tokens/s and parameters x tokens/s x 2, generate.py:251-268, :418-424),
`configs` (two more model sizes: Llama-3.2-3B with a batch of 16 unequal
prompts, Llama-2-13B decoding at batch 1/8/32), `clocks` (sampled with
nvidia-smi during the timed region) and `gpu_launches` (this library's kernel
launches inside the timed region).  The README number of gpt-fast for this
model is 93.89 tok/s at batch 1 on an A100 (README.md:98).

`--impl reference` runs gpt-fast itself (see baseline/reference_arm.py) on the
same workload and prints the same line with "impl": "reference".
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


def random_prompts(torch, vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def pages_up(n, page=64):
    return -(-n // page) * page


def decode_bench(gf, torch, model, prompts, context, steps, warmup, prefill_timing=False, full_cache=False):
    """Device-timed decode steps of len(prompts) sequences after their (packed) prefill.  Returns
    (ms per step, key/value bytes a step reads at mid-run, prefill ms or None)."""
    from gpt_fast_b200.engine.generate import _Sampler
    from gpt_fast_b200.sampling import SamplingParams
    batch = len(prompts)
    warmup = max(warmup, 3)
    room = warmup + steps + 4
    max_tokens = batch * context if full_cache else sum(pages_up(len(p) + room) for p in prompts)
    cache = model.new_cache(max_tokens=max_tokens, max_seqs=batch, max_seq_len=context)
    stepper = gf.Stepper(model, cache)
    pre_ms = None
    if prefill_timing:                                  # best of three packed prefills, slots given back in between
        for i in range(4):
            slots = cache.begin(batch)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            stepper.step(slots, prompts, "last")
            stop.record()
            torch.cuda.synchronize()
            cache.end(slots)
            if i > 0:
                pre_ms = min(pre_ms or 1e30, start.elapsed_time(stop))
    slots = cache.begin(batch)
    for s, p in zip(slots, prompts):
        cache.reserve(s, len(p) + room)
    logits = stepper.step(slots, prompts, "last")
    sampler = _Sampler(SamplingParams(0.8, 200, 1234), list(range(batch)), model.device)
    dec = gf.DecodeBatch(stepper, slots, True, sampler)
    gf.sample(logits, 0.8, 200, seed=1234, out=dec.tokens)
    for _ in range(warmup):
        dec.run()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        dec.run()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    stepper.check()
    kv_bytes = sum(len(p) + warmup + steps // 2 for p in prompts) * cache.kv_bytes_per_token()
    cache.end(slots)
    del dec, cache, stepper
    torch.cuda.empty_cache()
    return ms, kv_bytes, pre_ms


def prefill_bench(gf, torch, model, tokens, repeats=3):
    cache = model.new_cache(max_tokens=tokens + 64, max_seqs=1, max_seq_len=tokens + 64)
    stepper = gf.Stepper(model, cache)
    prompt = random_prompts(torch, model.vocab_size, [tokens], 2)[0]
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


def prefill_flops(args, n_layers, lengths, n_logit_rows=1):
    D, H, G, d, I, V = args.dim, args.n_head, args.n_local_heads, args.head_dim, args.intermediate_size, args.vocab_size
    per_token = 2 * (D * (H + 2 * G) * d + H * d * D + 3 * D * I)
    attn = sum(2 * 2 * H * d * (T * (T + 1) / 2) for T in lengths)          # causal QK^T and PV
    return n_layers * (per_token * sum(lengths) + attn) + 2 * D * V * n_logit_rows


def role_of(label, args):
    """Name a traced launch by what it does in a step."""
    D, H, G, d, I, V = args.dim, args.n_head, args.n_local_heads, args.head_dim, args.intermediate_size, args.vocab_size
    if label.startswith("linear "):
        shape, mode = label.split()[1:3]
        n, k = (int(v) for v in shape.split("x"))
        if mode == "swiglu":
            return "w13_swiglu"
        if n == V:
            return "lm_head"
        if n == (H + 2 * G) * d and mode == "store":
            return "qkv"
        if k == I:
            return "w2_add"
        return "wo_add"
    names = {"gfb_rmsnorm": "rmsnorm", "gfb_attn_decode_rope": "rope_append_attn_decode", "gfb_attn_decode": "attn_decode",
             "gfb_attn_prefill_tc": "attn_prefill", "gfb_rope_append": "rope_append",
             "gfb_sample": "sample", "gfb_embed": "embed", "gfb_advance_lengths": "advance_lengths",
             "gfb_add_partials": "add_partials"}
    return names.get(label, label)


def shares_of(records, args):
    from gpt_fast_b200 import ops
    by_role = {}
    for label, ms in ops.trace_times(records):
        r = role_of(label, args)
        by_role[r] = by_role.get(r, 0.0) + ms
    total = sum(by_role.values())
    return {r: {"ms": round(v, 4), "share": round(v / total, 4)} for r, v in sorted(by_role.items(), key=lambda kv: -kv[1])}, total


def kernel_shares(gf, torch, model, graph_ms, prefill_ms):
    """Events around every launch of one eager decode step (batch 8) and of one 2,048-token prefill."""
    from gpt_fast_b200 import ops
    from gpt_fast_b200.engine.generate import _Sampler
    from gpt_fast_b200.sampling import SamplingParams
    cache = model.new_cache(max_tokens=BATCH * pages_up(PROMPT_LEN + 16), max_seqs=BATCH, max_seq_len=CONTEXT)
    stepper = gf.Stepper(model, cache)
    prompts = random_prompts(torch, model.vocab_size, [PROMPT_LEN] * BATCH, 1)
    slots = cache.begin(BATCH)
    for s in slots:
        cache.reserve(s, PROMPT_LEN + 16)
    logits = stepper.step(slots, prompts, "last")
    dec = gf.DecodeBatch(stepper, slots, False, _Sampler(SamplingParams(0.8, 200, 1234), list(range(BATCH)), model.device))
    gf.sample(logits, 0.8, 200, seed=1234, out=dec.tokens)
    for _ in range(3):
        dec.run()
    with ops.trace() as records:
        dec.run()
    decode, total = shares_of(records, model.args)
    cache.end(slots)
    del dec, cache, stepper
    out = {"decode_b8": {"sum_ms": round(total, 4), "step_ms_in_graph": round(graph_ms, 4), "kernels": decode}}
    cache = model.new_cache(max_tokens=PREFILL_TOKENS + 64, max_seqs=1, max_seq_len=PREFILL_TOKENS + 64)
    stepper = gf.Stepper(model, cache)
    prompt = random_prompts(torch, model.vocab_size, [PREFILL_TOKENS], 2)
    for i in range(2):
        slot = cache.begin(1)
        if i == 0:
            stepper.step(slot, prompt, "last")
        else:
            with ops.trace() as records:
                stepper.step(slot, prompt, "last")
            pre, total = shares_of(records, model.args)
        cache.end(slot)
    out["prefill_2048"] = {"sum_ms": round(total, 4), "step_ms": round(prefill_ms, 4), "kernels": pre}
    out["method"] = ("CUDA events around every launch of one eager step: kernels do not overlap their neighbours as "
                     "they do in the captured step, so the sum exceeds the step time; shares say where the work is")
    del cache, stepper
    torch.cuda.empty_cache()
    return out


def reference_style(model, ms_per_step, batch):
    """gpt-fast's two printed figures (generate.py:418-424): model bytes without the embedding x tokens/s of one
    sequence, and parameters x all tokens/s x 2."""
    model_bytes = model.weight_bytes()
    itemsize = 2 if str(model.dtype).endswith("bfloat16") else 4
    steps_per_s = 1000.0 / ms_per_step
    return {"model_bytes": model_bytes, "bandwidth_gbs": model_bytes * steps_per_s / 1e9,
            "tflops": (model_bytes / itemsize) * steps_per_s * batch * 2 / 1e12,
            "note": "model bytes without the embedding x steps per second; parameters x tokens per second x 2"}


def other_config(gf, torch, pk, name, steps, warmup):
    """The two further sizes of the baseline: a batch of 16 unequal prompts on Llama-3.2-3B sizes, and decoding at
    batch 1/8/32 from 256-token prompts on Llama-2-13B sizes (4,096-token context)."""
    t0 = time.time()
    from gpt_fast_b200.config.registry import config_from_name
    cfg = config_from_name(name)
    if name == "llama-2-13b":
        cfg["max_position_embeddings"] = 4096          # Llama 2's own context; gpt-fast's "13B" entry keeps its default 2,048
    model = gf.load(cfg, dtype="bfloat16", device="cuda:0", random_weights=True, seed=0)
    torch.cuda.synchronize()
    ma = model.args
    res = {"layers": len(model.blocks), "dim": ma.dim, "n_head": ma.n_head, "n_kv_head": ma.n_local_heads,
           "intermediate_size": ma.intermediate_size, "vocab_size": ma.vocab_size, "tied": bool(model.spec.tie_embeddings),
           "weight_bytes_per_step": model.weight_bytes()}
    wb = model.weight_bytes()

    def point(prompts, context, prefill_timing=False):
        ms, kv, pre_ms = decode_bench(gf, torch, model, prompts, context, steps, warmup, prefill_timing)
        b = len(prompts)
        achieved = (wb + kv) / (ms * 1e-3) / 1e9
        r = {"batch": b, "ms_per_step": ms, "decode_tokens_per_s": b * 1000.0 / ms, "bytes_per_step": wb + kv,
             "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                          "frac": achieved / pk["hbm_gbs"]}}
        if pre_ms is not None:
            lens = [len(p) for p in prompts]
            fl = prefill_flops(ma, len(model.blocks), lens, n_logit_rows=b)
            r["prefill"] = {"tokens": sum(lens), "ms": pre_ms, "value": sum(lens) / (pre_ms * 1e-3),
                            "frac": fl / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}
        return r

    if name == "llama-3.2-3b":
        g = torch.Generator().manual_seed(4)
        lens = torch.randint(64, 1025, (16,), generator=g).tolist()
        res.update(workload="batch 16, prompt lengths uniform in 64..1,024 (seeded), packed prefill then decode",
                   context=8192, prompt_lengths=lens)
        res["b16_unequal"] = point(random_prompts(torch, model.vocab_size, lens, 5), 8192, prefill_timing=True)
    else:
        res.update(workload="decode at batch 1/8/32 from 256-token prompts", context=4096)
        for b in (1, 8, 32):
            res[f"decode_b{b}"] = point(random_prompts(torch, model.vocab_size, [256] * b, 6), 4096)
    res["seconds"] = time.time() - t0
    del model
    torch.cuda.empty_cache()
    return res


def reference_arm(a):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm as arm
        out = arm.run(a.steps, a.warmup, ClockSampler, peaks(), skip_points=a.skip_points)
    except Exception as e:          # noqa: BLE001  (the arm must always print its line)
        out = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:400]}
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="build fewer layers than the named size has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (quicker)")
    ap.add_argument("--skip-configs", action="store_true", help="leave out the Llama-3.2-3B and Llama-2-13B sizes")
    ap.add_argument("--skip-shares", action="store_true", help="leave out the per-kernel shares")
    a = ap.parse_args()
    if a.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.impl == "reference":
        return reference_arm(a)

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

    headline_prompts = random_prompts(torch, model.vocab_size, [PROMPT_LEN] * BATCH, 1)
    with ClockSampler() as clocks:
        ms, kv_bytes, _ = decode_bench(gf, torch, model, headline_prompts, CONTEXT, a.steps, a.warmup, full_cache=True)
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
    flops = prefill_flops(model.args, n_layers, [PREFILL_TOKENS])
    prefill = {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

    points, point_fracs = {}, {}
    if not a.skip_points:
        for b in (1, 64):
            pms, pkv, _ = decode_bench(gf, torch, model, random_prompts(torch, model.vocab_size, [PROMPT_LEN] * b, 1),
                                       CONTEXT, max(8, a.steps // 2), a.warmup, full_cache=True)
            points[f"decode_b{b}"] = b * 1000.0 / pms
            point_fracs[f"decode_b{b}"] = (weight_bytes + pkv) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"]

    # end to end: host token lists in, host token lists out, through generate()
    prompts = random_prompts(torch, model.vocab_size, [PROMPT_LEN] * BATCH, 3)
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
    model._default_cache = None
    torch.cuda.empty_cache()

    shares = None if a.skip_shares else kernel_shares(gf, torch, model, ms, pre_ms)
    ref_style = reference_style(model, ms, BATCH)
    ma = model.args
    del model
    torch.cuda.empty_cache()

    configs = {}
    if not a.skip_configs and n_layers == full_layers:
        for name in ("llama-3.2-3b", "llama-2-13b"):
            configs[name] = other_config(gf, torch, pk, name, max(8, a.steps // 2), a.warmup)

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
        "points": points, "points_roofline_frac": point_fracs, "clocks": clocks.summary(),
        "reference_style": ref_style, "kernel_shares": shares, "configs": configs,
        "vs_readme_a100_b1": (points.get("decode_b1") / README_B1_TOK_S) if points.get("decode_b1") else None,
        "load_seconds": load_s,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
