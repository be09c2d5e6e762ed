"""The reference arm of bench.py: pytorch-labs/gpt-fast itself, unmodified, on the
same workload as the library's own arm.

gpt-fast is a flat tree of modules (its setup.py's find_packages() installs
nothing), so "installing" it means copying model.py, generate.py and
tokenizer.py to baseline/_ref/ (git-ignored); they are imported from there and
from nowhere else.  Nothing of gpt_fast_b200 is imported here.

What runs is gpt-fast's stock path without a checkpoint: only its `main()`
needs model.pth and tokenizer.model (generate.py:290-293).
`Transformer.from_name("llama-3.1-8b")` (model.py:148-150) on the GPU, seeded
N(0, 0.02) matrices, `.to(bfloat16)`; `decode_one_token` compiled with
`torch.compile(mode="reduce-overhead", fullgraph=True)` as generate.py:338-345
does; `generate(model, prompt[128], max_new_tokens, batch_size=8,
temperature=0.8, top_k=200)` (generate.py:139-211).  A decode step is timed on
the device by CUDA events recorded from generate's own `callback`, which
gpt-fast calls once per decoded token (generate.py:77).  If torch.compile cannot
run on the box the arm falls back to the same functions uncompiled (gpt-fast
without `--compile`, also a stock path) and says so in `path`.
"""
import json
import os
import shutil
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
MODULES = ("model.py", "generate.py", "tokenizer.py")
SOURCE_DIRS = ("/root/reference",)


def ensure_installed():
    """Copy the reference's modules to baseline/_ref if they are not there yet."""
    missing = [m for m in MODULES if not os.path.isfile(os.path.join(REF_DIR, m))]
    if not missing:
        return None
    for src in SOURCE_DIRS:
        if all(os.path.isfile(os.path.join(src, m)) for m in MODULES):
            os.makedirs(REF_DIR, exist_ok=True)
            for m in MODULES:
                shutil.copyfile(os.path.join(src, m), os.path.join(REF_DIR, m))
            return None
    return f"baseline/_ref lacks {missing} and no reference source tree is at {SOURCE_DIRS}"


class _StepTimer:
    """generate()'s callback: records an event after `warmup` decoded tokens and after `warmup + steps`."""

    def __init__(self, torch, warmup, steps):
        self.torch, self.warmup, self.steps, self.n = torch, warmup, steps, 0
        self.start = torch.cuda.Event(enable_timing=True)
        self.stop = torch.cuda.Event(enable_timing=True)

    def __call__(self, token):
        self.n += 1
        if self.n == self.warmup:
            self.start.record()
        elif self.n == self.warmup + self.steps:
            self.stop.record()

    def ms_per_step(self):
        self.torch.cuda.synchronize()
        return self.start.elapsed_time(self.stop) / self.steps


def run(steps, warmup, clock_sampler_cls, peaks, skip_points=False, budget_s=420.0, model_name="llama-3.1-8b",
        batch=8, prompt_len=128, context=8192, prefill_tokens=2048, point_batches=(1, 64)):
    t_begin = time.time()
    why = ensure_installed()
    if why:
        return {"impl": "reference", "unavailable": why}
    sys.path.insert(0, REF_DIR)
    try:
        import torch
        if not torch.cuda.is_available():
            return {"impl": "reference", "unavailable": "no CUDA device"}
        import generate as ref_generate          # baseline/_ref/generate.py
        import model as ref_model                # baseline/_ref/model.py
        for mod in (ref_generate, ref_model):
            if os.path.dirname(os.path.abspath(mod.__file__)) != REF_DIR:
                return {"impl": "reference", "unavailable": f"module {mod.__name__} came from {mod.__file__}, not baseline/_ref"}
    except Exception as e:                       # noqa: BLE001
        return {"impl": "reference", "unavailable": f"import of the reference failed: {type(e).__name__}: {e}"[:400]}

    device = "cuda"
    warmup = max(warmup, 3)
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    t0 = time.time()
    with torch.device(device):
        model = ref_model.Transformer.from_name(model_name)
    with torch.no_grad():
        for p in model.parameters():
            if p.ndim >= 2:
                p.normal_(0.0, 0.02)
    model = model.to(device=device, dtype=torch.bfloat16).eval()
    torch.cuda.synchronize()
    load_s = time.time() - t0
    model_size, params = ref_generate._get_model_size(model)
    cfg = model.config

    sampling = dict(temperature=0.8, top_k=200)
    n_new = max(warmup + steps + 2, max(steps, 128) + 1)
    g = torch.Generator().manual_seed(1)
    prompt_host = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g, dtype=torch.int64).pin_memory()

    path = "torch.compile(decode_one_token, mode='reduce-overhead', fullgraph=True), eager prefill (gpt-fast --compile)"
    compile_error = None
    eager_decode = ref_generate.decode_one_token
    try:
        ref_generate.decode_one_token = torch.compile(eager_decode, mode="reduce-overhead", fullgraph=True)
        t0 = time.time()
        ref_generate.generate(model, prompt_host.to(device), n_new, batch_size=batch, interactive=False,
                              draft_model=None, **sampling)
        torch.cuda.synchronize()
        compile_s = time.time() - t0
    except Exception as e:                       # noqa: BLE001
        compile_error = f"{type(e).__name__}: {e}"[:400]
        ref_generate.decode_one_token = eager_decode
        path = "eager (gpt-fast without --compile): torch.compile failed on this box"
        t0 = time.time()
        try:
            torch._dynamo.reset()
            ref_generate.generate(model, prompt_host.to(device), n_new, batch_size=batch, interactive=False,
                                  draft_model=None, **sampling)
            torch.cuda.synchronize()
        except Exception as e2:                  # noqa: BLE001
            return {"impl": "reference", "unavailable": f"the reference failed to run: {type(e2).__name__}: {e2}"[:400],
                    "compile_error": compile_error}
        compile_s = time.time() - t0

    def fresh_caches():
        """gpt-fast keeps a cache that is large enough (model.py:118-119), but its forward needs the batch to be
        exactly the cache's (model.py:94-100); forgetting the sizes makes the next generate() set up anew."""
        model.max_batch_size, model.max_seq_length = -1, -1

    def timed_decode(b):
        timer = _StepTimer(torch, warmup, steps)
        ref_generate.generate(model, prompt_host.to(device), n_new, batch_size=b, interactive=False,
                              draft_model=None, callback=timer, **sampling)
        return timer.ms_per_step()

    with clock_sampler_cls() as clocks:
        ms = timed_decode(batch)
    cache_len = int(model.max_seq_length)
    ctx_len = prompt_len + warmup + steps // 2
    kv_per_token = 2 * cfg.n_layer * cfg.n_local_heads * cfg.head_dim * 2
    step_bytes = model_size + batch * ctx_len * kv_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # end to end: pinned host prompt in, host token lists out, the whole generate() call on the host clock
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    y, _ = ref_generate.generate(model, prompt_host.to(device, non_blocking=True), n_new, batch_size=batch,
                                 interactive=False, draft_model=None, **sampling)
    out_host = y.cpu()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e = {"value": batch * n_new / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": prompt_host.numel() * prompt_host.element_size() / n_new,
           "d2h_bytes_per_step": out_host.numel() * out_host.element_size() / n_new,
           "includes": "prefill of the prompts, sampling, host copies"}

    points = {}
    if not skip_points:
        for b in point_batches:
            if time.time() - t_begin > budget_s:
                points[f"decode_b{b}"] = None
                continue
            try:
                fresh_caches()
                ref_generate.generate(model, prompt_host.to(device), n_new, batch_size=b, interactive=False,
                                      draft_model=None, **sampling)          # compiles / records for this batch size
                points[f"decode_b{b}"] = b * 1000.0 / timed_decode(b)
            except Exception as e:               # noqa: BLE001
                points[f"decode_b{b}"] = None
                points[f"decode_b{b}_error"] = f"{type(e).__name__}: {e}"[:200]

    prefill = None
    try:
        fresh_caches()
        with torch.device(device):
            model.setup_caches(max_batch_size=1, max_seq_length=prefill_tokens)
        g = torch.Generator().manual_seed(2)
        x = torch.randint(0, cfg.vocab_size, (1, prefill_tokens), generator=g, dtype=torch.int64).to(device)
        pos = torch.arange(0, prefill_tokens, device=device)
        best = None
        with torch.no_grad():
            for i in range(4):
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                ref_generate.prefill(model, x, pos, **sampling)
                e.record()
                torch.cuda.synchronize()
                if i > 0:
                    t = s.elapsed_time(e)
                    best = t if best is None else min(best, t)
        D, H, G, d, I, V, L = cfg.dim, cfg.n_head, cfg.n_local_heads, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size, cfg.n_layer
        T = prefill_tokens
        flops = L * (2 * (D * (H + 2 * G) * d + H * d * D + 3 * D * I) * T + 4 * H * d * (T * (T + 1) / 2)) + 2 * D * V
        prefill = {"value": T / (best * 1e-3), "tokens": T, "ms": best,
                   "frac": flops / (best * 1e-3) / (peaks["bf16_tflops"] * 1e12),
                   "note": "eager prefill (gpt-fast's default); computes logits at all 2,048 places, counted as one"}
    except Exception as e:                       # noqa: BLE001
        prefill = {"error": f"{type(e).__name__}: {e}"[:300]}

    value = batch * 1000.0 / ms
    out = {
        "impl": "reference", "path": path,
        "metric": "Llama-3.1-8B bf16 decode tok/s @ batch 8 (points: batch 1/64; prefill tok/s @ 2,048 tok)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids",
        "config": {"model": model_name, "global_batch": batch, "seq_len": context, "cache_len": cache_len, "prompt_len": prompt_len,
                   "parallelism": "single-gpu", "layers": cfg.n_layer, "layers_full": cfg.n_layer, "dim": cfg.dim,
                   "n_head": cfg.n_head, "n_kv_head": cfg.n_local_heads, "head_dim": cfg.head_dim,
                   "intermediate_size": cfg.intermediate_size, "vocab_size": cfg.vocab_size, "rope_theta": cfg.rope_base,
                   "norm_eps": cfg.norm_eps,
                   "cache": "gpt-fast sizes its cache to prompt + new tokens (generate.py:160-168), at most block_size",
                   "l2": "inputs larger than L2: each step streams all weights", "sampling": "temperature 0.8, top_k 200"},
        "e2e": e2e, "gpu_launches": 0, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "bytes_per_step": step_bytes, "peaks": peaks["source"]},
        "reference_style": {"model_bytes": model_size, "bandwidth_gbs": model_size * (1000.0 / ms) / 1e9,
                            "note": "model bytes without the embedding x steps per second (generate.py:251-268, :422)"},
        "points": points, "clocks": clocks.summary(), "load_seconds": load_s, "compile_seconds": compile_s,
    }
    if compile_error:
        out["compile_error"] = compile_error
    return out


if __name__ == "__main__":
    print(json.dumps(ensure_installed() or "installed"))
