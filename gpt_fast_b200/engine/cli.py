"""Command line in the manner of gpt-fast's generate.py (generate.py:440-470):
the same option names and meanings where gpt-fast has them.

    python -m gpt_fast_b200.engine.cli --checkpoint_path FOLDER --prompt 128 --max_new_tokens 200 \
        --batch_size 8 --temperature 0.8 --top_k 200 --num_samples 5 --output tokens.jsonl

Differences: `--checkpoint_path` is the model FOLDER (config.json + safetensors), not a converted
model.pth; `--prompt` is text (needs `tokenizer.model` in the folder), an integer n (a synthetic
prompt of n random ids, as gpt-fast's integer prompt, generate.py:325-327), or a comma list of
integers (one synthetic prompt per length: a batch of unequal lengths); there is no torch.compile, so
`--compile`/`--compile_prefill` are accepted and ignored and `--no_cuda_graph` switches the
decode graph off; speculative decoding and the interactive mode are not part of this library.

What gpt-fast prints per sample (time, tokens/s, bandwidth, FLOPS: generate.py:418-424) is printed
here too.  The generated token ids of the last sample go to `--output` (one JSON object per request
and line), or to standard output when there is neither `--output` nor a tokenizer to turn them into
text.  `--profile FILE` (gpt-fast exports a profiler trace of the last sample, generate.py:380-407)
runs the last sample once more without the CUDA graph, with a pair of CUDA events around every
kernel launch, and writes the per-kernel totals as JSON.
"""
import argparse
import json
import os
import sys
import time
from pathlib import Path

NOMINAL_HBM_GBS = 7700.0           # HGX B200 data sheet; used only when no measured peak is given


def _prompt_arg(x):
    try:
        return [int(v) for v in x.split(",")]
    except ValueError:
        return x


def build_parser():
    p = argparse.ArgumentParser(description="Generate tokens with a Llama 2/3 model on one B200.")
    p.add_argument("--prompt", type=_prompt_arg, default="Hello, my name is",
                   help="Input prompt. An integer (or comma list of integers) generates synthetic prompts of those lengths.")
    p.add_argument("--num_samples", type=int, default=5, help="Number of samples.")
    p.add_argument("--max_new_tokens", type=int, default=200, help="Maximum number of new tokens.")
    p.add_argument("--batch_size", type=int, default=1, help="Batch size to benchmark with")
    p.add_argument("--top_k", type=int, default=200, help="Top-k for sampling.")
    p.add_argument("--temperature", type=float, default=0.8, help="Temperature for sampling (0 = greedy).")
    p.add_argument("--checkpoint_path", type=Path, default=None, help="Model folder (config.json + safetensors).")
    p.add_argument("--compile", action="store_true", help="Accepted for compatibility; there is nothing to compile.")
    p.add_argument("--compile_prefill", action="store_true", help="Accepted for compatibility; ignored.")
    p.add_argument("--profile", type=Path, default=None,
                   help="Write per-kernel timings (CUDA events around every launch of the last sample, run eagerly) here.")
    p.add_argument("--device", type=str, default="cuda", help="Device to use (a CUDA device)")
    # not in gpt-fast
    p.add_argument("--model_name", type=str, default=None, help="Named size for --random_weights (e.g. llama-3.1-8b)")
    p.add_argument("--random_weights", action="store_true", help="Seeded random weights instead of a checkpoint")
    p.add_argument("--seed", type=int, default=1234, help="Seed of sampling (and of random weights/prompts)")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--stop_token", type=int, action="append", default=None, help="Stop token id (repeatable)")
    p.add_argument("--no_cuda_graph", action="store_true", help="Run decode steps without a CUDA graph")
    p.add_argument("--max_seq", type=int, default=None,
                   help="Longest sequence (prompt + new tokens) to make room for; default: what this run needs")
    p.add_argument("--output", type=Path, default=None, help="Write the last sample's token ids here, one JSON line per request")
    p.add_argument("--hbm_peak_gbs", type=float, default=None,
                   help="Memory bandwidth to report fractions against (default: MEASURED_PEAKS.json beside the package, else nominal)")
    return p


def _hbm_peak(given):
    if given:
        return given, "given"
    candidates = [Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"]
    if os.environ.get("GPT_FAST_B200_PEAKS"):
        candidates.insert(0, Path(os.environ["GPT_FAST_B200_PEAKS"]))
    for path in candidates:
        try:
            if path.is_file():
                return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (OSError, ValueError, KeyError):
            pass
    return NOMINAL_HBM_GBS, "nominal"


def _fail(msg) -> int:
    print(msg, file=sys.stderr)
    return 2


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    import torch
    import gpt_fast_b200 as gf
    from gpt_fast_b200 import ops

    if not a.device.startswith("cuda"):
        return _fail(f"--device {a.device}: this library runs on a CUDA device only")
    if not torch.cuda.is_available():
        return _fail("no CUDA device is available")
    print(f"Using device={a.device}")
    t0 = time.time()
    try:
        if a.random_weights:
            source = a.model_name or (str(a.checkpoint_path) if a.checkpoint_path else None)
            if source is None:
                return _fail("--random_weights needs --model_name or a folder with config.json")
            model = gf.load(source, dtype=a.dtype, device=a.device, random_weights=True, seed=a.seed)
        else:
            if a.checkpoint_path is None or not a.checkpoint_path.is_dir():
                return _fail(f"--checkpoint_path must be a model folder, got {a.checkpoint_path}")
            model = gf.load(str(a.checkpoint_path), dtype=a.dtype, device=a.device)
    except (gf.ConfigError, gf.WeightError, FileNotFoundError) as e:
        return _fail(f"cannot load the model: {e}")
    torch.cuda.synchronize()
    print(f"Time to load model: {time.time() - t0:.02f} seconds")

    tokenizer = None
    if isinstance(a.prompt, str):
        from .tokenizer import get_tokenizer
        tok_path = (a.checkpoint_path or Path(".")) / "tokenizer.model"
        if not tok_path.is_file():
            return _fail(f"a text prompt needs {tok_path}; give --prompt an integer for a synthetic prompt")
        tokenizer = get_tokenizer(tok_path, str(a.checkpoint_path))
        encoded = [tokenizer.bos_id()] + tokenizer.encode(a.prompt)
        prompts = [encoded] * a.batch_size
    else:
        g = torch.Generator().manual_seed(a.seed)
        lens = a.prompt if len(a.prompt) > 1 else a.prompt * a.batch_size
        if min(lens) < 1:
            return _fail("a synthetic prompt needs at least one token")
        prompts = [torch.randint(0, model.vocab_size, (n,), generator=g).tolist() for n in lens]
    batch = len(prompts)
    prompt_length = sum(len(p) for p in prompts) / batch
    longest = max(len(p) for p in prompts) + a.max_new_tokens
    limit = model.spec.max_position or longest
    max_seq = a.max_seq or longest
    if longest > limit:
        return _fail(f"prompt + --max_new_tokens = {longest} tokens exceed the model's longest sequence {limit}")
    if max_seq > limit:
        return _fail(f"--max_seq {max_seq} exceeds the model's longest sequence {limit}")
    if longest > max_seq:
        return _fail(f"prompt + --max_new_tokens = {longest} tokens do not fit --max_seq {max_seq}")
    from .generate import cache_tokens_needed
    from ..cache.paged import DEFAULT_PAGE_SIZE
    cache = model.new_cache(cache_tokens_needed([len(p) for p in prompts], a.max_new_tokens, batch, DEFAULT_PAGE_SIZE),
                            max_seqs=batch, max_seq_len=max_seq)

    model_size = model.weight_bytes()
    itemsize = 2 if a.dtype == "bfloat16" else 4
    params = model_size // itemsize
    hbm_peak, peak_source = _hbm_peak(a.hbm_peak_gbs)
    kv_per_token = cache.kv_bytes_per_token()
    tokens_per_sec = []
    seqs = None
    for i in range(-1, a.num_samples):                # sample -1 warms up (libraries, graphs), as gpt-fast's compile run
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        seqs, stats = gf.generate(model, prompts, a.max_new_tokens, temperature=a.temperature, top_k=a.top_k,
                                  seed=a.seed + max(i, 0), stop_tokens=a.stop_token, use_graph=not a.no_cuda_graph,
                                  cache=cache)
        torch.cuda.synchronize()
        t = time.perf_counter() - t0
        if i == -1:
            print(f"Warm-up time: {t:.2f} seconds")
            continue
        if tokenizer is not None:
            if batch > 1:
                print("Only displaying the first generation of the batch")
            print(tokenizer.decode(seqs[0]))
        generated = stats.generated_tokens / batch
        tps = generated / t
        tokens_per_sec.append(tps)
        decode_tps = stats.decode_tokens / max(stats.decode_seconds, 1e-9)
        print(f"Time for inference {i + 1}: {t:.02f} sec total, {tps:.02f} tokens/sec per sequence, "
              f"{tps * batch:.02f} tokens/sec in all (decode only: {decode_tps:.02f})")
        print(f"Bandwidth achieved: {model_size * tps / 1e9:.02f} GB/s")
        total_tokens = sum(len(s) for s in seqs)
        print(f"FLOPS achieved: {params * (total_tokens / t) * 2 / 1e12:.02f} TF/s")
        if stats.decode_steps:
            # what a decode step must read: every weight once and the cache of the live sequences (mid-run lengths)
            mean_len = prompt_length + generated / 2
            step_bytes = model_size + (stats.decode_tokens / stats.decode_steps) * mean_len * kv_per_token
            gbs = step_bytes * stats.decode_steps / max(stats.decode_seconds, 1e-9) / 1e9
            print(f"Decode steps read {gbs:.02f} GB/s: {gbs / hbm_peak:.3f} of the {peak_source} memory bandwidth "
                  f"({hbm_peak:.0f} GB/s)")
        print()
    print("==========")
    print(f"Batch Size: {batch}")
    print(f"Prompt Length: {prompt_length:g}")
    print(f"Generated tokens: {a.max_new_tokens}")
    print(f"Average tokens/sec: {sum(tokens_per_sec) / max(len(tokens_per_sec), 1):.2f}")
    print(f"Memory used: {torch.cuda.max_memory_reserved() / 1e9:.02f} GB")

    if seqs is not None and (a.output is not None or tokenizer is None):
        lines = [json.dumps({"request": r, "prompt": p, "tokens": s[len(p):]})
                 for r, (p, s) in enumerate(zip(prompts, seqs))]
        if a.output is not None:
            a.output.write_text("\n".join(lines) + "\n")
        else:
            print("\n".join(lines))

    if a.profile:
        last_seed = a.seed + max(a.num_samples - 1, 0)
        with ops.trace() as records:
            gf.generate(model, prompts, a.max_new_tokens, temperature=a.temperature, top_k=a.top_k, seed=last_seed,
                        stop_tokens=a.stop_token, use_graph=False, cache=cache)
        per = {}
        for label, ms in ops.trace_times(records):
            c = per.setdefault(label, [0, 0.0])
            c[0] += 1
            c[1] += ms
        total = sum(v[1] for v in per.values()) or 1.0
        kernels = [{"kernel": k, "launches": n, "total_ms": round(ms, 4), "mean_us": round(1000 * ms / n, 3),
                    "share": round(ms / total, 4)} for k, (n, ms) in sorted(per.items(), key=lambda kv: -kv[1][1])]
        a.profile.write_text(json.dumps({
            "what": "CUDA events around every kernel launch of the last sample, run without the CUDA graph "
                    "(kernels do not overlap their neighbours here, so the sum exceeds the time of a captured step)",
            "launches": len(records), "sum_ms": round(total, 4), "kernels": kernels}, indent=1) + "\n")
        print(f"Per-kernel timings of the last sample: {a.profile}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
