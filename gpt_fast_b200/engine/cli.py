"""Command line in the manner of gpt-fast's generate.py (generate.py:440-470):
the same option names and meanings where gpt-fast has them.

    python -m gpt_fast_b200.engine.cli --checkpoint_path FOLDER --prompt 128 --max_new_tokens 200 \
        --batch_size 8 --temperature 0.8 --top_k 200 --num_samples 5

Differences: `--checkpoint_path` is the model FOLDER (config.json + safetensors), not a converted
model.pth; `--prompt` is text (needs `tokenizer.model` in the folder), an integer n (a synthetic
prompt of n random ids, as gpt-fast's integer prompt, generate.py:325-327), or a comma list of
integers (one synthetic prompt per length: a batch of unequal lengths); there is no torch.compile, so
`--compile`/`--compile_prefill` are accepted and ignored and `--no_cuda_graph` switches the
decode graph off; speculative decoding and the interactive mode are not part of this library.
"""
import argparse
import sys
import time
from pathlib import Path

import torch


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
    p.add_argument("--profile", type=Path, default=None, help="Write per-sample timings to this file.")
    p.add_argument("--device", type=str, default="cuda", help="Device to use (a CUDA device)")
    # not in gpt-fast
    p.add_argument("--model_name", type=str, default=None, help="Named size for --random_weights (e.g. llama-3.1-8b)")
    p.add_argument("--random_weights", action="store_true", help="Seeded random weights instead of a checkpoint")
    p.add_argument("--seed", type=int, default=1234, help="Seed of sampling (and of random weights/prompts)")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--stop_token", type=int, action="append", default=None, help="Stop token id (repeatable)")
    p.add_argument("--no_cuda_graph", action="store_true", help="Run decode steps without a CUDA graph")
    return p


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    import gpt_fast_b200 as gf

    print(f"Using device={a.device}")
    t0 = time.time()
    if a.random_weights:
        source = a.model_name or (str(a.checkpoint_path) if a.checkpoint_path else None)
        if source is None:
            print("--random_weights needs --model_name or a folder with config.json", file=sys.stderr)
            return 2
        model = gf.load(source, dtype=a.dtype, device=a.device, random_weights=True, seed=a.seed)
    else:
        if a.checkpoint_path is None or not a.checkpoint_path.is_dir():
            print(f"--checkpoint_path must be a model folder, got {a.checkpoint_path}", file=sys.stderr)
            return 2
        model = gf.load(str(a.checkpoint_path), dtype=a.dtype, device=a.device)
    torch.cuda.synchronize()
    print(f"Time to load model: {time.time() - t0:.02f} seconds")

    tokenizer = None
    if isinstance(a.prompt, str):
        from .tokenizer import get_tokenizer
        tok_path = (a.checkpoint_path or Path(".")) / "tokenizer.model"
        if not tok_path.is_file():
            print(f"a text prompt needs {tok_path}; give --prompt an integer for a synthetic prompt", file=sys.stderr)
            return 2
        tokenizer = get_tokenizer(tok_path, str(a.checkpoint_path))
        encoded = [tokenizer.bos_id()] + tokenizer.encode(a.prompt)
        prompts = [encoded] * a.batch_size
    else:
        g = torch.Generator().manual_seed(a.seed)
        lens = a.prompt if len(a.prompt) > 1 else a.prompt * a.batch_size
        prompts = [torch.randint(0, model.vocab_size, (n,), generator=g).tolist() for n in lens]
    batch = len(prompts)
    prompt_length = sum(len(p) for p in prompts) / batch

    model_size = model.weight_bytes()
    tokens_per_sec = []
    lines = []
    for i in range(-1, a.num_samples):                # sample -1 warms up (libraries, graphs), as gpt-fast's compile run
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        seqs, stats = gf.generate(model, prompts, a.max_new_tokens, temperature=a.temperature, top_k=a.top_k,
                                  seed=a.seed + max(i, 0), stop_tokens=a.stop_token, use_graph=not a.no_cuda_graph)
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
        line = (f"Time for inference {i + 1}: {t:.02f} sec total, {tps:.02f} tokens/sec per sequence, "
                f"{tps * batch:.02f} tokens/sec in all (decode only: {decode_tps:.02f})")
        print(line)
        lines.append(line)
        print(f"Bandwidth achieved: {model_size * tps / 1e9:.02f} GB/s")
        print()
    print("==========")
    print(f"Batch Size: {batch}")
    print(f"Prompt Length: {prompt_length:g}")
    print(f"Generated tokens: {a.max_new_tokens}")
    print(f"Average tokens/sec: {sum(tokens_per_sec) / max(len(tokens_per_sec), 1):.2f}")
    print(f"Memory used: {torch.cuda.max_memory_reserved() / 1e9:.02f} GB")
    if a.profile:
        a.profile.write_text("\n".join(lines) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
