"""Times single kernels of the library at given sizes (CUDA events around a
CUDA graph of repeated launches, so that host time is not measured), and is
the small, self-ending workload that profiler captures are taken on.

    python -m gpt_fast_b200.engine.kernel_bench linear --m 8 --n 28672 --k 4096 --mode swiglu
    python -m gpt_fast_b200.engine.kernel_bench linear --m 2048 --n 6144 --k 4096 --mode store
    python -m gpt_fast_b200.engine.kernel_bench attention --batch 8 --context 4000
    python -m gpt_fast_b200.engine.kernel_bench attention --batch 1 --context 0 --new 2048
    python -m gpt_fast_b200.engine.kernel_bench sample --batch 8 --vocab 128256

Weights are cycled through enough copies to exceed the L2 cache, so a memory-
bound kernel is timed against DRAM.  gpt-fast has no per-kernel timing; its
`--profile` exports a torch profiler trace of one sample (generate.py:380-407).
"""
import argparse
import math
import sys

import torch

from .. import ops
from ..ops.types import BatchMeta, PagedKV

L2_BYTES = 126e6


def graph_time_us(fn, reps, warm=2):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def bench_linear(a):
    M, N, K = a.m, a.n, a.k
    copies = max(2, int(3 * L2_BYTES // (N * K * 2)) + 1) if M <= 128 else 1
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out_dtype = torch.float32 if a.mode == "add" else torch.bfloat16
    out = torch.zeros(M, N // 2 if a.mode == "swiglu" else N, device="cuda", dtype=out_dtype)
    us = graph_time_us(lambda i: ops.linear(x, ws[i % copies], out, a.mode, defer=a.mode != "swiglu"), a.reps)
    gbs = N * K * 2 / us / 1e3
    tfs = 2.0 * M * N * K / us / 1e6
    print(f"linear M={M} N={N} K={K} mode={a.mode}: {us:.1f} us, weights at {gbs:.0f} GB/s, {tfs:.0f} TFLOP/s "
          f"(plan swap,bn,splits,stages = {ops.kernels().tc_plan(M, N, K, a.mode)})")


def paged_batch(batch, context, new, heads_kv, head_dim, device="cuda"):
    """`batch` sequences with `context` cached tokens each, bringing `new` tokens; pages in shuffled order."""
    total = context + new
    pages_each = -(-total // 64)
    n_pages = batch * pages_each
    perm = torch.randperm(n_pages).to(torch.int32).view(batch, pages_each)
    table = perm.to(device)
    cu = torch.arange(batch + 1, dtype=torch.int32) * new
    meta = BatchMeta(cu.to(device), torch.arange(batch, dtype=torch.int32).repeat_interleave(new).to(device),
                     torch.arange(batch, dtype=torch.int32).to(device),
                     torch.full((batch,), context, dtype=torch.int32, device=device), batch, batch * new, new, total,
                     ops.new_status(device))
    k = torch.randn(n_pages, heads_kv, 64, head_dim, device=device, dtype=torch.bfloat16)
    v = torch.randn(n_pages, heads_kv, 64, head_dim, device=device, dtype=torch.bfloat16)
    return meta, PagedKV(k, v, table, 64)


def bench_attention(a):
    H, G, d = a.heads, a.kv_heads, a.head_dim
    meta, kv = paged_batch(a.batch, a.context, a.new, G, d)
    q = torch.randn(meta.n_tokens, H, d, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(meta.n_tokens, H * d, device="cuda", dtype=torch.bfloat16)
    kv_bytes = a.batch * (a.context + a.new) * G * d * 2 * 2
    if a.new == 1 and a.partials >= 0:
        # the decode step's kernel: rotary encoding and cache append from the q/k/v product (its partial sums), then attention
        W = (H + 2 * G) * d
        parts = torch.randn(a.partials, meta.n_tokens, W, device="cuda") if a.partials else None
        qkv = torch.randn(meta.n_tokens, W, device="cuda", dtype=torch.bfloat16)
        table = torch.empty(a.context + a.new + 64, d // 2, 2, device="cuda")
        ops.rope_table((1.0 / (10000 ** (torch.arange(d // 2).float() * 2 / d))).cuda(), table)
        us = graph_time_us(lambda i: ops.rope_append_attention(qkv, parts, kv, meta, table, out, H, G, d, "interleaved", True,
                                                               1 / math.sqrt(d)), a.reps)
        print(f"rotary + append + attention decode batch={a.batch} context={a.context} partial sums={a.partials}: {us:.1f} us, "
              f"K/V at {kv_bytes / us / 1e3:.0f} GB/s")
        ops.check_status(meta.status)
        return
    if a.new > 1 and a.tiles:
        run = lambda i: ops.kernels()._attention_bf16(q, kv, meta, out, H, G, d, 1 / math.sqrt(d), None, prefill=True, tiles=a.tiles,
                                                      max_blocks=a.max_blocks)
    else:
        run = lambda i: ops.attention(q, kv, meta, out, H, G, d, 1 / math.sqrt(d))
    us = graph_time_us(run, a.reps)
    if a.new == 1:
        print(f"attention decode batch={a.batch} context={a.context}: {us:.1f} us, K/V at {kv_bytes / us / 1e3:.0f} GB/s")
    else:
        T0, T1 = a.context, a.context + a.new
        flops = a.batch * 4.0 * H * d * (T1 * (T1 + 1) / 2 - T0 * (T0 + 1) / 2)
        print(f"attention prefill batch={a.batch} context={a.context} new={a.new}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s (causal)")
    ops.check_status(meta.status)


def bench_sample(a):
    logits = torch.randn(a.batch, a.vocab, device="cuda")
    tok = torch.empty(a.batch, dtype=torch.int32, device="cuda")
    us = graph_time_us(lambda i: ops.sample(logits, tok, 0.8, a.top_k or None, 1), a.reps)
    print(f"sample batch={a.batch} vocab={a.vocab} top_k={a.top_k}: {us:.1f} us")
    us = graph_time_us(lambda i: ops.argmax(logits, tok), a.reps)
    print(f"argmax batch={a.batch} vocab={a.vocab}: {us:.1f} us")


def bench_norm(a):
    """RMSNorm of the residual stream, as a decode step runs it: the rows' pending partial sums are added on the way."""
    x = torch.randn(a.rows, a.dim, device="cuda")
    w = torch.ones(a.dim, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(a.rows, a.dim, device="cuda", dtype=torch.bfloat16)
    pending = torch.randn(a.partials, a.rows, a.dim, device="cuda") if a.partials else None
    us = graph_time_us(lambda i: ops.rmsnorm(x, w, 1e-5, out, None, pending), a.reps)
    print(f"rmsnorm rows={a.rows} dim={a.dim} pending partial sums={a.partials}: {us:.1f} us")


def main(argv=None):
    ap = argparse.ArgumentParser(prog="kernel_bench")
    sub = ap.add_subparsers(dest="what", required=True)
    p = sub.add_parser("linear")
    p.add_argument("--m", type=int, default=8); p.add_argument("--n", type=int, default=28672)
    p.add_argument("--k", type=int, default=4096); p.add_argument("--mode", default="swiglu", choices=["store", "add", "swiglu"])
    p.add_argument("--reps", type=int, default=10)
    p = sub.add_parser("attention")
    p.add_argument("--batch", type=int, default=8); p.add_argument("--context", type=int, default=4000)
    p.add_argument("--new", type=int, default=1); p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv_heads", type=int, default=8); p.add_argument("--head_dim", type=int, default=128)
    p.add_argument("--tiles", type=int, default=0, help="prefill, head_dim 128: query tiles per block of the tcgen05 kernel (0: its own choice)")
    p.add_argument("--max_blocks", type=int, default=0, help="with --tiles 1: cap of the persistent kernel's grid (0: one block per SM)")
    p.add_argument("--partials", type=int, default=-1,
                   help="decode only: time the fused rotary + append + attention kernel fed by this many partial sums (0: bfloat16 qkv)")
    p.add_argument("--reps", type=int, default=10)
    p = sub.add_parser("sample")
    p.add_argument("--batch", type=int, default=8); p.add_argument("--vocab", type=int, default=128256)
    p.add_argument("--top_k", type=int, default=200); p.add_argument("--reps", type=int, default=10)
    p = sub.add_parser("norm")
    p.add_argument("--rows", type=int, default=8); p.add_argument("--dim", type=int, default=4096)
    p.add_argument("--partials", type=int, default=9); p.add_argument("--reps", type=int, default=10)
    a = ap.parse_args(argv)
    {"linear": bench_linear, "attention": bench_attention, "sample": bench_sample, "norm": bench_norm}[a.what](a)
    ops.check_status(ops.new_status("cuda"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
