"""The decode-attention entry point for callers that cannot allocate device
memory (csrc/attn_decode_noalloc.h), called through its exported C symbol.

Some users of the kernels run where cudaMalloc is off limits (a plug-in inside
a process that owns all device memory, a loop that may not block on the
allocator).  They pass inputs and outputs; the scratch of the split-KV kernel
comes from a fixed array inside the library.  The test calls the symbol several
times in a row, with different inputs, and checks each result against the ordinary
entry point, which gets its scratch from the caller (same kernel, same slices,
same merge order, so the outputs are equal bit for bit: the array's stale contents
from an earlier call must not leak into a later one), and against the plain
statement of attention.  This file sorts last, so a run that stops at the first
failure has already run every other test."""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from gpt_fast_b200.csrc import build
from gpt_fast_b200.ops.types import PagedKV
from test_kernels_gpu import DEV, REF, make_batch, rnd

pytestmark = pytest.mark.gpu
SCRATCH_FLOATS = 1 << 20


def _args(q, out, k, v, table, batch, H, G, d, scale, window, splits):
    p = lambda t: c_void_p(t.data_ptr())
    return [p(q), p(out), p(k), p(v), p(table), c_int(table.shape[1]), c_int(64), c_int(k.shape[0]),
            p(batch.cu_seqlens), p(batch.tok_seq), p(batch.slots), p(batch.lengths), c_int(batch.n_seqs),
            c_int(batch.n_tokens), c_int(H), c_int(G), c_int(d), c_float(scale), c_int(window), c_int(splits)]


def test_no_alloc_entry_point_matches_the_ordinary_one_twice():
    lib = ctypes.CDLL(build.build("attention_bf16"))
    lib.gfb_last_error.restype = ctypes.c_char_p
    noalloc, ordinary = lib.gfb_attn_decode_noalloc, lib.gfb_attn_decode
    noalloc.restype = ordinary.restype = c_int
    H, G, d = 8, 2, 128
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    # the larger call first, so that the array is full of it when the smaller ones run; the last call has one
    # slice and uses no scratch at all
    for call, (starts, seed, splits) in enumerate([([700, 65, 129], 1, 4), ([3, 900, 64], 2, 4), ([300, 20, 64], 3, 2),
                                                   ([40, 500, 1], 4, 1)]):
        batch, table, n_pages = make_batch([1, 1, 1], starts, 7, 64, 20, seed=seed)
        k = rnd(n_pages, G, 64, d, dtype=torch.bfloat16, seed=10 + seed)
        v = rnd(n_pages, G, 64, d, dtype=torch.bfloat16, seed=20 + seed)
        q = rnd(3, H, d, dtype=torch.bfloat16, seed=30 + seed)
        got = torch.zeros(3, H * d, dtype=torch.bfloat16, device=DEV)
        want = torch.zeros_like(got)
        scratch = torch.full((3 * H * splits * (d + 2),), float("nan"), dtype=torch.float32, device=DEV)
        a = _args(q, got, k, v, table, batch, H, G, d, 1 / math.sqrt(d), 0, splits)
        assert noalloc(*a, c_void_p(batch.status.data_ptr()), stream) == 0, lib.gfb_last_error().decode()
        b = _args(q, want, k, v, table, batch, H, G, d, 1 / math.sqrt(d), 0, splits)
        assert ordinary(*b, c_void_p(scratch.data_ptr()), c_void_p(batch.status.data_ptr()), stream) == 0
        torch.cuda.synchronize()
        assert batch.status.tolist()[0] == 0
        assert want.float().abs().sum() > 0
        assert torch.equal(got, want), f"call {call}: the two entry points differ"
        plain = torch.empty_like(got)
        REF.attention(q, PagedKV(k, v, table, 64), batch, plain, H, G, d, 1 / math.sqrt(d), None)
        torch.testing.assert_close(got.float(), plain.float(), rtol=2e-2, atol=1e-2,
                                   msg=lambda m: f"call {call} against the plain statement\n{m}")


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = ctypes.CDLL(build.build("attention_bf16"))
    lib.gfb_last_error.restype = ctypes.c_char_p
    lib.gfb_attn_decode_noalloc.restype = c_int
    H, G, d, splits, T = 32, 8, 128, 32, 16                   # 16*32*32*130 floats > 2^20
    assert T * H * splits * (d + 2) > SCRATCH_FLOATS
    batch, table, n_pages = make_batch([1] * T, [10] * T, T, 64, 2)
    k = torch.zeros(n_pages, G, 64, d, dtype=torch.bfloat16, device=DEV)
    q = torch.zeros(T, H, d, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(T, H * d, dtype=torch.bfloat16, device=DEV)
    a = _args(q, out, k, k, table, batch, H, G, d, 1.0, 0, splits)
    rc = lib.gfb_attn_decode_noalloc(*a, c_void_p(batch.status.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and b"exceed the built-in" in lib.gfb_last_error()
