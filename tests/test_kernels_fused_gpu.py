"""Kernels that finish a sum split over K on their way: RMSNorm with pending
partial sums, rotary + append from partial sums, the deferred tensor-core product."""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.ops.types import PagedKV
from test_kernels_gpu import DEV, REF, make_batch, rnd

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,D,S", [(1, 64, 2), (8, 4096, 8), (5, 144, 3), (64, 1000, 4), (300, 4096, 4), (200, 520, 3)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_completes_a_pending_sum(T, D, S, out_dtype):
    x = rnd(T, D, scale=2.0)
    pending = rnd(S, T, D, seed=1)
    w = (1 + 0.1 * rnd(D, seed=2))
    x_ref = x.clone()
    out, ref = torch.empty(T, D, dtype=out_dtype, device=DEV), torch.empty(T, D, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w, 1e-5, out, None, pending)
    REF.rmsnorm(x_ref, w, 1e-5, ref, None, pending)
    torch.testing.assert_close(x, x_ref, rtol=1e-6, atol=1e-6)                       # the residual itself was completed
    tol = dict(rtol=2e-5, atol=2e-5) if out_dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.float(), ref.float(), **tol)
    # with a row gather the sum is completed first, for every row
    x2, x2_ref = rnd(T, D, seed=3), rnd(T, D, seed=3)
    rows = torch.tensor([T - 1], dtype=torch.int32, device=DEV)
    o2, r2 = torch.empty(1, D, device=DEV), torch.empty(1, D, device=DEV)
    ops.rmsnorm(x2, w, 1e-5, o2, rows, pending)
    REF.rmsnorm(x2_ref, w, 1e-5, r2, rows, pending)
    torch.testing.assert_close(x2, x2_ref, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(o2, r2, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,q_lens,starts", [(4, 4, 16, [5, 11], [0, 3]), (6, 2, 24, [1, 1, 1], [0, 64, 130]),
                                                 (32, 8, 128, [1] * 8, [128] * 8), (32, 8, 128, [200, 100], [0, 70])])
def test_rope_append_from_partial_sums(dtype, H, G, d, q_lens, starts):
    batch, table, n_pages = make_batch(q_lens, starts, 9, 64, 8)
    T, W = batch.n_tokens, (H + 2 * G) * d
    partials = rnd(3, T, W, seed=1)
    rt = torch.empty(8 * 64, d // 2, 2, device=DEV)
    ops.rope_table((1.0 / (10000 ** (torch.arange(d // 2).float() * 2 / d))).to(DEV), rt)
    pools = [torch.zeros(n_pages, G, 64, d, dtype=dtype, device=DEV) for _ in range(4)]
    q, q_ref = torch.empty(T, H, d, dtype=dtype, device=DEV), torch.empty(T, H, d, dtype=dtype, device=DEV)
    unused = torch.empty(T, W, dtype=dtype, device=DEV)
    ops.rope_append(unused, q, PagedKV(pools[0], pools[1], table, 64), batch, rt, H, G, d, "interleaved", True, partials)
    REF.rope_append(unused, q_ref, PagedKV(pools[2], pools[3], table, 64), batch, rt, H, G, d, "interleaved", True, partials)
    ops.check_status(batch.status)
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q.float(), q_ref.float(), **tol)
    torch.testing.assert_close(pools[0].float(), pools[2].float(), **tol)
    torch.testing.assert_close(pools[1].float(), pools[3].float(), **tol)


@pytest.mark.parametrize("M,N,K", [(8, 4096, 4096), (1, 6144, 4096), (64, 4096, 14336), (16, 512, 1024),
                                   (200, 4096, 4096), (384, 520, 1032), (512, 1000, 4096), (129, 264, 2048)])   # several column tiles of tokens
def test_deferred_product_leaves_partial_sums(M, N, K):
    a = rnd(M, K, dtype=torch.bfloat16)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.02, seed=1)
    x = rnd(M, N, seed=2)
    ref = x.clone()
    pending = ops.linear(a, w, x, "add", defer=True)
    REF.linear(a, w, ref, "add")
    if pending is not None:
        assert pending.shape[1:] == (M, N) and pending.shape[0] > 1
        ops.add_partials(x, pending)
    torch.testing.assert_close(x, ref, rtol=1e-4, atol=2e-4)


PREFILL_CASES = [  # H, G, d, q_lens, starts
    (32, 8, 128, [130, 1, 70], [0, 300, 30]),
    (8, 1, 64, [17, 200], [63, 0]),
    (6, 2, 64, [45, 3, 129], [5, 64, 100]),           # 3 heads per group: 42 tokens per tile, 2 idle rows
    (5, 5, 128, [260], [0]),                          # one head per group: 128 tokens per tile
    (16, 2, 128, [33, 64], [1000, 7]),                # 8 heads per group
    (32, 8, 128, [700], [0]),                         # many key blocks per tile, from position 0
    (8, 2, 128, [300, 150, 64], [500, 1000, 129]),    # long contexts: blocks far below the diagonal
    (24, 8, 128, [200, 45, 3, 129], [0, 5, 64, 1000]),  # head_dim 128, 3 heads per group on the tcgen05 kernel: 42 tokens, 126 rows
    (10, 2, 128, [131, 77], [90, 0]),                 # 5 per group: 25 tokens, 125 rows
    (12, 2, 128, [260], [300]),                       # 6 per group: 21 tokens, 126 rows
    (7, 1, 128, [100, 20], [37, 640]),                # 7 per group: 18 tokens, 126 rows
]


@pytest.mark.parametrize("tiles", [1, 2, -3])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("H,G,d,q_lens,starts", PREFILL_CASES)
def test_attention_bf16_prefill(tiles, window, H, G, d, q_lens, starts):
    """tiles: query tiles per block of the tcgen05 kernel (head_dim 128); the other kernels ignore it.  -3: the
    one-tile kernel on three blocks only, so that every block walks through several tiles in a row."""
    max_blocks = 3 if tiles < 0 else 0
    tiles = 1 if tiles < 0 else tiles
    batch, table, n_pages = make_batch(q_lens, starts, 5, 64, 24, seed=3)
    T, dt = batch.n_tokens, torch.bfloat16
    kv = PagedKV(rnd(n_pages, G, 64, d, dtype=dt, seed=4), rnd(n_pages, G, 64, d, dtype=dt, seed=5), table, 64)
    q = rnd(T, H, d, dtype=dt, seed=6)
    out, ref = torch.empty(T, H * d, dtype=dt, device=DEV), torch.empty(T, H * d, dtype=dt, device=DEV)
    ops.kernels()._attention_bf16(q, kv, batch, out, H, G, d, 1 / math.sqrt(d), window, prefill=True, tiles=tiles,
                                  max_blocks=max_blocks)
    REF.attention(q, kv, batch, ref, H, G, d, 1 / math.sqrt(d), window)
    ops.check_status(batch.status)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)


def test_prefill_attention_finds_a_far_key_and_respects_the_diagonal():
    """A key far back dominates every later query; a key made huge at position p must not leak into queries before p."""
    H, G, d = 8, 2, 128
    batch, table, n_pages = make_batch([300], [0], 2, 64, 8, seed=9)
    dt = torch.bfloat16
    k = rnd(n_pages, G, 64, d, dtype=dt, scale=0.1, seed=1)
    v = rnd(n_pages, G, 64, d, dtype=dt, seed=2)
    q = rnd(300, H, d, dtype=dt, scale=0.1, seed=3)
    slot = int(batch.slots[0])
    q[:, :, 0] = 30.0
    for pos in (3, 200):
        k[int(table[slot, pos // 64]), :, pos % 64, 0] = 30.0 if pos == 3 else 60.0
    kv = PagedKV(k, v, table, 64)
    v3 = v[int(table[slot, 0]), :, 3].repeat_interleave(H // G, dim=0).reshape(H * d).float()
    v200 = v[int(table[slot, 200 // 64]), :, 200 % 64].repeat_interleave(H // G, dim=0).reshape(H * d).float()
    for tiles in (1, 2):
        out = torch.empty(300, H * d, dtype=dt, device=DEV)
        ops.kernels()._attention_bf16(q, kv, batch, out, H, G, d, 1.0, None, prefill=True, tiles=tiles)
        for t in (3, 64, 199):
            torch.testing.assert_close(out[t].float(), v3, rtol=1e-2, atol=1e-2)
        for t in (200, 299):
            torch.testing.assert_close(out[t].float(), v200, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("H,G,d,q_lens,starts", [(32, 8, 128, [200, 31], [0, 77]), (6, 2, 24, [64, 70], [3, 0]), (4, 4, 16, [130], [60])])
def test_rope_append_many_tokens(H, G, d, q_lens, starts):
    """The 16-byte path of the rotary kernel (bfloat16, 64 tokens or more)."""
    dtype = torch.bfloat16
    batch, table, n_pages = make_batch(q_lens, starts, 5, 64, 8)
    T = batch.n_tokens
    qkv = rnd(T, (H + 2 * G) * d, dtype=dtype)
    rt = torch.empty(8 * 64, d // 2, 2, device=DEV)
    ops.rope_table((1.0 / (10000 ** (torch.arange(d // 2).float() * 2 / d))).to(DEV), rt)
    pools = [torch.zeros(n_pages, G, 64, d, dtype=dtype, device=DEV) for _ in range(4)]
    q, q_ref = torch.empty(T, H, d, dtype=dtype, device=DEV), torch.empty(T, H, d, dtype=dtype, device=DEV)
    ops.rope_append(qkv, q, PagedKV(pools[0], pools[1], table, 64), batch, rt, H, G, d)
    REF.rope_append(qkv, q_ref, PagedKV(pools[2], pools[3], table, 64), batch, rt, H, G, d)
    ops.check_status(batch.status)
    torch.testing.assert_close(q.float(), q_ref.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(pools[0].float(), pools[2].float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(pools[1], pools[3])


DECODE_ROPE_CASES = [  # H, G, d, starts (one new token per sequence)
    (32, 8, 128, [0, 63, 64, 130, 700, 5, 127, 1]),
    (6, 2, 64, [0, 200, 64]),
    (5, 5, 128, [1000]),                              # long enough to be cut into slices of the cache
    (16, 2, 64, [33, 639]),
]


@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("pairing", ["interleaved", "half"])
@pytest.mark.parametrize("source", ["partials", "qkv"])
@pytest.mark.parametrize("H,G,d,starts", DECODE_ROPE_CASES)
def test_rotary_append_and_decode_attention_in_one_kernel(window, pairing, source, H, G, d, starts):
    """The decode step's fused kernel against the plain rotary/append followed by the plain attention: the same
    output, and the same keys and values in the cache, at page edges, at position 0 and with a sliced cache."""
    q_lens = [1] * len(starts)
    batch, table, n_pages = make_batch(q_lens, starts, 9, 64, 32, seed=3)
    T, W = batch.n_tokens, (H + 2 * G) * d
    dt = torch.bfloat16
    rt = torch.empty(32 * 64, d // 2, 2, device=DEV)
    ops.rope_table((1.0 / (10000 ** (torch.arange(d // 2).float() * 2 / d))).to(DEV), rt)
    k0, v0 = rnd(n_pages, G, 64, d, dtype=dt, seed=4), rnd(n_pages, G, 64, d, dtype=dt, seed=5)
    kv, kv_ref = PagedKV(k0.clone(), v0.clone(), table, 64), PagedKV(k0.clone(), v0.clone(), table, 64)
    if source == "partials":
        partials, qkv = rnd(3, T, W, seed=1), torch.empty(T, W, dtype=dt, device=DEV)
    else:
        partials, qkv = None, rnd(T, W, dtype=dt, seed=1)
    scale = 1 / math.sqrt(d)
    out, ref = torch.empty(T, H * d, dtype=dt, device=DEV), torch.empty(T, H * d, dtype=dt, device=DEV)
    assert ops.kernels().rope_append_attention(qkv, partials, kv, batch, rt, out, H, G, d, pairing, True, scale, window)
    q_ref = torch.empty(T, H, d, dtype=dt, device=DEV)
    REF.rope_append(qkv, q_ref, kv_ref, batch, rt, H, G, d, pairing, True, partials)
    REF.attention(q_ref, kv_ref, batch, ref, H, G, d, scale, window)
    ops.check_status(batch.status)
    torch.testing.assert_close(kv.k_pool.float(), kv_ref.k_pool.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(kv.v_pool.float(), kv_ref.v_pool.float(), rtol=2e-2, atol=2e-2)
    assert not torch.equal(kv.k_pool, k0)                                   # something was appended
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
    # The kernel asks for its first pages ahead of its dependency wait, on the lengths as they are then, and checks
    # them afterwards: with other lengths at that first read (one step behind; nonsense) nothing may change.
    stale = (batch.lengths - 1).clamp(min=0)
    wild = torch.randint(-5, 1 << 20, batch.lengths.shape, generator=torch.Generator().manual_seed(1)).to(torch.int32).to(DEV)
    for early in (stale, wild):
        kv2, out3 = PagedKV(k0.clone(), v0.clone(), table, 64), torch.empty_like(out)
        assert ops.kernels().rope_append_attention(qkv, partials, kv2, batch, rt, out3, H, G, d, pairing, True, scale, window,
                                                   lengths_early=early)
        ops.check_status(batch.status)
        assert torch.equal(out3, out) and torch.equal(kv2.k_pool, kv.k_pool) and torch.equal(kv2.v_pool, kv.v_pool)
    # append=False: the cache (as the reference left it) is only read
    kept = kv_ref.k_pool.clone()
    out2 = torch.empty_like(out)
    assert ops.kernels().rope_append_attention(qkv, partials, kv_ref, batch, rt, out2, H, G, d, pairing, False, scale, window)
    ops.check_status(batch.status)
    assert torch.equal(kv_ref.k_pool, kept)
    torch.testing.assert_close(out2.float(), ref.float(), rtol=2e-2, atol=1e-2)


def test_fused_decode_attention_sees_the_new_token_and_a_far_key():
    """Weights cannot hide a wrong row here: the new token's own key is made to dominate for one sequence (its
    value must come out), a key hundreds of positions back for another."""
    H, G, d = 8, 2, 128
    starts = [300, 300]
    batch, table, n_pages = make_batch([1, 1], starts, 4, 64, 8, seed=1)
    dt = torch.bfloat16
    rt = torch.empty(8 * 64, d // 2, 2, device=DEV)
    ops.rope_table(torch.zeros(d // 2, device=DEV), rt)                      # no rotation: keys stay what they are
    k_pool = 0.01 * rnd(n_pages, G, 64, d, dtype=dt, seed=4)
    v_pool = rnd(n_pages, G, 64, d, dtype=dt, seed=5)
    W = (H + 2 * G) * d
    qkv = 0.01 * rnd(2, W, dtype=dt, seed=6)
    probe = torch.zeros(d, device=DEV)
    probe[3] = 30.0
    qkv[:, : H * d] = probe.repeat(H).to(dt)                                # every query looks along dimension 3
    qkv[0, H * d: (H + G) * d] = probe.repeat(G).to(dt)                     # sequence 0: its own new key answers
    slots = batch.slots.tolist()
    far_page = int(table[slots[1], 1])                                       # sequence 1: position 64 + 9 answers
    k_pool[far_page, :, 9, :] = probe.to(dt)
    kv = PagedKV(k_pool, v_pool, table, 64)
    out = torch.empty(2, H * d, dtype=dt, device=DEV)
    assert ops.kernels().rope_append_attention(qkv, None, kv, batch, rt, out, H, G, d, "interleaved", True, 1.0, None)
    ops.check_status(batch.status)
    new_v = qkv[0, (H + G) * d:].view(G, d).float()
    for h in range(H):
        torch.testing.assert_close(out[0, h * d:(h + 1) * d].float(), new_v[h // (H // G)], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out[1, h * d:(h + 1) * d].float(), v_pool[far_page, h // (H // G), 9].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("stride,n", [(37, 64), (211, 64), (37, 20), (37, 4)])
def test_decode_attention_of_a_large_batch(stride, n):
    """Many sequences at scattered positions: the fused and the plain entry of the decode kernel against the plain
    implementation.  The cases run the kernel's three buffer depths: more than three blocks per SM with few pages
    each (two tile pairs), with many pages or a grid of about one block per SM (three), and a grid on a quarter of
    the SMs (five)."""
    H, G, d = 32, 8, 128
    starts = [(stride * i) % (8 * stride) for i in range(n)]
    pages = max(starts) // 64 + 2
    batch, table, n_pages = make_batch([1] * n, starts, n + 3, 64, pages, seed=5)
    dt = torch.bfloat16
    W = (H + 2 * G) * d
    rt = torch.empty(pages * 64, d // 2, 2, device=DEV)
    ops.rope_table((1.0 / (10000 ** (torch.arange(d // 2).float() * 2 / d))).to(DEV), rt)
    k0, v0 = rnd(n_pages, G, 64, d, dtype=dt, seed=4), rnd(n_pages, G, 64, d, dtype=dt, seed=5)
    kv, kv_ref = PagedKV(k0.clone(), v0.clone(), table, 64), PagedKV(k0.clone(), v0.clone(), table, 64)
    partials = rnd(3, n, W, seed=1)
    scale = 1 / math.sqrt(d)
    out, ref = torch.empty(n, H * d, dtype=dt, device=DEV), torch.empty(n, H * d, dtype=dt, device=DEV)
    assert ops.kernels().rope_append_attention(None, partials, kv, batch, rt, out, H, G, d, "interleaved", True, scale, None)
    q_ref = torch.empty(n, H, d, dtype=dt, device=DEV)
    REF.rope_append(None, q_ref, kv_ref, batch, rt, H, G, d, "interleaved", True, partials)
    REF.attention(q_ref, kv_ref, batch, ref, H, G, d, scale, None)
    ops.check_status(batch.status)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
    torch.testing.assert_close(kv.k_pool.float(), kv_ref.k_pool.float(), rtol=2e-2, atol=2e-2)
    out2 = torch.empty_like(out)
    ops.kernels()._attention_bf16(q_ref, kv_ref, batch, out2, H, G, d, scale, None, splits=1)
    torch.testing.assert_close(out2.float(), ref.float(), rtol=2e-2, atol=1e-2)


def test_fused_decode_attention_with_a_sequence_that_brings_no_token():
    """Token t is sequence t only while every sequence brings a token; with one that brings none the kernel has to
    look the sequence up (its other way of indexing), and the result is that of the same tokens without that
    sequence in the batch."""
    H, G, d = 8, 2, 128
    starts = [70, 500, 3, 129]
    dt = torch.bfloat16
    W = (H + 2 * G) * d
    rt = torch.empty(10 * 64, d // 2, 2, device=DEV)
    ops.rope_table((1.0 / (10000 ** (torch.arange(d // 2).float() * 2 / d))).to(DEV), rt)
    scale = 1 / math.sqrt(d)
    outs = []
    for q_lens in ([1, 0, 1, 1], [1, 1, 1, 1]):
        batch, table, n_pages = make_batch(q_lens, starts, 6, 64, 10, seed=2)
        T = batch.n_tokens
        k0, v0 = rnd(n_pages, G, 64, d, dtype=dt, seed=4), rnd(n_pages, G, 64, d, dtype=dt, seed=5)
        kv = PagedKV(k0.clone(), v0.clone(), table, 64)
        rows = [i for i, q in enumerate(q_lens) if q]
        qkv = rnd(4, W, dtype=dt, seed=1)[rows].contiguous()
        out = torch.empty(T, H * d, dtype=dt, device=DEV)
        assert ops.kernels().rope_append_attention(qkv, None, kv, batch, rt, out, H, G, d, "interleaved", True, scale, None)
        ops.check_status(batch.status)
        if len(rows) < 4:
            kv_ref, ref, q_ref = PagedKV(k0.clone(), v0.clone(), table, 64), torch.empty_like(out), torch.empty(T, H, d, dtype=dt, device=DEV)
            REF.rope_append(qkv, q_ref, kv_ref, batch, rt, H, G, d, "interleaved", True, None)
            REF.attention(q_ref, kv_ref, batch, ref, H, G, d, scale, None)
            torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
            torch.testing.assert_close(kv.k_pool.float(), kv_ref.k_pool.float(), rtol=2e-2, atol=2e-2)
        outs.append((rows, out))
    (rows_a, a), (rows_b, b) = outs
    assert torch.equal(a, b[rows_a])                      # the same pages and tokens: bit for bit the same rows
