"""Each kernel alone against its plain reference (tests/plain_ops.py), at sizes
other than the engine's: head sizes in steps of 16, odd head and group counts,
widths and vocabularies that are no power of two, both precisions."""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.ops.types import BatchMeta, PagedKV
import plain_ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
REF = plain_ops.PlainOps()
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def make_batch(q_lens, starts, n_slots, page_size, max_pages, seed=0):
    """A batch whose sequences sit in shuffled slots with shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    n = len(q_lens)
    slots = torch.randperm(n_slots, generator=g)[:n].tolist()
    lengths = torch.zeros(n_slots, dtype=torch.int32)
    table = torch.full((n_slots, max_pages), -1, dtype=torch.int32)
    need = [-(-(s + q) // page_size) for s, q in zip(starts, q_lens)]
    n_pages = sum(need) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    for i, s in enumerate(slots):
        lengths[s] = starts[i]
        for j in range(min(need[i], max_pages)):
            table[s, j] = perm.pop()
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    tok_seq = [i for i, q in enumerate(q_lens) for _ in range(q)]
    batch = BatchMeta(torch.tensor(cu, dtype=torch.int32).to(DEV), torch.tensor(tok_seq, dtype=torch.int32).to(DEV),
                      torch.tensor(slots, dtype=torch.int32).to(DEV), lengths.to(DEV), n, cu[-1], max(q_lens),
                      max(s + q for s, q in zip(starts, q_lens)), ops.new_status(DEV))
    return batch, table.to(DEV), n_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,D,V", [(7, 80, 100), (33, 4096, 517), (1, 144, 320)])
def test_embed(dtype, T, D, V):
    table = rnd(V, D, dtype=dtype)
    tokens = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    out, ref = torch.empty(T, D, device=DEV), torch.empty(T, D, device=DEV)
    st = ops.new_status(DEV)
    ops.embed(tokens, table, out, st)
    REF.embed(tokens, table, ref, st.clone())
    assert torch.equal(out, ref)
    ops.check_status(st)


def test_embed_reports_bad_token():
    table = rnd(10, 16)
    tokens = torch.tensor([1, 12, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, 16, device=DEV)
    st = ops.new_status(DEV)
    ops.embed(tokens, table, out, st)
    with pytest.raises(ops.KernelError, match="token id out of range"):
        ops.check_status(st)
    assert out[1].abs().sum() == 0
    ops.check_status(st)        # cleared


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("w_dtype", DTYPES)
@pytest.mark.parametrize("T,D,eps", [(5, 64, 1e-5), (19, 144, 1e-6), (3, 4096, 1e-5), (2, 5000, 1e-3)])
def test_rmsnorm(out_dtype, w_dtype, T, D, eps):
    x = rnd(T, D, scale=3.0)
    w = (1 + 0.1 * rnd(D, seed=1)).to(w_dtype)
    out, ref = torch.empty(T, D, dtype=out_dtype, device=DEV), torch.empty(T, D, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w, eps, out)
    REF.rmsnorm(x, w, eps, ref)
    torch.testing.assert_close(out.float(), ref.float(), **tol(out_dtype))
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    out2, ref2 = out[:2].clone(), ref[:2].clone()
    ops.rmsnorm(x, w, eps, out2, rows)
    REF.rmsnorm(x, w, eps, ref2, rows)
    torch.testing.assert_close(out2.float(), ref2.float(), **tol(out_dtype))


def test_rmsnorm_small_values_need_eps():
    """With tiny activations eps dominates: a kernel that put eps outside the root would differ."""
    x = rnd(4, 96, scale=1e-4)
    w = torch.ones(96, device=DEV)
    out, ref = torch.empty(4, 96, device=DEV), torch.empty(4, 96, device=DEV)
    ops.rmsnorm(x, w, 1e-5, out)
    REF.rmsnorm(x, w, 1e-5, ref)
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-9)


@pytest.mark.parametrize("mode", ["store", "add", "swiglu"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 172, 64), (3, 64, 172), (70, 130, 37), (129, 320, 144), (8, 258, 200)])
def test_linear_generic(mode, dtype, M, N, K):
    a = rnd(M, K, dtype=dtype)
    w = rnd(N, K, dtype=dtype, scale=0.1, seed=1)
    if mode == "add":
        out = rnd(M, N, seed=2)
        ref = out.clone()
    else:
        No = N // 2 if mode == "swiglu" else N
        out = torch.empty(M, No, dtype=dtype, device=DEV)
        ref = torch.empty_like(out)
    ops.linear(a, w, out, mode)
    REF.linear(a, w, ref, mode)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))


def test_linear_f32_rows_do_not_depend_on_the_batch():
    a = rnd(37, 200)
    w = rnd(90, 200, scale=0.1, seed=1)
    whole = torch.empty(37, 90, device=DEV)
    ops.linear(a, w, whole)
    for m in (0, 17, 36):
        one = torch.empty(1, 90, device=DEV)
        ops.linear(a[m:m + 1].contiguous(), w, one)
        assert torch.equal(one[0], whole[m])


def test_linear_bf16_to_f32_logits():
    a = rnd(4, 144, dtype=torch.bfloat16)
    w = rnd(320, 144, dtype=torch.bfloat16, scale=0.1, seed=1)
    out, ref = torch.empty(4, 320, device=DEV), torch.empty(4, 320, device=DEV)
    ops.linear(a, w, out)
    REF.linear(a, w, ref)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("P,half", [(70, 8), (300, 12), (1000, 64)])
def test_rope_table(P, half):
    inv = (1.0 / (10000 ** (torch.arange(half).float() / half))).to(DEV)
    t, r = torch.empty(P, half, 2, device=DEV), torch.empty(P, half, 2, device=DEV)
    ops.rope_table(inv, t)
    REF.rope_table(inv, r)
    torch.testing.assert_close(t, r, rtol=0, atol=2e-6)


KV_CASES = [  # H, G, d, page_size, q_lens, starts
    (4, 4, 16, 64, [5, 11, 17], [0, 0, 0]),
    (6, 2, 24, 64, [1, 7, 30, 64], [0, 0, 0, 0]),
    (6, 2, 48, 64, [1, 1, 1], [63, 64, 200]),
    (3, 1, 80, 16, [4, 1, 9], [30, 0, 17]),
    (8, 2, 128, 64, [130, 1], [0, 300]),
]


@pytest.mark.parametrize("pairing", ["interleaved", "half"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,page,q_lens,starts", KV_CASES)
def test_rope_append(pairing, dtype, H, G, d, page, q_lens, starts):
    max_pages = 8 if page == 64 else 32
    batch, table, n_pages = make_batch(q_lens, starts, 9, page, max_pages)
    T = batch.n_tokens
    qkv = rnd(T, (H + 2 * G) * d, dtype=dtype)
    rt = torch.empty(max_pages * page, d // 2, 2, device=DEV)
    ops.rope_table((1.0 / (10000 ** (torch.arange(d // 2).float() * 2 / d))).to(DEV), rt)
    pools = [torch.zeros(n_pages, G, page, d, dtype=dtype, device=DEV) for _ in range(4)]
    kv, kv_ref = PagedKV(pools[0], pools[1], table, page), PagedKV(pools[2], pools[3], table, page)
    q, q_ref = torch.empty(T, H, d, dtype=dtype, device=DEV), torch.empty(T, H, d, dtype=dtype, device=DEV)
    ops.rope_append(qkv, q, kv, batch, rt, H, G, d, pairing)
    REF.rope_append(qkv, q_ref, kv_ref, batch, rt, H, G, d, pairing)
    ops.check_status(batch.status)
    torch.testing.assert_close(q.float(), q_ref.float(), **tol(dtype))
    torch.testing.assert_close(pools[0].float(), pools[2].float(), **tol(dtype))
    assert torch.equal(pools[1], pools[3])
    # append=False leaves the cache alone
    before = pools[0].clone()
    ops.rope_append(qkv, q, kv, batch, rt, H, G, d, pairing, append=False)
    assert torch.equal(before, pools[0])


def test_rope_append_reports_a_position_beyond_the_cache():
    batch, table, n_pages = make_batch([3], [126], 2, 64, 2)
    H, G, d = 2, 1, 16
    qkv = rnd(3, (H + 2 * G) * d)
    rt = torch.zeros(128, d // 2, 2, device=DEV)
    pool = torch.zeros(n_pages, G, 64, d, device=DEV)
    q = torch.empty(3, H, d, device=DEV)
    ops.rope_append(qkv, q, PagedKV(pool, pool.clone(), table, 64), batch, rt, H, G, d)
    with pytest.raises(ops.KernelError, match="position beyond the cache"):
        ops.check_status(batch.status)


@pytest.mark.parametrize("window", [None, 5])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,page,q_lens,starts", KV_CASES)
def test_attention_generic(window, dtype, H, G, d, page, q_lens, starts):
    max_pages = 8 if page == 64 else 32
    batch, table, n_pages = make_batch(q_lens, starts, 9, page, max_pages, seed=3)
    T = batch.n_tokens
    kv = PagedKV(rnd(n_pages, G, page, d, dtype=dtype, seed=4), rnd(n_pages, G, page, d, dtype=dtype, seed=5), table, page)
    q = rnd(T, H, d, dtype=dtype, seed=6)
    out, ref = torch.empty(T, H * d, dtype=dtype, device=DEV), torch.empty(T, H * d, dtype=dtype, device=DEV)
    ops.attention(q, kv, batch, out, H, G, d, 1 / math.sqrt(d), window)
    REF.attention(q, kv, batch, ref, H, G, d, 1 / math.sqrt(d), window)
    ops.check_status(batch.status)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key(dtype):
    """One key far back is made to dominate: the output must be its value."""
    H, G, d, page = 4, 2, 32, 64
    batch, table, n_pages = make_batch([1], [700], 3, page, 12, seed=7)
    k = rnd(n_pages, G, page, d, dtype=dtype, scale=0.1, seed=8)
    v = rnd(n_pages, G, page, d, dtype=dtype, seed=9)
    q = rnd(1, H, d, dtype=dtype, scale=0.1, seed=10)
    slot = int(batch.slots[0])
    far = 3                                            # position 3 of 701
    pg = int(table[slot, far // page])
    q[0, :, 0] = 30.0
    k[pg, :, far % page, 0] = 30.0
    kv = PagedKV(k, v, table, page)
    out = torch.empty(1, H * d, dtype=dtype, device=DEV)
    ops.attention(q, kv, batch, out, H, G, d, 1.0, None)
    want = v[pg, :, far % page].repeat_interleave(H // G, dim=0).reshape(1, H * d)
    torch.testing.assert_close(out.float(), want.float(), rtol=1e-3, atol=1e-3)


def test_advance_lengths_and_add_into():
    batch, _, _ = make_batch([3, 1, 5], [4, 0, 9], 6, 64, 2)
    before = batch.lengths.clone()
    ops.advance_lengths(batch)
    want = before.clone()
    for s, q in zip(batch.slots.tolist(), [3, 1, 5]):
        want[s] += q
    assert torch.equal(batch.lengths, want)
    for dtype in DTYPES:
        x, y = rnd(7, 33), rnd(7, 33, dtype=dtype, seed=1)
        ref = x + y.float()
        ops.add_into(x, y)
        assert torch.equal(x, ref)


def test_embed_scale_and_logit_softcap():
    table = rnd(50, 72, dtype=torch.bfloat16)
    tokens = torch.randint(0, 50, (9,), dtype=torch.int32, device=DEV)
    out, ref = torch.empty(9, 72, device=DEV), torch.empty(9, 72, device=DEV)
    st = ops.new_status(DEV)
    ops.embed(tokens, table, out, st, 8.5)
    REF.embed(tokens, table, ref, st.clone(), 8.5)
    assert torch.equal(out, ref)                           # one 32-bit product of a widened value: exact
    ops.embed(tokens, table, out, st)
    assert torch.equal(out, table[tokens.long()].float())  # the default scale changes no bit
    x = rnd(7, 1001, scale=20.0)
    want = x.clone()
    ops.softcap(x, 30.0)
    REF.softcap(want, 30.0)
    torch.testing.assert_close(x, want, rtol=2e-6, atol=2e-6)
    assert float(x.abs().max()) <= 30.0
    with pytest.raises(ops.KernelError, match="positive"):
        ops.softcap(x, 0.0)


@pytest.mark.parametrize("B,V", [(1, 256), (5, 320), (3, 128256), (2, 1001)])
def test_argmax(B, V):
    logits = rnd(B, V)
    logits[0, V // 2] = logits[0, V - 1] = 50.0         # a tie: the lower index wins
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    assert int(out[0]) == V // 2
    assert out[1:].tolist() == torch.argmax(logits[1:], -1).tolist()


@pytest.mark.parametrize("B,V,top_k,temp", [(4, 320, 50, 0.8), (3, 1001, None, 1.0), (2, 128256, 200, 0.8),
                                            (2, 256, 1, 0.7), (2, 300, 5000, 1.3)])
def test_sample_matches_the_exponential_race(B, V, top_k, temp):
    logits = rnd(B, V, scale=2.0)
    req = torch.tensor([7, 1 << 40, 3, 9][:B], dtype=torch.int64, device=DEV)
    tix = torch.tensor([5, 0, 77, 1000, 12], dtype=torch.int32, device=DEV)
    imap = torch.tensor([4, 2, 0, 1][:B], dtype=torch.int32, device=DEV)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    noise = torch.empty(B, V, device=DEV)
    ops.sample(logits, out, temp, top_k, 1234, req, tix, imap, noise)
    ref = torch.empty(B, dtype=torch.int32)
    ref_noise = torch.empty(B, V)
    REF.sample(logits.cpu(), ref, temp, top_k, 1234, req.cpu(), tix.cpu(), imap.cpu(), ref_noise)
    torch.testing.assert_close(noise.cpu(), ref_noise, rtol=1e-5, atol=1e-6)
    assert out.cpu().tolist() == ref.tolist()
    if top_k == 1:
        assert out.cpu().tolist() == torch.argmax(logits, -1).cpu().tolist()


@pytest.mark.parametrize("V", [1001, 128256, 140000])
def test_sample_wide_and_narrow_rows_choose_alike_and_never_a_nan(V):
    """Rows wider than 131,072 take the one-block kernel, narrower ones the cluster kernel: from the same noise both
    must choose what the exponential race chooses, far-down logits included (scores in the log domain do not
    underflow), and an entry that is not a number never wins nor becomes the top-k pivot."""
    logits = rnd(3, V, scale=2.0, seed=4)
    logits[:, ::7] -= 150.0                                   # exp(x - max) of these underflows in 32-bit
    logits[0, 5] = logits[1, V - 1] = logits[2, 0] = float("nan")
    clean = torch.where(torch.isnan(logits), torch.full_like(logits, float("-inf")), logits)
    req = torch.tensor([11, 12, 1 << 33], dtype=torch.int64, device=DEV)
    for top_k in (None, 40, 3):
        out = torch.empty(3, dtype=torch.int32, device=DEV)
        ref = torch.empty(3, dtype=torch.int32)
        ops.sample(logits, out, 0.9, top_k, 77, req)
        REF.sample(clean.cpu(), ref, 0.9, top_k, 77, req.cpu())
        assert out.cpu().tolist() == ref.tolist(), f"top_k {top_k}"
        assert not torch.isnan(logits[torch.arange(3), out.long()]).any()
    # all but NaN and one finite entry: that entry is the answer whatever the noise
    lone = torch.full((1, V), float("nan"), device=DEV)
    lone[0, V // 3] = -3.0
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    ops.sample(lone, out, 1.0, 5, 1)
    assert int(out[0]) == V // 3


@pytest.mark.parametrize("kind", ["five-values", "two-humps", "heavy-tail", "mostly-masked", "constant"])
def test_sample_on_rows_that_are_far_from_normal(kind):
    """The sampler looks for the top-k entries above a threshold guessed from the row's mean and deviation; rows
    whose values are nothing like a normal sample must give the same token as the plain race, by the retries
    or by the radix select over the whole row."""
    V, B = 50000, 3
    g = torch.Generator().manual_seed(5)
    if kind == "five-values":                             # thousands of ties around the k-th value
        logits = torch.randint(0, 5, (B, V), generator=g).float()
    elif kind == "two-humps":
        logits = torch.randn(B, V, generator=g) + 30.0 * (torch.rand(B, V, generator=g) < 0.001).float()
    elif kind == "heavy-tail":
        logits = torch.randn(B, V, generator=g) * torch.exp(2.0 * torch.randn(B, V, generator=g))
    elif kind == "mostly-masked":                         # fewer finite entries than top_k
        logits = torch.full((B, V), float("-inf"))
        logits[:, :37] = torch.randn(B, 37, generator=g)
    else:
        logits = torch.full((B, V), 1.25)
    logits = logits.to(DEV)
    req = torch.tensor([3, 4, 5], dtype=torch.int64, device=DEV)
    for top_k in (1, 100, 2000):
        out = torch.empty(B, dtype=torch.int32, device=DEV)
        ref = torch.empty(B, dtype=torch.int32)
        ops.sample(logits, out, 0.7, top_k, 9, req)
        REF.sample(logits.cpu(), ref, 0.7, top_k, 9, req.cpu())
        assert out.cpu().tolist() == ref.tolist(), f"{kind}, top_k {top_k}"


def test_sample_keeps_ties_with_the_kth_value():
    V = 64
    logits = torch.full((1, V), -5.0, device=DEV)
    logits[0, [3, 9, 20]] = 2.0                          # three equal leaders, top_k = 2 keeps all three
    seen = set()
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    for seed in range(60):
        ops.sample(logits, out, 1.0, 2, seed)
        seen.add(int(out[0]))
    assert seen == {3, 9, 20}


def test_sample_frequencies_follow_softmax():
    V = 8
    logits = torch.tensor([[0.0, 1.0, 2.0, 0.5, -1.0, 0.0, 1.5, -2.0]], device=DEV).repeat(4000, 1)
    req = torch.arange(4000, dtype=torch.int64, device=DEV)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, 1.0, None, 99, req)
    freq = torch.bincount(out.long().cpu(), minlength=V).float() / 4000
    p = torch.softmax(logits[0].cpu(), -1)
    assert (freq - p).abs().max() < 0.03


# ---- tensor-core product (tcgen05 + TMA) -------------------------------------------------
TC_SHAPES = [(1, 384, 144), (8, 512, 256), (5, 320, 144), (16, 1024, 4096), (17, 6144, 512), (64, 768, 2048),
             (100, 1008, 200), (128, 256, 64), (129, 512, 1024), (300, 640, 456), (256, 2048, 4096), (1000, 4352, 512), (2048, 1024, 1024),
             # more 256 x 256 tiles than pairs of SMs, not a multiple of them, ragged rows and K
             (2048, 4096, 512), (600, 7680, 456), (300, 28672, 192), (2048, 6144, 1024)]


@pytest.mark.parametrize("mode", ["store", "store32", "add", "swiglu"])
@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_linear_tensor_core(mode, M, N, K):
    a = rnd(M, K, dtype=torch.bfloat16)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    k = ops.kernels()
    m = "store" if mode == "store32" else mode
    assert k._tc_fits(M, N, K, m)
    if mode == "add":
        out = rnd(M, N, seed=2)
        ref = out.clone()
    else:
        No = N // 2 if mode == "swiglu" else N
        out = torch.empty(M, No, dtype=torch.float32 if mode == "store32" else torch.bfloat16, device=DEV)
        ref = torch.empty_like(out)
    ops.linear(a, w, out, m)
    REF.linear(a, w, ref, m)
    ops.check_status(ops.new_status(DEV))
    if out.dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
    else:
        torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("swap,bn,splits,stages", [(1, 16, 1, 2), (1, 16, 3, 6), (1, 32, 2, 4), (1, 64, 5, 3), (1, 128, 1, 4),
                                                   (1, 128, 4, 3), (0, 128, 1, 3), (0, 128, 1, 6), (0, 256, 1, 4), (0, 256, 1, 3), (0, 512, 1, 4), (0, 512, 1, 2), (0, 1024, 1, 6), (0, 1024, 1, 3)])
@pytest.mark.parametrize("mode", ["store", "add", "swiglu"])
def test_tensor_core_plans(swap, bn, splits, stages, mode):
    """Every orientation, tile width, split and ring depth gives the same product."""
    M, N, K = (bn if swap else 150), 800, 1160
    M = min(M, 70) if bn >= 64 and swap else M
    a = rnd(M, K, dtype=torch.bfloat16)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    if mode == "add":
        out = rnd(M, N, seed=2)
        ref = out.clone()
    else:
        out = torch.empty(M, N // 2 if mode == "swiglu" else N, dtype=torch.bfloat16, device=DEV)
        ref = torch.empty_like(out)
    ops.kernels()._linear_tc(a, w, out, mode, plan=(swap, bn, splits, stages))
    REF.linear(a, w, ref, mode)
    ops.check_status(ops.new_status(DEV))
    if mode == "add":
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
    else:
        torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


# ---- bfloat16 attention over the paged cache ------------------------------------------------
BF16_ATTN_CASES = [  # H, G, d, q_lens, starts
    (4, 4, 16, [1, 1, 1], [4, 63, 64]),
    (6, 2, 24, [1, 1, 1, 1], [0, 6, 129, 700]),
    (32, 8, 128, [1, 1], [127, 1500]),
    (8, 1, 64, [1, 1, 1], [300, 65, 2]),
    (6, 2, 48, [5, 1, 70], [0, 200, 30]),          # also correct (if not fast) for longer runs of new tokens
    (5, 5, 256, [1, 3], [90, 10]),
]


@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("H,G,d,q_lens,starts", BF16_ATTN_CASES)
def test_attention_bf16_decode(splits, window, H, G, d, q_lens, starts):
    batch, table, n_pages = make_batch(q_lens, starts, 9, 64, 32, seed=3)
    T = batch.n_tokens
    dt = torch.bfloat16
    kv = PagedKV(rnd(n_pages, G, 64, d, dtype=dt, seed=4), rnd(n_pages, G, 64, d, dtype=dt, seed=5), table, 64)
    q = rnd(T, H, d, dtype=dt, seed=6)
    out, ref = torch.empty(T, H * d, dtype=dt, device=DEV), torch.empty(T, H * d, dtype=dt, device=DEV)
    ops.kernels()._attention_bf16(q, kv, batch, out, H, G, d, 1 / math.sqrt(d), window, splits=splits)
    REF.attention(q, kv, batch, ref, H, G, d, 1 / math.sqrt(d), window)
    ops.check_status(batch.status)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
