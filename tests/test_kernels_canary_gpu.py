"""Nothing is written outside an output: every kernel's outputs lie between guard words that must still hold their
pattern afterwards, at sizes with ragged last tiles, rows and pages.  (A memory checker that stops the process is
not used on the shared GPUs of this project; kernels report bad ids, positions and pages through status words, and
this file is the check for the other kind of fault, a stray store.)"""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.ops.types import PagedKV
from test_kernels_gpu import DEV, make_batch, rnd

pytestmark = pytest.mark.gpu
GUARD = 256                                   # elements before and after; a multiple of 16 bytes for every dtype used


class Guarded:
    """A tensor of `shape` in the middle of a larger buffer whose ends hold a pattern."""

    def __init__(self, *shape, dtype=torch.float32, fill=None):
        n = math.prod(shape)
        self.pattern = 12345 if dtype in (torch.int32, torch.int64) else -7777.0
        self.buf = torch.full((n + 2 * GUARD,), self.pattern, dtype=dtype, device=DEV)
        self.t = self.buf[GUARD:GUARD + n].view(*shape)
        if fill is not None:
            self.t.copy_(fill)

    def check(self, what):
        head, tail = self.buf[:GUARD], self.buf[-GUARD:]
        assert bool((head == self.pattern).all()), f"{what}: a store in front of the output"
        assert bool((tail == self.pattern).all()), f"{what}: a store behind the output"
        assert not bool((self.t == self.pattern).all()), f"{what}: the output was never written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_kernels_stay_inside_their_outputs(dtype):
    T, D, V = 13, 200, 97
    table = rnd(V, D, dtype=dtype)
    tokens = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    x = Guarded(T, D)
    ops.embed(tokens, table, x.t, ops.new_status(DEV))
    x.check("embed")
    pending = rnd(3, T, D, seed=1)
    h = Guarded(T, D, dtype=dtype)
    ops.rmsnorm(x.t, 1 + 0.1 * rnd(D, seed=2), 1e-5, h.t, None, pending)
    x.check("rmsnorm (the residual it completes)")
    h.check("rmsnorm")
    rows = torch.tensor([T - 1, 0, 5], dtype=torch.int32, device=DEV)
    g = Guarded(3, D, dtype=dtype)
    ops.rmsnorm(x.t, 1 + 0.1 * rnd(D, seed=2), 1e-5, g.t, rows)
    g.check("rmsnorm with a row gather")
    y = Guarded(T, D, fill=rnd(T, D, seed=3))
    ops.add_into(y.t, rnd(T, D, dtype=dtype, seed=4))
    y.check("add_into")
    ops.add_partials(y.t, pending)
    y.check("add_partials")


@pytest.mark.parametrize("M,N,K", [(1, 264, 200), (7, 1000, 456), (40, 904, 776), (100, 136, 72), (129, 520, 264),
                                   (300, 776, 520), (513, 264, 1032)])
def test_products_stay_inside_their_outputs(M, N, K):
    a = rnd(M, K, dtype=torch.bfloat16)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    for mode in ("store", "add", "swiglu"):
        if mode == "swiglu" and N % 16:
            continue
        out = Guarded(M, N // 2 if mode == "swiglu" else N, dtype=torch.float32 if mode == "add" else torch.bfloat16,
                      fill=0.0)
        pending = ops.linear(a, w, out.t, mode, defer=mode == "add")
        if pending is not None:                      # a sum split over K, left to the caller: finish it
            ops.add_partials(out.t, pending)
        ops.check_status(ops.new_status(DEV))
        out.check(f"tensor-core product {mode}")
    # the 32-bit product on CUDA cores, sizes that are multiples of nothing
    a32, w32 = rnd(M, K - 3), rnd(N - 5, K - 3, scale=0.05, seed=1)
    out = Guarded(M, N - 5)
    ops.linear(a32, w32, out.t, "store")
    out.check("32-bit product")


@pytest.mark.parametrize("dtype,H,G,d", [(torch.float32, 6, 2, 24), (torch.bfloat16, 6, 2, 24), (torch.bfloat16, 8, 2, 128),
                                         (torch.bfloat16, 6, 2, 64)])
def test_attention_kernels_stay_inside_their_outputs_and_pages(dtype, H, G, d):
    for q_lens, starts in (([1, 1, 1], [130, 63, 0]), ([45, 3, 129], [5, 64, 100])):
        batch, table, n_pages = make_batch(q_lens, starts, 5, 64, 8, seed=3)
        T, W = batch.n_tokens, (H + 2 * G) * d
        kp = Guarded(n_pages, G, 64, d, dtype=dtype, fill=rnd(n_pages, G, 64, d, dtype=dtype, seed=4))
        vp = Guarded(n_pages, G, 64, d, dtype=dtype, fill=rnd(n_pages, G, 64, d, dtype=dtype, seed=5))
        kv = PagedKV(kp.t, vp.t, table, 64)
        rt = torch.empty(8 * 64, d // 2, 2, device=DEV)
        ops.rope_table((1.0 / (10000 ** (torch.arange(d // 2).float() * 2 / d))).to(DEV), rt)
        qkv = rnd(T, W, dtype=dtype, seed=6)
        out = Guarded(T, H * d, dtype=dtype)
        before_k = kp.t.clone()
        ops.rope_append_attention(qkv, None, kv, batch, rt, out.t, H, G, d, "interleaved", True, 1 / math.sqrt(d), None)
        ops.check_status(batch.status)
        what = f"rotary + append + attention, {q_lens}"
        out.check(what)
        kp.check(what + " (key pool)")
        vp.check(what + " (value pool)")
        # only the new tokens' places in the pools changed: T rows of G heads
        changed = (kp.t != before_k).any(dim=-1)
        assert int(changed.sum()) <= T * G


def test_sampling_stays_inside_its_output():
    for B, V, top_k in ((3, 1001, 50), (5, 128256, 200), (2, 140000, None), (4, 320, 0)):
        logits = rnd(B, V, scale=2.0, seed=B)
        out = Guarded(B, dtype=torch.int32)
        ops.sample(logits, out.t, 0.8, top_k, 7)
        out.check(f"sample V={V} top_k={top_k}")
        out = Guarded(B, dtype=torch.int32)
        ops.argmax(logits, out.t)
        out.check(f"argmax V={V}")
