"""ctypes bindings of the kernel libraries: host-side checks, kernel choice,
launch on the current stream."""
import ctypes
from ctypes import c_float, c_int, c_long, c_ulonglong, c_void_p
from typing import Optional

import torch

from ..csrc import build
from .types import BatchMeta, PagedKV

_DT = {torch.float32: 0, torch.bfloat16: 1}
_EPI = {"store": 0, "add": 1, "swiglu": 2}
_PAIRING = {"interleaved": 0, "half": 1}


def _fail(msg):
    from . import KernelError
    raise KernelError(msg)


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        _fail(f"kernels take float32 or bfloat16, got {t.dtype}")
    return _DT[t.dtype]


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, dtype=None, shape=None, name="tensor"):
    if not t.is_cuda:
        _fail(f"{name} is on {t.device}: the kernels of this library run on a CUDA device only")
    if not t.is_contiguous():
        _fail(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        _fail(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        _fail(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream of the current device as a handle for the kernels.  Asked for at every launch (a capture
    runs on a stream of its own); the short way through torch's C module costs a tenth of `current_stream()`."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def decode_slices(max_kv_len: int, page_size: int, blocks: int, sm_count: int) -> int:
    """Into how many slices a decode step cuts each sequence's cache (`blocks` = tokens x key/value heads, the
    blocks of one slice).  A simple cost model fitted to measurements on a B200 (contexts of 600 to 32,000,
    batches of 1 to 64): two blocks fit on an SM, so blocks * slices run in ceil(blocks * slices / (2 SMs))
    rounds; a round costs the pages of a slice plus about four pages' worth of fixed work per block; a slice
    keeps at least 4 pages.  The cheapest count wins, the smaller one on ties."""
    pages = -(-max(max_kv_len, 1) // page_size)
    cap = 2 * sm_count
    best, best_cost = 1, None
    for s in range(1, max(1, min(pages // 4, 48)) + 1):
        cost = -(-blocks * s // cap) * (pages / s + 4.0)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


class CudaKernels:
    """The operations of `ops`, bound to the sm_100a libraries.  A library is
    compiled and loaded when its first function is needed."""

    def __init__(self):
        if not torch.cuda.is_available():
            _fail("no CUDA device: this library has no CPU path")
        self._fn = {}
        self._sm_count = None
        self._status = None
        self.trace = None                  # a list: (label, start event, stop event) of every launch is appended
        self._label = None                 # what the next launch is called in the trace (default: the entry point)

    def _f(self, lib: str, name: str):
        key = (lib, name)
        fn = self._fn.get(key)
        if fn is None:
            handle = build.library(lib)
            fn = getattr(handle, name)
            fn.restype = c_int
            self._fn[key] = fn
            fn._lib = handle
        return fn

    def _call(self, lib, name, *args):
        fn = self._f(lib, name)
        trace = self.trace
        if trace is not None:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        rc = fn(*args)
        if trace is not None:
            stop.record()
            trace.append((self._label or name, start, stop))
        self._label = None
        if rc != 0:
            _fail(f"{name}: {fn._lib.gfb_last_error().decode()}")

    # -- element-wise / per-row -------------------------------------------------
    def embed(self, tokens, table, out, status, scale=1.0):
        T = tokens.shape[0]
        V, D = table.shape
        _need(tokens, torch.int32, name="tokens")
        _need(table, name="embedding table")
        _need(out, torch.float32, (T, D), "embedding output")
        self._call("core", "gfb_embed", _ptr(tokens), _ptr(table), c_int(_dt(table)), _ptr(out),
                   c_int(T), c_int(D), c_int(V), c_float(scale), _ptr(status), _stream())

    def softcap(self, x, cap):
        _need(x, torch.float32, name="logits")
        self._call("core", "gfb_softcap", _ptr(x), c_long(x.numel()), c_float(cap), _stream())

    def rmsnorm(self, x, weight, eps, out, rows=None, pending=None):
        D = x.shape[-1]
        R = out.shape[0]
        _need(x, torch.float32, name="norm input")
        _need(weight, shape=(D,), name="norm weight")
        _need(out, shape=(R, D), name="norm output")
        if rows is not None:
            _need(rows, torch.int32, (R,), "rows")
            if pending is not None:
                self.add_partials(x, pending)
                pending = None
        elif x.shape[0] != R:
            _fail(f"norm output has {R} rows, input {x.shape[0]}")
        S = 0
        if pending is not None:
            S = pending.shape[0]
            _need(pending, torch.float32, (S,) + tuple(x.shape), "pending partial sums")
        self._call("core", "gfb_rmsnorm", _ptr(x), _ptr(pending), c_int(S), c_long(x.numel()), _ptr(weight),
                   c_int(_dt(weight)), _ptr(out), c_int(_dt(out)), _ptr(rows), c_int(R), c_int(D), c_float(eps), _stream())

    def add_partials(self, x, pending):
        _need(x, torch.float32, name="sum")
        _need(pending, torch.float32, (pending.shape[0],) + tuple(x.shape), "pending partial sums")
        self._call("core", "gfb_add_partials", _ptr(x), _ptr(pending), c_int(pending.shape[0]), c_long(x.numel()), _stream())

    def rope_table(self, inv_freq, table):
        P, half, two = table.shape
        _need(inv_freq, torch.float32, (half,), "inv_freq")
        _need(table, torch.float32, name="rotary table")
        self._call("core", "gfb_rope_table", _ptr(inv_freq), _ptr(table), c_int(P), c_int(half), _stream())

    def _batch_args(self, b: BatchMeta):
        return (_ptr(b.cu_seqlens), _ptr(b.tok_seq), _ptr(b.slots), _ptr(b.lengths), c_int(b.n_seqs), c_int(b.n_tokens))

    def _kv_args(self, kv: PagedKV):
        return (_ptr(kv.k_pool), _ptr(kv.v_pool), _ptr(kv.page_table), c_int(kv.page_table.shape[1]),
                c_int(kv.page_size), c_int(kv.k_pool.shape[0]))

    def rope_append(self, qkv, q_out, kv, batch, table, n_head, n_kv, head_dim, pairing, append, partials=None):
        T = batch.n_tokens
        W = (n_head + 2 * n_kv) * head_dim
        if partials is not None:
            _need(partials, torch.float32, (partials.shape[0], T, W), "partial sums of qkv")
            src, n_part = partials, partials.shape[0]
        else:
            _need(qkv, shape=(T, W), name="qkv")
            src, n_part = qkv, 0
        _need(q_out, shape=(T, n_head, head_dim), name="q_out")
        qkv = q_out                                     # the element type of the outputs
        _need(table, torch.float32, name="rotary table")
        if append:
            _need(kv.k_pool, qkv.dtype, name="key pool")
            if tuple(kv.k_pool.shape[1:]) != (n_kv, kv.page_size, head_dim):
                _fail(f"key pool pages are {tuple(kv.k_pool.shape[1:])}, the layer needs {(n_kv, kv.page_size, head_dim)}")
        self._call("core", "gfb_rope_append", _ptr(src), c_int(n_part), _ptr(q_out), c_int(_dt(q_out)), *self._kv_args(kv),
                   *self._batch_args(batch), _ptr(table), c_int(table.shape[0]), c_int(n_head), c_int(n_kv),
                   c_int(head_dim), c_int(_PAIRING[pairing]), c_int(1 if append else 0), _ptr(batch.status), _stream())

    def advance_lengths(self, batch):
        self._call("core", "gfb_advance_lengths", _ptr(batch.lengths), _ptr(batch.slots), _ptr(batch.cu_seqlens),
                   c_int(batch.n_seqs), _stream())

    def add_into(self, out, y):
        _need(out, torch.float32, name="sum")
        _need(y, shape=out.shape, name="addend")
        self._call("core", "gfb_add_into", _ptr(out), _ptr(y), c_int(_dt(y)), c_long(out.numel()), _stream())

    # -- matrix products -----------------------------------------------------------
    def linear(self, a, w, out, mode="store", defer=False):
        M, K = a.shape
        N = w.shape[0]
        _need(a, name="activation")
        _need(w, a.dtype, (N, K), "weight")
        No = N // 2 if mode == "swiglu" else N
        _need(out, shape=(M, No), name="product output")
        if mode == "add" and out.dtype != torch.float32:
            _fail("the residual sum is kept in float32")
        if mode != "add" and out.dtype not in (a.dtype, torch.float32):
            _fail(f"product of {a.dtype} cannot be stored as {out.dtype}")
        self._label = f"linear {N}x{K} {mode}"
        if a.dtype == torch.bfloat16 and self._tc_fits(M, N, K, mode):
            return self._linear_tc(a, w, out, mode, defer=defer and mode in ("store", "add"))
        if a.dtype == torch.float32 and out.dtype != torch.float32:
            _fail("a float32 product is stored as float32")
        self._call("gemm_simt", "gfb_gemm_simt", _ptr(a), _ptr(w), _ptr(out), c_int(_dt(a)), c_int(_dt(out)),
                   c_int(M), c_int(N), c_int(K), c_int(_EPI[mode]), _stream())

    def _tc_fits(self, M, N, K, mode) -> bool:
        """The tensor-core kernel takes rows of whole 16-byte units (TMA) and stores in 16-byte vectors."""
        return K % 8 == 0 and N % (16 if mode == "swiglu" else 8) == 0

    def tc_plan(self, M, N, K, mode="store"):
        """(swap, bn, splits, stages) for the tensor-core product.  Few tokens: the weight rows fill the
        128 MMA rows and the tokens are its columns, split over K until about two blocks per SM stream
        weights; many tokens: 256 x 256 tiles on pairs of SMs (bn = 1024 names that kernel, 512 the
        one-SM persistent kernel, 128/256 one tile per block).  In between (129 to 512 tokens) a product
        that may be split over K stays in the first form, with several column tiles of 128 tokens: one or two
        row tiles of 256 x 256 leave most pairs of SMs idle unless the weight matrix is wide (measured at 256
        tokens: q/k/v 26.8 -> 15.5 us, output projection 29.4 -> 12.8, down projection 78.1 -> 31.8; the
        gate/up product with its SwiGLU cannot be split and is wide enough: 57 us on pairs, 78 us this way; so is
        the output product: 224 us on pairs, 383 us this way, hence the count of 256 x 256 tiles in the rule)."""
        if 128 < M <= 512 and mode != "swiglu" and -(-M // 256) * -(-N // 256) < self.sm_count // 2:
            blocks = -(-N // 128) * -(-M // 128)
            total_kb = -(-K // 64)
            splits = max(1, min(total_kb // 8, (2 * self.sm_count) // blocks))
            return 1, 128, splits, 3
        if M <= 128:
            bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
            blocks = -(-N // 128)
            total_kb = -(-K // 64)
            splits = max(1, min(total_kb // 8, (2 * self.sm_count) // blocks))
            stage = 16384 + bn * 128
            stages = max(2, min(8, (100 * 1024) // stage))
            if blocks > 4 * self.sm_count:
                stages = 3          # many rounds of blocks (the output product): four short rings per SM stream better than two long ones
            return 1, bn, splits, stages
        if N >= 256:
            # pairs of SMs on 256 x 256 tiles (bn 1024 = the cta_group::2 kernel), persistent, two
            # accumulators in tensor memory so that a tile's epilogue hides behind the next main loop
            return 0, 1024, 1, 6
        return 0, 128, 1, 6

    @property
    def sm_count(self):
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        return self._sm_count

    @property
    def status(self):
        """Error words of kernels that take no status of a step (bounded waits that ran out)."""
        if self._status is None:
            self._status = torch.zeros(4, dtype=torch.int32, device="cuda")
        return self._status

    def _linear_tc(self, a, w, out, mode, plan=None, defer=False):
        M, K = a.shape
        N = w.shape[0]
        swap, bn, splits, stages = plan or self.tc_plan(M, N, K, mode)
        ws = torch.empty(splits, M, N, dtype=torch.float32, device=a.device) if splits > 1 else None
        used = c_int(1)
        self._call("gemm_tc", "gfb_gemm_tc", _ptr(a), _ptr(w), _ptr(out), c_int(_dt(out)), c_int(M), c_int(N), c_int(K),
                   c_int(_EPI[mode]), c_int(swap), c_int(bn), c_int(splits), c_int(stages), _ptr(ws),
                   c_int(0 if defer else 1), ctypes.byref(used), _ptr(self.status), _stream())
        if defer and used.value > 1:
            return ws[:used.value]
        return None

    # -- attention ---------------------------------------------------------------------
    def attention(self, q, kv, batch, out, n_head, n_kv, head_dim, scale, window=None):
        T = batch.n_tokens
        _need(q, shape=(T, n_head, head_dim), name="q")
        _need(out, q.dtype, (T, n_head * head_dim), "attention output")
        _need(kv.k_pool, q.dtype, name="key pool")
        if (q.dtype == torch.bfloat16 and kv.page_size == 64 and head_dim % 8 == 0 and head_dim <= 256
                and n_head // n_kv <= 8):
            return self._attention_bf16(q, kv, batch, out, n_head, n_kv, head_dim, scale, window)
        self._call("attention_generic", "gfb_attention_generic", _ptr(q), _ptr(out), c_int(_dt(q)),
                   *self._kv_args(kv), *self._batch_args(batch), c_int(n_head), c_int(n_kv), c_int(head_dim),
                   c_float(scale), c_int(window or 0), _ptr(batch.status), _stream())

    def decode_slices(self, max_kv_len, page_size, blocks) -> int:
        return decode_slices(max_kv_len, page_size, blocks, self.sm_count)

    def _attention_bf16(self, q, kv, batch, out, n_head, n_kv, head_dim, scale, window, splits=None, prefill=None, tiles=0,
                        max_blocks=0):
        T = batch.n_tokens
        if prefill is None:
            prefill = splits is None and batch.max_q_len > 1 and head_dim in (64, 128)
        if prefill and head_dim in (64, 128) and n_head // n_kv <= 8:
            self._call("attention_tc", "gfb_attn_prefill_tc", _ptr(q), _ptr(out), *self._kv_args(kv), *self._batch_args(batch),
                       c_int(n_head), c_int(n_kv), c_int(head_dim), c_float(scale), c_int(window or 0), c_int(tiles),
                       c_int(max_blocks), _ptr(batch.status), _stream())
            return
        if splits is None:
            splits = 1
            if batch.max_q_len == 1:
                splits = self.decode_slices(batch.max_kv_len, kv.page_size, T * n_kv)
        scratch = None
        if splits > 1:
            scratch = torch.empty(T * n_head * splits * (head_dim + 2), dtype=torch.float32, device=q.device)
        self._call("attention_bf16", "gfb_attn_decode", _ptr(q), _ptr(out), *self._kv_args(kv), *self._batch_args(batch),
                   c_int(n_head), c_int(n_kv), c_int(head_dim), c_float(scale), c_int(window or 0), c_int(splits),
                   _ptr(scratch), _ptr(batch.status), _stream())

    def rope_append_attention(self, qkv, partials, kv, batch, table, out, n_head, n_kv, head_dim, pairing, append,
                              scale, window=None, lengths_early=None) -> bool:
        """Rotary encoding, cache append and attention of a decode step in one launch, where the kernel for
        it fits (bfloat16, one token per sequence, head_dim 64 or 128, pages of 64, at most 8 query heads per
        key/value head).  Returns False, having done nothing, where it does not.  lengths_early (tests only):
        what the kernel's read of the lengths ahead of its dependency wait is to see."""
        T = batch.n_tokens
        if not (out.dtype == torch.bfloat16 and batch.max_q_len == 1 and head_dim in (64, 128) and kv.page_size == 64
                and n_head // n_kv <= 8):
            return False
        W = (n_head + 2 * n_kv) * head_dim
        if partials is not None:
            _need(partials, torch.float32, (partials.shape[0], T, W), "partial sums of qkv")
            src, n_part = partials, partials.shape[0]
        else:
            _need(qkv, torch.bfloat16, (T, W), "qkv")
            src, n_part = qkv, 0
        _need(out, torch.bfloat16, (T, n_head * head_dim), "attention output")
        _need(table, torch.float32, name="rotary table")
        _need(kv.k_pool, torch.bfloat16, name="key pool")
        if tuple(kv.k_pool.shape[1:]) != (n_kv, kv.page_size, head_dim):
            _fail(f"key pool pages are {tuple(kv.k_pool.shape[1:])}, the layer needs {(n_kv, kv.page_size, head_dim)}")
        splits = self.decode_slices(batch.max_kv_len, kv.page_size, T * n_kv)
        scratch = None
        if splits > 1:
            scratch = torch.empty(T * n_head * splits * (head_dim + 2), dtype=torch.float32, device=out.device)
        self._call("attention_bf16", "gfb_attn_decode_rope", _ptr(src), c_int(n_part), _ptr(out), *self._kv_args(kv),
                   *self._batch_args(batch), _ptr(table), c_int(table.shape[0]), c_int(n_head), c_int(n_kv), c_int(head_dim),
                   c_int(_PAIRING[pairing]), c_int(1 if append else 0), c_float(scale), c_int(window or 0), c_int(splits),
                   _ptr(scratch), _ptr(batch.status), _ptr(lengths_early), c_int(int(batch.max_kv_len)), _stream())
        return True

    # -- sampling --------------------------------------------------------------------------
    def argmax(self, logits, out):
        B, V = logits.shape
        _need(logits, torch.float32, name="logits")
        _need(out, torch.int32, (B,), "token output")
        self._call("sampling", "gfb_argmax", _ptr(logits), _ptr(out), c_int(B), c_int(V), _stream())

    def sample(self, logits, out, temperature, top_k, seed, request_ids=None, token_index=None, index_map=None,
               noise_out=None, seed_dev=None):
        B, V = logits.shape
        _need(logits, torch.float32, name="logits")
        _need(out, torch.int32, (B,), "token output")
        if request_ids is not None:
            _need(request_ids, torch.int64, (B,), "request ids")
        if token_index is not None:
            _need(token_index, torch.int32, name="token index")
        if index_map is not None:
            _need(index_map, torch.int32, (B,), "index map")
        elif token_index is not None and token_index.shape[0] < B:
            _fail("token index has fewer entries than logits has rows")
        if noise_out is not None:
            _need(noise_out, torch.float32, (B, V), "noise output")
        self._call("sampling", "gfb_sample", _ptr(logits), _ptr(out), c_int(B), c_int(V), c_float(temperature),
                   c_int(int(top_k) if top_k else 0), c_ulonglong(seed & (2 ** 64 - 1)), _ptr(seed_dev), _ptr(request_ids),
                   _ptr(token_index), _ptr(index_map), _ptr(noise_out), _stream())
