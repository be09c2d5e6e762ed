"""The operations a model step is made of, each one a hand-written sm_100a
kernel (sources under `csrc/`).

Parts call the functions of this module; the functions check shapes and
types on the host, pick the kernel that fits (tensor-core kernels for aligned
bfloat16 shapes, the generic kernels otherwise and for 32-bit) and launch it
on the current CUDA stream.  There is no CPU or library fallback: if the
kernel libraries cannot be built or the tensors are not on a CUDA device, the
call raises.  `kernels()` returns the object that implements the operations;
tests may put a stand-in there with `use_kernels` to exercise the host-side
logic without a GPU.
"""
from contextlib import contextmanager
from typing import Optional

import torch

from .types import BatchMeta, PagedKV

STATUS_WORDS = 4
_STATUS_TEXT = {
    1: "token id out of range (token index {a}, id {b})",
    2: "position beyond the cache or the rotary table (token index {a}, position {b})",
    3: "a device-side wait ran out (wait {a}, block {b})",
    4: "page table has no page there (slot {a}, page index {b})",
}

_kernels = None


class KernelError(RuntimeError):
    pass


def kernels():
    global _kernels
    if _kernels is None:
        from .cuda import CudaKernels
        _kernels = CudaKernels()
    return _kernels


def use_kernels(obj):
    """Replace the kernel object (a test seam); returns the previous one."""
    global _kernels
    prev, _kernels = _kernels, obj
    return prev


@contextmanager
def trace():
    """Time every kernel launch made inside the block: yields a list that receives (label, start event,
    stop event) per launch; `trace_times` turns it into milliseconds.  The events sit between the
    launches, so kernels no longer overlap their neighbours: the times say where a step's work is, not
    how long the step takes in a CUDA graph.  Not for use under stream capture."""
    k = kernels()
    prev, k.trace = k.trace, []
    try:
        yield k.trace
    finally:
        k.trace = prev


def trace_times(records):
    """[(label, milliseconds)] of a finished trace, in launch order (synchronises)."""
    torch.cuda.synchronize()
    return [(label, start.elapsed_time(stop)) for label, start, stop in records]


def new_status(device) -> torch.Tensor:
    return torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor) -> None:
    """Read the device-side error words (this synchronises) and raise if a
    kernel reported something; the words are cleared afterwards."""
    own = getattr(_kernels, "_status", None)
    if own is not None and own is not status:
        check_status(own)
    s = status.tolist()
    if s[0] != 0:
        status.zero_()
        text = _STATUS_TEXT.get(s[0], "device error code {c}").format(a=s[1], b=s[2], c=s[0])
        raise KernelError(f"a kernel reported: {text}")


# ---- the operations ---------------------------------------------------------------

def embed(tokens, table, out, status, scale: float = 1.0):
    """out[t] = table[tokens[t]] * scale widened to 32-bit.  tokens int32 [T]; table
    [V, D]; out float32 [T, D]."""
    return kernels().embed(tokens, table, out, status, scale)


def softcap(x, cap: float):
    """x (float32, in place) = cap * tanh(x / cap)."""
    return kernels().softcap(x, cap)


def rmsnorm(x, weight, eps: float, out, rows=None, pending=None):
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight.  x float32
    [T, D]; weight [D] (bfloat16 or float32); out [R, D]; rows int32 [R] or None.
    pending (float32 [S, T, D], only without rows): partial sums still owed to x;
    the kernel first completes x += sum_s pending[s] (written back), then norms."""
    return kernels().rmsnorm(x, weight, eps, out, rows, pending)


def linear(a, w, out, mode: str = "store", defer: bool = False):
    """a [M, K] times w [N, K] transposed.  mode 'store': out [M, N] = product;
    'add': out float32 [M, N] += product (the residual sum, in 32-bit);
    'swiglu': w's rows alternate gate, up and out [M, N/2] = silu(gate) * up.

    defer=True (modes 'store' and 'add'): if the kernel splits the sum over K it
    may return the partial sums (float32 [S, M, N]) INSTEAD of finishing `out`;
    the caller hands them to the kernel that consumes the result (`rmsnorm`'s
    `pending`, `rope_append`'s `partials`, or `add_partials`).  Returns None when
    `out` is complete."""
    return kernels().linear(a, w, out, mode, defer)


def add_partials(x, pending):
    """x (float32 [T, D]) += sum_s pending[s] in ascending s."""
    return kernels().add_partials(x, pending)


def rope_table(inv_freq, table):
    """table[p, i] = (cos, sin)(p * inv_freq[i]) in 32-bit.  table float32 [P, d/2, 2]."""
    return kernels().rope_table(inv_freq, table)


def rope_append(qkv, q_out, kv: PagedKV, batch: BatchMeta, table, n_head: int, n_kv: int, head_dim: int,
                pairing: str = "interleaved", append: bool = True, partials=None):
    """Rotate the q and k heads of qkv [T, (H+2G)d] by each token's position;
    q goes to q_out [T, H, d]; k and v go to the token's place in the cache
    (unless append is False).  With partials (float32 [S, T, (H+2G)d], the
    deferred result of `linear`) qkv is their sum and the `qkv` argument is not read."""
    return kernels().rope_append(qkv, q_out, kv, batch, table, n_head, n_kv, head_dim, pairing, append, partials)


def attention(q, kv: PagedKV, batch: BatchMeta, out, n_head: int, n_kv: int, head_dim: int, scale: float,
              window: Optional[int] = None):
    """Causal grouped-query attention of q [T, H, d] over the cache (which
    already holds this step's keys and values); out [T, H*d]."""
    return kernels().attention(q, kv, batch, out, n_head, n_kv, head_dim, scale, window)


def rope_append_attention(qkv, partials, kv: PagedKV, batch: BatchMeta, table, out, n_head: int, n_kv: int, head_dim: int,
                          pairing: str, append: bool, scale: float, window: Optional[int] = None):
    """`rope_append` followed by `attention`: qkv [T, (H+2G)d] (or its deferred partial sums) -> out [T, H*d].
    Where a kernel does both in one launch (a decode step in bfloat16) that kernel runs; q then never goes
    through memory."""
    k = kernels()
    fused = getattr(k, "rope_append_attention", None)
    if fused is not None and fused(qkv, partials, kv, batch, table, out, n_head, n_kv, head_dim, pairing, append, scale, window):
        return
    q = torch.empty(batch.n_tokens, n_head, head_dim, dtype=out.dtype, device=out.device)
    k.rope_append(qkv, q, kv, batch, table, n_head, n_kv, head_dim, pairing, append, partials)
    k.attention(q, kv, batch, out, n_head, n_kv, head_dim, scale, window)


def advance_lengths(batch: BatchMeta):
    """lengths[slot] += number of new tokens, for every sequence of the batch."""
    return kernels().advance_lengths(batch)


def add_into(out, y):
    """out (float32) += y."""
    return kernels().add_into(out, y)


def argmax(logits, out):
    """out[b] = index of the largest logits[b, :], lowest index on ties."""
    return kernels().argmax(logits, out)


def sample(logits, out, temperature: float, top_k: Optional[int], seed: int, request_ids=None, token_index=None,
           index_map=None, noise_out=None, seed_dev=None):
    """Temperature / top-k / exponential-race draw per row of float32 logits.
    The noise of row b is keyed by (seed, request_ids[b], token_index[index_map[b]
    or b], vocabulary index), so it does not depend on the row's place in the batch.
    seed_dev (int64 [1] on the device) overrides `seed`: a captured graph can then be replayed with another seed."""
    return kernels().sample(logits, out, temperature, top_k, seed, request_ids, token_index, index_map, noise_out, seed_dev)
