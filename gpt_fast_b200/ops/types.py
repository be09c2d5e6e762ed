"""What a step hands to the kernels: the batch's bookkeeping and a view of one
cache entry.  Plain data, device tensors plus the host-side bounds that size
the launches."""
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class BatchMeta:
    """n sequences with T packed tokens.  Token t belongs to sequence
    tok_seq[t]; sequence s owns tokens cu_seqlens[s]..cu_seqlens[s+1]-1 and
    cache slot slots[s]; lengths[slot] tokens were cached before this step, so
    token t sits at position lengths[slot] + (t - cu_seqlens[s])."""
    cu_seqlens: torch.Tensor      # int32 [n+1]
    tok_seq: torch.Tensor         # int32 [T]
    slots: torch.Tensor           # int32 [n]
    lengths: torch.Tensor         # int32 [n_slots], owned by the cache
    n_seqs: int
    n_tokens: int
    max_q_len: int                # host bound: longest run of new tokens
    max_kv_len: int               # host bound: longest sequence after this step
    status: torch.Tensor          # int32 [4], device-side error words


@dataclass
class PagedKV:
    """Keys and values of one cache entry: pools of pages [n_pages, n_kv,
    page_size, head_dim]; page_table[slot, i] is the page that holds the
    slot's positions i*page_size .. (i+1)*page_size-1."""
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    page_table: torch.Tensor      # int32 [n_slots, max_pages]
    page_size: int
    workspace: Optional[object] = None   # scratch of the split-KV decode kernel
