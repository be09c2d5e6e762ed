"""The model: an embedding, the layers a `ModelSpec` lists, run in the order of
its schedule, a final norm and the output product.

gpt-fast's `Transformer` (model.py:102-150) hard-wires one kind of block and
computes logits for every position; this one is built from the spec's parts,
runs a packed batch of sequences of unequal lengths against the paged cache
and computes logits only for the rows that are asked for.  It knows no
architecture: everything specific came in through the spec.
"""
from typing import Dict, Optional

import torch

from .. import ops
from ..cache import Cache, CacheNeeds
from ..config.spec import ModelSpec, PartSpec
from ..ops.types import BatchMeta
from ..parts.residual import Residual
from ..parts import NORMS, POSITIONS, build_block, build_part
from ..weights.loader import ParamSpec

COMPUTE_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def compute_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the model runs in bfloat16 or float32, not {dtype}")
        return dtype
    if dtype not in COMPUTE_DTYPES:
        raise ValueError(f"unknown dtype '{dtype}' (bfloat16 or float32)")
    return COMPUTE_DTYPES[dtype]


class Transformer:
    def __init__(self, spec: ModelSpec, dtype=torch.bfloat16, device="cuda"):
        spec.validate()
        self.spec = spec
        self.dtype = compute_dtype(dtype)
        self.device = torch.device(device)
        self.dim, self.vocab_size = spec.dim, spec.vocab_size

        positions = []                             # (PartSpec, object): one object per distinct spec

        def position_for(ps: Optional[PartSpec]):
            if ps is None:
                return None
            for known, obj in positions:
                if known is ps or known == ps:
                    return obj
            obj = build_part(POSITIONS, ps)
            positions.append((ps, obj))
            return obj

        self.blocks = [build_block(ls, spec.dim, self.dtype, position_for(ls.position)) for ls in spec.layers]
        self.positions = [obj for _, obj in positions]
        self.final_norm = build_part(NORMS, spec.final_norm, dtype=self.dtype)
        self.embed_weight = None
        self.head_weight = None

    # ---- parameters -------------------------------------------------------------
    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"embed.weight": ParamSpec((self.vocab_size, self.dim)),
                 "head.weight": ParamSpec((self.vocab_size, self.dim))}
        for name, s in self.final_norm.param_specs().items():
            specs[f"final_norm.{name}"] = s
        for i, b in enumerate(self.blocks):
            for pname, part in b.parts().items():
                for name, s in part.param_specs().items():
                    specs[f"layers.{i}.{pname}.{name}"] = s
        return specs

    def load_params(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand every part its tensors (as named by `param_specs`)."""
        want = self.param_specs()
        missing = sorted(set(want) - set(tensors))
        if missing:
            raise KeyError(f"model parameters without a tensor: {missing}")
        for name, s in want.items():
            if tuple(tensors[name].shape) != tuple(s.shape):
                raise ValueError(f"parameter {name}: expected shape {tuple(s.shape)}, got {tuple(tensors[name].shape)}")

        def sub(prefix):
            return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
        self.embed_weight = tensors["embed.weight"]
        self.head_weight = tensors["head.weight"]
        if self.spec.tie_embeddings and self.head_weight.data_ptr() != self.embed_weight.data_ptr():
            raise ValueError("the spec ties the output to the embedding, but two tensors were given")
        self.final_norm.load(sub("final_norm."))
        for i, b in enumerate(self.blocks):
            for pname, part in b.parts().items():
                part.load(sub(f"layers.{i}.{pname}."))

    def export_params(self) -> Dict[str, torch.Tensor]:
        """Every parameter under the name and in the layout of `param_specs` (the inverse of `load_params`);
        each part gives its own back through `export()`."""
        out = {"embed.weight": self.embed_weight, "head.weight": self.head_weight}
        for name, t in self.final_norm.export().items():
            out[f"final_norm.{name}"] = t
        for i, b in enumerate(self.blocks):
            for pname, part in b.parts().items():
                if not hasattr(part, "export"):
                    raise NotImplementedError(f"part '{pname}' of layer {i} ({type(part).__name__}) has no export()")
                for name, t in part.export().items():
                    out[f"layers.{i}.{pname}.{name}"] = t
        return out

    def graph_safe(self) -> bool:
        """Whether a step of this model may be captured in a CUDA graph: every part launches kernels only.  A part
        that reads device values on the host says so with `graph_safe = False`."""
        parts = [self.final_norm] + [p for b in self.blocks for p in b.parts().values()] + list(self.positions)
        return all(getattr(p, "graph_safe", True) for p in parts + list(self.blocks))

    def weight_bytes(self, with_embedding=False) -> int:
        """Bytes of the parameters a decode step streams (every matrix once)."""
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.head_weight)
        if with_embedding:
            add(self.embed_weight)
        for e in self.spec.schedule:
            for part in self.blocks[e.layer].parts().values():
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        add(v)
        for v in vars(self.final_norm).values():
            if isinstance(v, torch.Tensor):
                add(v)
        return total

    # ---- cache ---------------------------------------------------------------------
    def cache_needs(self) -> Dict[int, CacheNeeds]:
        needs = {}
        for e in self.spec.schedule:
            if e.owns_cache:
                needs[e.cache] = self.blocks[e.layer].cache_needs()
        return needs

    def new_cache(self, max_tokens: int, max_seqs: Optional[int] = None, max_seq_len: Optional[int] = None,
                  page_size: Optional[int] = None) -> Cache:
        limit = self.spec.max_position or None
        if max_seq_len is None:
            max_seq_len = limit
        elif limit and max_seq_len > limit:
            raise ValueError(f"max_seq_len {max_seq_len} exceeds the model's longest sequence {limit}")
        kw = {} if page_size is None else {"page_size": page_size}
        cache = Cache(self.cache_needs(), self.dtype, self.device, max_tokens=max_tokens, max_seqs=max_seqs,
                      max_seq_len=max_seq_len, **kw)
        for p in self.positions:
            p.prepare(cache.max_pages * cache.page_size, self.device)
        return cache

    def default_cache(self, max_tokens: int, max_seqs: int, max_seq_len: int) -> Cache:
        """The cache `generate` uses when none is given: kept between calls and replaced only when a
        call needs more tokens, sequences or length than it has (gpt-fast's setup_caches grows the
        same way, model.py:117-119)."""
        c = getattr(self, "_default_cache", None)
        if (c is None or c.n_pages * c.page_size < max_tokens or c.n_slots < max_seqs or c.max_seq_len < max_seq_len
                or c.slots.n_free != c.n_slots):
            self._default_cache = None            # let the old pools go before the new ones are made
            c = self.new_cache(max_tokens, max_seqs=max_seqs,
                               max_seq_len=min(max(max_seq_len, 1), self.spec.max_position or max_seq_len))
            self._default_cache = c
        return c

    # ---- one step ------------------------------------------------------------------------
    def forward(self, tokens: torch.Tensor, batch: BatchMeta, cache: Cache,
                want_rows: Optional[torch.Tensor], n_want: Optional[int] = None) -> torch.Tensor:
        """tokens int32 [T] (packed) -> float32 logits [W, V] at the packed rows
        `want_rows` (int32 [W]); None wants every row.  Appends this step's keys
        and values to the cache; the caller advances the lengths afterwards."""
        T = batch.n_tokens
        x = torch.empty(T, self.dim, dtype=torch.float32, device=self.device)
        ops.embed(tokens, self.embed_weight, x, batch.status, 1.0 if self.spec.embed_scale is None else float(self.spec.embed_scale))
        x = Residual(x)
        for e in self.spec.schedule:
            self.blocks[e.layer].forward(x, batch, cache.view(e.cache), append=e.owns_cache)
        W = T if want_rows is None else (n_want if n_want is not None else want_rows.shape[0])
        logits = torch.empty(W, self.vocab_size, dtype=torch.float32, device=self.device)
        if W:
            h = torch.empty(W, self.dim, dtype=self.dtype, device=self.device)
            self.final_norm.forward(x, h, want_rows)
            ops.linear(h, self.head_weight, logits)
            if self.spec.logit_cap is not None:
                ops.softcap(logits, float(self.spec.logit_cap))
        return logits
