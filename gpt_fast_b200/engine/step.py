"""The step function: a batch of sequences that started together, each with
its own length, moves on by the tokens it is given.

gpt-fast's forward takes `idx [B, S]` and ONE position vector for all rows
(model.py:136-146, generate.py:178-185), so all rows have the same length.
Here a step takes, per sequence, its slot and its next tokens (any number:
whole prompts in the first step, one token each afterwards), runs exactly
those tokens as one packed batch against the cache, and returns float32
logits at the places asked for.  Nothing is padded, so nothing depends on
padding.

`Stepper.step` is the general entry (host lists in, bookkeeping uploaded once
per step).  `Stepper.decode_batch` prepares the fixed-shape one-token-each
step whose kernel sequence is captured in a CUDA graph and replayed without
host work; generation and the benchmark use it.
"""
import gc
from typing import Sequence, Union

import torch

from .. import ops
from ..cache import Cache
from ..ops.types import BatchMeta
from .model import Transformer

Want = Union[str, Sequence[Sequence[int]]]


class Stepper:
    def __init__(self, model: Transformer, cache: Cache):
        self.model, self.cache = model, cache
        self.device = model.device
        self.status = ops.new_status(self.device)
        self._pin = self.device.type == "cuda"
        self._decode_batches = {}

    @classmethod
    def of(cls, model: Transformer, cache: Cache) -> "Stepper":
        """The stepper that belongs to `cache` (made on first use): it keeps the decode graphs that
        were captured for this cache, so that later calls replay them instead of capturing again."""
        st = getattr(cache, "_stepper", None)
        if st is None or st.model is not model:
            st = cls(model, cache)
            cache._stepper = st
        return st

    # ---- general step ----------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], want: Want = "last") -> torch.Tensor:
        """Advance sequence i (in cache slot slots[i]) by tokens[i].

        want: 'last' (the last new token of each sequence), 'all', 'none', or per
        sequence a list of places among ITS new tokens.  Returns float32 logits
        [number of wanted places, vocab], ordered by sequence, then by place."""
        n = len(slots)
        if n == 0 or len(tokens) != n:
            raise ValueError("a step needs one token list per slot, and at least one sequence")
        if len(set(slots)) != n:
            raise ValueError(f"a slot appears twice in one step: {list(slots)}")
        q_lens = [len(t) for t in tokens]
        if min(q_lens) < 1:
            raise ValueError("every sequence of a step brings at least one token")
        cache = self.cache
        for s, q in zip(slots, q_lens):
            cache.reserve(s, cache.lengths_host[s] + q)
        cache.sync_tables()

        cu = [0]
        for q in q_lens:
            cu.append(cu[-1] + q)
        T = cu[-1]
        if want == "last":
            rows = [cu[i + 1] - 1 for i in range(n)]
        elif want == "all":
            rows = list(range(T))
        elif want == "none":
            rows = []
        else:
            if len(want) != n:
                raise ValueError("`want` needs one list of places per sequence")
            rows = []
            for i, places in enumerate(want):
                for p in places:
                    if not 0 <= p < q_lens[i]:
                        raise ValueError(f"sequence {i} brings {q_lens[i]} tokens; place {p} is not among them")
                    rows.append(cu[i] + p)
        tok_seq = [i for i, q in enumerate(q_lens) for _ in range(q)]
        flat = [int(t) for seq in tokens for t in seq]
        packed = torch.tensor(cu + tok_seq + list(slots) + rows + flat, dtype=torch.int32)
        if self._pin:
            packed = packed.pin_memory()
        dev = packed.to(self.device, non_blocking=True)
        o = 0
        cu_d = dev[o:o + n + 1]; o += n + 1
        seq_d = dev[o:o + T]; o += T
        slots_d = dev[o:o + n]; o += n
        rows_d = dev[o:o + len(rows)]; o += len(rows)
        tok_d = dev[o:o + T]
        batch = BatchMeta(cu_seqlens=cu_d, tok_seq=seq_d, slots=slots_d, lengths=cache.lengths, n_seqs=n, n_tokens=T,
                          max_q_len=max(q_lens),
                          max_kv_len=max(cache.lengths_host[s] + q for s, q in zip(slots, q_lens)),
                          status=self.status)
        logits = self.model.forward(tok_d, batch, cache, rows_d, len(rows))
        ops.advance_lengths(batch)
        cache.note_advance(slots, q_lens)
        return logits

    def check(self) -> None:
        """Raise if a kernel of an earlier step reported an error (synchronises)."""
        ops.check_status(self.status)

    # ---- fixed-shape decode ----------------------------------------------------------------
    def decode_batch(self, slots: Sequence[int], use_graph: bool = True, sampling=None, request_ids=None) -> "DecodeBatch":
        """The fixed-shape decode step for these slots.  With `sampling` (a SamplingParams) the step
        also draws the next tokens.  A batch made earlier for the same slots and the same sampling
        constants is handed out again, with its captured graph; request ids and seed are rewritten."""
        if sampling is None:
            return DecodeBatch(self, slots, use_graph)
        from .generate import _Sampler
        # the number of slices the attention cuts a sequence into is fixed when the step is captured, from the
        # longest reservation among the slots: a batch captured for short sequences would run long ones in
        # one slice (right, but slow), so the reservation's power-of-two bracket is part of the key
        reach = max(self.cache.reserved_host[s] for s in slots)
        key = (tuple(slots), bool(use_graph), sampling.temperature, sampling.top_k, max(reach, 1).bit_length())
        batch = self._decode_batches.get(key)
        if batch is None:
            if len(self._decode_batches) >= 64:
                self._decode_batches.clear()
            batch = DecodeBatch(self, slots, use_graph, _Sampler(sampling, request_ids, self.device))
            self._decode_batches[key] = batch
        else:
            batch.sampler.retarget(sampling, request_ids)
        return batch


class DecodeBatch:
    """One token for each of a fixed set of sequences, again and again.

    `tokens` (int32 [n], on the device) holds each sequence's next input token;
    `run()` executes the step and leaves float32 logits [n, vocab] in
    `logits`.  With a `sampler` (a callable `(logits, tokens_out, batch)` that
    launches kernels only) the step also writes the chosen tokens back into
    `tokens`, so that steps chain on the device.  After a first eager run the
    kernel sequence is captured in a CUDA graph and replayed; positions come
    from the cache's device-side lengths, so the same graph serves every step.
    Pages for all steps to come must be reserved before the first run."""

    def __init__(self, stepper: Stepper, slots: Sequence[int], use_graph: bool = True, sampler=None):
        self.stepper, self.slots = stepper, list(slots)
        self.model, self.cache = stepper.model, stepper.cache
        n = len(self.slots)
        dev = stepper.device
        self.n = n
        self.tokens = torch.zeros(n, dtype=torch.int32, device=dev)
        ar = torch.arange(n + 1, dtype=torch.int32)
        self.batch = BatchMeta(cu_seqlens=ar.to(dev), tok_seq=ar[:n].to(dev),
                               slots=torch.tensor(self.slots, dtype=torch.int32).to(dev),
                               lengths=self.cache.lengths, n_seqs=n, n_tokens=n, max_q_len=1,
                               max_kv_len=max([self.cache.reserved_host[s] for s in self.slots] + [self.cache.page_size]),
                               status=stepper.status)
        self.sampler = sampler
        self.logits = None
        # a part that looks at device values on the host (`graph_safe = False` on its class or instance) cannot be
        # captured: the step then runs eagerly, launch by launch, with the same results
        self.use_graph = use_graph and dev.type == "cuda" and self.model.graph_safe()
        self.graph = None
        self.steps_run = 0

    def _body(self):
        self.logits = self.model.forward(self.tokens, self.batch, self.cache, None)
        ops.advance_lengths(self.batch)
        if self.sampler is not None:
            self.sampler(self.logits, self.tokens, self.batch)

    def run(self) -> torch.Tensor:
        for s in self.slots:
            if self.cache.lengths_host[s] + 1 > self.cache.reserved_host[s]:
                self.cache.reserve(s, self.cache.lengths_host[s] + 1)
        self.cache.sync_tables()
        if not self.use_graph:
            self._body()
        elif self.graph is None and self.steps_run == 0:
            self._body()                               # eager: loads libraries, warms allocations
        elif self.graph is None:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            # No garbage collection while the stream is capturing: a collection that happens to free an OLD
            # captured step (caches, steppers and their decode batches refer to each other, so they die by
            # collection, at a moment of Python's choosing) destroys its CUDA graph, which is not permitted
            # during a capture and silently invalidates this one.  torch collects once before it starts.
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g):
                    self._body()
            finally:
                if gc_was_on:
                    gc.enable()
            self.graph = g
            g.replay()
        else:
            self.graph.replay()
        self.steps_run += 1
        self.cache.note_advance(self.slots, [1] * self.n)
        return self.logits
