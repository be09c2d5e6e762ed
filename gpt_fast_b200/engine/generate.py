"""The generation loop: requests in, token sequences out.

gpt-fast's `generate` (generate.py:139-211) repeats ONE prompt batch_size
times, produces exactly max_new_tokens tokens per row (one from `prefill`, the
rest from `decode_n_tokens`) and knows no stop token.  This loop keeps those
three functions and the token budget, and adds what a library needs around
them: requests with prompts of unequal lengths, taken batch_size at a time,
one batch after another; all prompts of a batch in ONE prefill step; stop
tokens per sequence (the stop token is kept in the output); sequences that end
early leave the batch, which goes on with the rest; slots and pages go back to
the cache when a batch ends and serve the next one.
"""
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from ..cache import Cache
from ..sampling import SamplingParams, sample
from .model import Transformer
from .step import DecodeBatch, Stepper


@dataclass
class GenerationStats:
    batches: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    decode_tokens: int = 0           # tokens produced by decode steps (excludes each prefill's first token)
    per_batch: List[dict] = field(default_factory=list)


class _Sampler:
    """Launches the sampling kernel for a fixed number of requests; the token
    index of a row is its sequence's length on the device (the position the
    new token will take), read through the batch's slots.  Request ids and seed
    live in device memory, so that a captured decode graph can serve another
    call: `retarget` rewrites them in place."""

    def __init__(self, params: SamplingParams, request_ids: Sequence[int], device):
        self.temperature, self.top_k = params.temperature, params.top_k
        self.request_ids = torch.tensor(list(request_ids), dtype=torch.int64).to(device)
        self.seed = torch.tensor([params.seed & (2 ** 63 - 1)], dtype=torch.int64).to(device)

    def key(self):
        return (self.temperature, self.top_k, self.request_ids.shape[0])

    def retarget(self, params: SamplingParams, request_ids: Sequence[int]) -> None:
        self.request_ids.copy_(torch.tensor(list(request_ids), dtype=torch.int64), non_blocking=True)
        self.seed.copy_(torch.tensor([params.seed & (2 ** 63 - 1)], dtype=torch.int64), non_blocking=True)

    def __call__(self, logits, tokens_out, batch):
        sample(logits, self.temperature, self.top_k, seed=0, seed_dev=self.seed, request_ids=self.request_ids,
               token_index=batch.lengths, index_map=batch.slots, out=tokens_out)


def prefill(stepper: Stepper, slots: Sequence[int], prompts: Sequence[Sequence[int]], sampler: _Sampler) -> torch.Tensor:
    """All prompts of a batch in one step; returns each sequence's first new
    token (int32 [n], on the device).  gpt-fast: generate.py:59-62."""
    logits = stepper.step(slots, prompts, want="last")
    out = torch.empty(len(slots), dtype=torch.int32, device=logits.device)
    n = len(slots)
    from ..ops.types import BatchMeta
    ar = torch.arange(n + 1, dtype=torch.int32).to(logits.device)
    meta = BatchMeta(ar, ar[:n], torch.tensor(list(slots), dtype=torch.int32).to(logits.device), stepper.cache.lengths,
                     n, n, 1, 0, stepper.status)
    sampler(logits, out, meta)
    return out


def decode_one_token(batch: DecodeBatch) -> torch.Tensor:
    """One step of one token per sequence; `batch.tokens` holds the inputs and
    receives the sampled tokens.  gpt-fast: generate.py:64-68."""
    batch.run()
    return batch.tokens


def decode_n_tokens(batch: DecodeBatch, n_steps: int, history: torch.Tensor, first_row: int, cols: torch.Tensor,
                    after_step: Optional[Callable] = None) -> int:
    """Up to n_steps decode steps back to back; row first_row + i of `history` receives step i's tokens in
    the columns `cols` (the batch's sequences).  after_step(tokens), if given, runs on the host after each
    step has been launched (the GPU is already busy with it) and ends the stretch by returning True.
    Returns the number of steps run.  gpt-fast: generate.py:70-83."""
    for i in range(n_steps):
        toks = decode_one_token(batch)
        history[first_row + i].index_copy_(0, cols, toks)
        if after_step is not None and after_step(toks):
            return i + 1
    return n_steps


def _plan_batches(n_requests: int, batch_size: int) -> List[List[int]]:
    if batch_size < 1:
        raise ValueError("batch_size must be at least 1")
    return [list(range(i, min(i + batch_size, n_requests))) for i in range(0, n_requests, batch_size)]


def cache_tokens_needed(prompt_lens: Sequence[int], max_new_tokens: int, batch_size: int, page_size: int) -> int:
    """Tokens (whole pages per sequence) the largest batch of a run holds."""
    worst = 0
    for ids in _plan_batches(len(prompt_lens), batch_size):
        worst = max(worst, sum(-(-(prompt_lens[i] + max_new_tokens) // page_size) * page_size for i in ids))
    return worst


@torch.no_grad()
def generate(model: Transformer, prompts: Sequence[Sequence[int]], max_new_tokens: int, *,
             batch_size: Optional[int] = None, temperature: float = 0.8, top_k: Optional[int] = 200,
             seed: int = 1234, stop_tokens: Optional[Sequence[int]] = None, callback: Optional[Callable] = None,
             cache: Optional[Cache] = None, use_graph: bool = True, first_request_id: int = 0):
    """Continue every prompt (a list of token ids) by up to max_new_tokens tokens.

    Returns (sequences, stats): sequences[i] is prompt i followed by its new
    tokens, a list of ints; a sequence ends early, its stop token included,
    when it draws one of `stop_tokens` (default: the model's own, may be empty).
    Requests are served batch_size at a time (default: all at once), one batch
    after another on the same cache.  callback(request_ids, tokens) is called
    once for the prefill and once per decode step with the ids of the requests
    that were still running and their new tokens (an int32 tensor); a decode
    step's call comes while the next step is already running on the GPU."""
    prompts = [list(map(int, p)) for p in prompts]
    if not prompts:
        return [], GenerationStats()
    if any(len(p) == 0 for p in prompts):
        raise ValueError("a prompt must hold at least one token")
    if max_new_tokens < 1:
        raise ValueError("max_new_tokens must be at least 1")
    batch_size = batch_size or len(prompts)
    stops = frozenset(model.spec.stop_tokens if stop_tokens is None else stop_tokens)
    params = SamplingParams(temperature, top_k, seed)
    lens = [len(p) for p in prompts]
    if cache is None:
        # like gpt-fast's setup_caches (model.py:117-119): the model keeps its cache and only replaces
        # it when a call needs more
        from ..cache.paged import DEFAULT_PAGE_SIZE
        cache = model.default_cache(cache_tokens_needed(lens, max_new_tokens, batch_size, DEFAULT_PAGE_SIZE),
                                    min(batch_size, len(prompts)), max(lens) + max_new_tokens)
    stepper = Stepper.of(model, cache)
    stats = GenerationStats()
    results: List[Optional[List[int]]] = [None] * len(prompts)
    sync = torch.cuda.synchronize if model.device.type == "cuda" else (lambda: None)

    for ids in _plan_batches(len(prompts), batch_size):
        n = len(ids)
        slots = cache.begin(n)
        try:
            for s, i in zip(slots, ids):
                cache.reserve(s, lens[i] + max_new_tokens)
            req_ids = [first_request_id + i for i in ids]
            history = torch.zeros(max_new_tokens, n, dtype=torch.int32, device=model.device)
            sync()
            t0 = time.perf_counter()
            first = prefill(stepper, slots, [prompts[i] for i in ids], _Sampler(params, req_ids, model.device))
            history[0].copy_(first)
            if callback is not None:
                callback(req_ids, first)
            sync()
            t1 = time.perf_counter()

            # Decode.  `live` lists the columns of `history` (sequences of this batch) still being
            # continued.  The host looks at a step's tokens one step late: while the GPU runs step
            # k, the host reads step k-1's tokens (copied to pinned memory behind an event) and
            # decides who has stopped.  A sequence that drew a stop token therefore takes part in
            # one more step, whose token is dropped; the outputs are the same as with an immediate
            # check, and the host work no longer sits between two steps.
            watch = bool(stops) or callback is not None
            done = [False] * n
            n_new = [1] * n                                        # tokens kept so far, per column

            def look(tokens_host, cols_of_step):
                """Digest one step's tokens: callback, stop tokens, counts."""
                keep = [(j, t) for j, t in zip(cols_of_step, tokens_host) if not done[j]]
                if callback is not None and keep and cols_of_step is not None:
                    callback([req_ids[j] for j, _ in keep],
                             torch.tensor([t for _, t in keep], dtype=torch.int32))
                for j, t in keep:
                    n_new[j] += 1
                    if t in stops:
                        done[j] = True

            if stops:
                for j, t in enumerate(first.tolist()):
                    if t in stops:
                        done[j] = True
            live = list(range(n))
            cur = first
            batch = None
            pending = None                                         # (event, pinned tokens, columns) of the step in flight
            pins = [torch.empty(n, dtype=torch.int32, pin_memory=model.device.type == "cuda") for _ in range(2)]
            row = 1
            steps = 0
            decode_tokens = 0

            def after_step(cur_tokens):
                """On the host while the step just launched runs: queue its tokens for the next look, digest
                the step before it; True if a sequence has ended (the batch is then made anew)."""
                nonlocal pending, steps, decode_tokens
                this = None
                if watch:
                    pin = pins[steps & 1]
                    pin[:len(live)].copy_(cur_tokens, non_blocking=True)
                    ev = torch.cuda.Event() if model.device.type == "cuda" else None
                    if ev is not None:
                        ev.record()
                    this = (ev, pin, list(live))
                else:
                    for j in live:
                        n_new[j] += 1
                decode_tokens += len(live)
                steps += 1
                if pending is not None:                            # the step before this one, while this one runs
                    ev, pin, pcols = pending
                    if ev is not None:
                        ev.synchronize()
                    look(pin[:len(pcols)].tolist(), pcols)
                pending = this
                return any(done[j] for j in live)

            while row < max_new_tokens:
                keep = [j for j in live if not done[j]]
                if not keep:
                    break
                if batch is None or keep != live:
                    idx = torch.tensor([live.index(j) for j in keep], dtype=torch.long).to(model.device)
                    nxt = cur.index_select(0, idx)
                    live = keep
                    batch = stepper.decode_batch([slots[j] for j in live], use_graph, params, [req_ids[j] for j in live])
                    batch.tokens.copy_(nxt)
                    cols = torch.tensor(live, dtype=torch.long).to(model.device)
                row += decode_n_tokens(batch, max_new_tokens - row, history, row, cols, after_step)
                cur = batch.tokens
            if pending is not None:
                ev, pin, pcols = pending
                if ev is not None:
                    ev.synchronize()
                look(pin[:len(pcols)].tolist(), pcols)
            sync()
            t2 = time.perf_counter()
            stepper.check()
            hist = history.cpu()
            for j, i in enumerate(ids):
                results[i] = prompts[i] + hist[:n_new[j], j].tolist()
        finally:
            cache.end(slots)
        stats.batches += 1
        stats.prompt_tokens += sum(lens[i] for i in ids)
        stats.generated_tokens += sum(n_new)
        stats.prefill_seconds += t1 - t0
        stats.decode_seconds += t2 - t1
        stats.decode_steps += steps
        stats.decode_tokens += decode_tokens
        stats.per_batch.append(dict(requests=n, prefill_seconds=t1 - t0, decode_seconds=t2 - t1, decode_steps=steps,
                                    decode_tokens=decode_tokens))
    return results, stats
