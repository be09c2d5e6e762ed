"""The engine against the plain implementation: whole requests, the last 32
tokens one by one, batches of unequal lengths one after another (slots used
again), long decoding, first tokens, greedy generation.

Every test runs twice: on the CPU with the plain statement of the kernels
standing in (this checks the library's host-side logic, and the test itself,
without a GPU), and, marked gpu, on the device with the real kernels in
float32 and bfloat16."""
import pytest
import torch

import gpt_fast_b200 as gf
from gpt_fast_b200 import ops
from gpt_fast_b200.engine.replay import Replayer
import plain_llama
import plain_ops
import traces
from conftest import assert_within_bf16_noise

LENGTHS = {"tiny-a": [5, 11, 17, 70, 33, 64, 1], "tiny-b": [1, 7, 30, 64, 129, 40, 65]}
BACKENDS = [
    pytest.param(("cpu", "float32"), id="cpu-standin-f32"),
    pytest.param(("cuda", "float32"), id="cuda-f32", marks=pytest.mark.gpu),
    pytest.param(("cuda", "bfloat16"), id="cuda-bf16", marks=pytest.mark.gpu),
]


def tolerance(dtype):
    # float32: rounding of 32-bit sums in another order.  bfloat16 is not judged by a tolerance but against
    # the measured noise of the format on this model (`assert_within_bf16_noise`).
    assert dtype == "float32"
    return dict(rtol=1e-4, atol=2e-5)


@pytest.fixture(params=BACKENDS)
def backend(request):
    device, dtype = request.param
    prev = ops.use_kernels(plain_ops.PlainOps()) if device == "cpu" else None
    yield device, dtype
    if device == "cpu":
        ops.use_kernels(prev)


@pytest.fixture(params=["tiny-a", "tiny-b"])
def setup(request, backend, tiny_folders):
    device, dtype = backend
    folder = tiny_folders[request.param]
    model = gf.load(folder, dtype=dtype, device=device)
    p, cfg = plain_llama.load_folder(folder)
    reqs = traces.make_requests(cfg["vocab_size"], LENGTHS[request.param], seed=5)
    return dict(name=request.param, model=model, p=p, cfg=cfg, reqs=reqs, dtype=dtype, device=device, folder=folder)


def replay(model, steps):
    rp = Replayer(model, traces.peak_tokens(steps), None)
    outputs = {}
    for st in steps:
        outputs[st["step"]] = rp.run_step(st)
    assert not rp.slot_of, "a trace must end every request"
    assert rp.cache.slots.n_free == rp.cache.n_slots and rp.cache.pages_free == rp.cache.n_pages
    return outputs


def plain_rows(s, act=None):
    rows = {}
    for rid, toks in s["reqs"].items():
        logits = plain_llama.forward(toks, s["p"], s["cfg"], act=act)
        k = traces.tail_of(toks)
        for j in range(len(toks) - k, len(toks)):
            rows[(rid, j)] = logits[j]
    return rows


def compare(rows, ref, dtype, emu=None):
    """float32: close to the plain logits; bfloat16: within the format's noise (`emu`: the plain
    implementation with activations rounded to bfloat16)."""
    assert set(rows) == set(ref)
    for key in sorted(ref):
        got = torch.as_tensor(rows[key])
        where = f"first wrong place: request {key[0]}, token {key[1]}"
        if dtype == "float32":
            try:
                torch.testing.assert_close(got, ref[key], **tolerance(dtype))
            except AssertionError as e:
                raise AssertionError(f"{where}\n{e}") from None
        else:
            assert_within_bf16_noise(got, ref[key], emu[key], where)


@pytest.mark.parametrize("cut", ["whole", "stepped", "batched"])
def test_replay_matches_plain(setup, cut):
    s = setup
    with torch.no_grad():
        steps = {"whole": traces.whole, "stepped": traces.stepped,
                 "batched": lambda r: traces.batched(r, 3)}[cut](s["reqs"])
        rows = traces.collect(steps, replay(s["model"], steps), s["cfg"]["vocab_size"])
        compare(rows, plain_rows(s), s["dtype"], plain_rows(s, torch.bfloat16) if s["dtype"] == "bfloat16" else None)


def test_cuts_agree_with_each_other(setup):
    """The same place gives the same logits however the tokens were cut into steps
    and whatever else was in the batch (float32: to rounding of 32-bit sums)."""
    s = setup
    with torch.no_grad():
        got = {}
        for name, fn in (("whole", traces.whole), ("stepped", traces.stepped), ("batched", lambda r: traces.batched(r, 3))):
            steps = fn(s["reqs"])
            got[name] = traces.collect(steps, replay(s["model"], steps), s["cfg"]["vocab_size"])
        # bfloat16: two ways of running the same tokens are two samples of the format's noise, so they
        # are compared with each other at twice the single-sample bound
        emu, ref = (plain_rows(s, torch.bfloat16), plain_rows(s)) if s["dtype"] == "bfloat16" else (None, None)
        for other in ("stepped", "batched"):
            for key in sorted(got["whole"]):
                a, b = torch.as_tensor(got[other][key]), torch.as_tensor(got["whole"][key])
                where = f"{other} against whole: request {key[0]}, token {key[1]}"
                if s["dtype"] == "float32":
                    torch.testing.assert_close(a, b, rtol=1e-5, atol=2e-6, msg=lambda m: f"{where}\n{m}")
                else:
                    assert_within_bf16_noise(a, b, b + (emu[key] - ref[key]), where, rms_factor=3.0, max_factor=4.0)


def test_first_tokens_and_long_decoding(setup):
    """One sequence from its very first token, one token per step, across several
    pages: every step's logits against the whole sequence's."""
    s = setup
    V = s["cfg"]["vocab_size"]
    toks = traces.make_requests(V, [min(150, s["model"].spec.max_position - 4)], seed=9)["r0"]
    with torch.no_grad():
        model = s["model"]
        cache = model.new_cache(max_tokens=192)
        st = gf.Stepper(model, cache)
        slot = cache.begin(1)
        rows = [st.step(slot, [[t]], "last")[0].cpu() for t in toks]
        st.check()
        cache.end(slot)
    ref = plain_llama.forward(toks, s["p"], s["cfg"])
    emu = plain_llama.forward(toks, s["p"], s["cfg"], act=torch.bfloat16) if s["dtype"] == "bfloat16" else None
    for j, row in enumerate(rows):
        if s["dtype"] == "bfloat16":
            assert_within_bf16_noise(row, ref[j], emu[j], f"first wrong token: {j}")
            continue
        try:
            torch.testing.assert_close(row, ref[j], **tolerance(s["dtype"]))
        except AssertionError as e:
            raise AssertionError(f"first wrong token: {j}\n{e}") from None


def test_greedy_generation_through_the_entry_point(setup):
    s = setup
    prompts = [t[: max(1, len(t) // 2)] for t in s["reqs"].values()][:5]
    n_new = 10
    seqs, stats = gf.generate(s["model"], prompts, n_new, temperature=0.0, batch_size=2)
    assert stats.batches == 3 and stats.generated_tokens == n_new * len(prompts)
    for pr, seq in zip(prompts, seqs):
        assert seq[:len(pr)] == pr and len(seq) == len(pr) + n_new
        if s["dtype"] == "float32":
            assert seq[len(pr):] == plain_llama.greedy_generate(pr, n_new, s["p"], s["cfg"])
        else:
            # bfloat16 may pick another token where two logits are close: follow the engine's
            # own sequence and require that each chosen token is (nearly) the plain argmax
            # (by how much?  the chosen token's 32-bit logit can trail the best one by at most twice the
            # largest error of a bfloat16 logit, and that error is bounded by twice the format's measured noise)
            logits = plain_llama.forward(seq[:-1], s["p"], s["cfg"])
            noise = plain_llama.forward(seq[:-1], s["p"], s["cfg"], act=torch.bfloat16) - logits
            for j in range(len(pr) - 1, len(seq) - 1):
                assert logits[j, seq[j + 1]] >= logits[j].max() - 4 * float(noise[j].abs().max()), f"token {j + 1}"


def test_sampled_generation_is_the_same_alone_and_in_a_batch(setup):
    s = setup
    prompts = [t[: max(1, len(t) // 2)] for t in s["reqs"].values()][:4]
    kw = dict(temperature=0.8, top_k=50, seed=7)
    together, _ = gf.generate(s["model"], prompts, 8, batch_size=4, **kw)
    for i, pr in enumerate(prompts):
        alone, _ = gf.generate(s["model"], [pr], 8, first_request_id=i, **kw)
        if s["dtype"] == "float32":
            assert alone[0] == together[i]
        else:
            # bfloat16 products sum in another order for another batch shape, so a near tie between two noisy
            # scores may fall the other way and the sequences part there; the noise itself (keyed by seed,
            # request and place) must be the same, which shows in the first token: its logits come from the
            # same prompt and the scores of the race are far apart for these seeds
            assert alone[0][len(pr)] == together[i][len(pr)], f"request {i}: first sampled token differs alone and in a batch"


def test_stop_tokens_end_a_sequence_early(setup):
    s = setup
    prompts = [t[: max(1, len(t) // 2)] for t in s["reqs"].values()][:3]
    free, _ = gf.generate(s["model"], prompts, 12, temperature=0.0)
    stop = free[0][len(prompts[0]) + 3]                       # the 4th new token of request 0
    seqs, stats = gf.generate(s["model"], prompts, 12, temperature=0.0, stop_tokens=[stop])
    for pr, f, q in zip(prompts, free, seqs):
        new = f[len(pr):]
        cut = new.index(stop) + 1 if stop in new else len(new)
        assert q == pr + new[:cut]                              # the stop token is kept, nothing follows it
    assert len(seqs[0]) <= len(prompts[0]) + 4


def test_repeated_calls_reuse_the_cache_and_its_decode_graphs(setup):
    """generate() keeps the model's cache between calls, and the cache keeps the captured decode
    steps; a later call with other prompts, another seed and other request ids must give what a
    fresh model gives."""
    s = setup
    model = s["model"]
    prompts = [t[: max(1, len(t) // 2)] for t in s["reqs"].values()][:3]
    other = [p[: max(1, len(p) - 1)][::-1] for p in prompts]          # no longer than the first call's: the cache fits
    first, _ = gf.generate(model, prompts, 6, temperature=0.8, top_k=40, seed=3)
    cache = model._default_cache
    again, _ = gf.generate(model, other, 6, temperature=0.8, top_k=40, seed=9, first_request_id=100)
    assert model._default_cache is cache and cache.slots.n_free == cache.n_slots      # same cache, everything given back
    fresh = gf.load(s["folder"], dtype=s["dtype"], device=s["device"])
    want, _ = gf.generate(fresh, other, 6, temperature=0.8, top_k=40, seed=9, first_request_id=100)
    if s["dtype"] == "float32":
        assert again == want
    else:
        assert [a[:len(p) + 1] for a, p in zip(again, other)] == [w[:len(p) + 1] for w, p in zip(want, other)]
    repeat, _ = gf.generate(model, prompts, 6, temperature=0.8, top_k=40, seed=3)
    assert repeat == first                                                              # and the same call gives the same tokens
