"""The serving kernels at the layer sizes of Llama-3.1-8B (two layers, random
weights): head_dim 128, 32 heads in 8 groups, width 4096, feed-forward 14336,
vocabulary 128256.  The tiny configurations never reach the tensor-core
attention kernels or the split-K / persistent products; this does."""
import pytest
import torch

import gpt_fast_b200 as gf
import plain_llama
import traces
from gpt_fast_b200.engine.replay import Replayer
from conftest import assert_within_bf16_noise

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    cfg = gf.config_from_name("llama-3.1-8b")
    cfg["num_hidden_layers"] = 2
    cfg["max_position_embeddings"] = 4096
    d = str(tmp_path_factory.mktemp("llama8b_2layers"))
    gf.write_model_folder(d, cfg, seed=5)
    p, pc = plain_llama.load_folder(d)
    reqs = traces.make_requests(cfg["vocab_size"], [40, 3, 200, 77], seed=3)
    ref = {"float32": {}, "bfloat16": {}}
    for rid, toks in reqs.items():
        for name, act in (("float32", None), ("bfloat16", torch.bfloat16)):
            logits = plain_llama.forward(toks, p, pc, act=act)
            for j in range(len(toks) - traces.tail_of(toks), len(toks)):
                ref[name][(rid, j)] = logits[j]
    return d, reqs, ref, cfg["vocab_size"], (p, pc)


def run(model, steps, V):
    rp = Replayer(model, traces.peak_tokens(steps), None)
    out = {st["step"]: rp.run_step(st) for st in steps}
    return traces.collect(steps, out, V)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_8b_layer_sizes_all_cuts(big, dtype):
    folder, reqs, refs, V, _ = big
    ref, emu = refs["float32"], refs["bfloat16"]
    model = gf.load(folder, dtype=dtype, device="cuda")
    with torch.no_grad():
        for cut, steps in (("whole", traces.whole(reqs)), ("stepped", traces.stepped(reqs)), ("batched", traces.batched(reqs, 3))):
            rows = run(model, steps, V)
            assert set(rows) == set(ref)
            for key in sorted(ref):
                got, want = torch.from_numpy(rows[key].copy()), ref[key]
                where = f"{cut}: request {key[0]}, token {key[1]}"
                if dtype == "float32":
                    torch.testing.assert_close(got, want, rtol=1e-3, atol=2e-4, msg=lambda m: f"{where}\n{m}")
                else:
                    # How far may bfloat16 be from the 32-bit logits?  As far as the plain implementation is
                    # when its activations are rounded to bfloat16 where the library stores them (`emu`): that
                    # is the noise of the format on this model (about 1 % of a row's scale), measured, not
                    # guessed.  Two ways of running the same tokens give two samples of that noise, so they are
                    # not compared with each other but each with the 32-bit logits: the library's error must
                    # stay within 1.5 x the plain implementation's in the mean and 2 x at the worst element.
                    # A wrong position, head or page shows as an error of the order of the scale itself.
                    assert_within_bf16_noise(got, want, emu[key], where)


def test_8b_layer_sizes_greedy_tokens_agree_between_precisions(big):
    """Greedy generation in both precisions against the plain implementation: in 32-bit the tokens are the plain
    argmax wherever its two best logits are not nearly tied; in bfloat16 each chosen token's 32-bit logit trails
    the best one by no more than the format's measured noise allows (twice the largest error of a logit, which is
    itself bounded by twice the noise), along the sequence that was actually generated."""
    folder, reqs, _, _, (p, pc) = big
    prompts = [t[:20] for t in reqs.values() if len(t) >= 20]
    n_new = 8
    for dtype in ("float32", "bfloat16"):
        model = gf.load(folder, dtype=dtype, device="cuda")
        out, _ = gf.generate(model, prompts, n_new, temperature=0.0, stop_tokens=[])
        for pr, seq in zip(prompts, out):
            assert seq[:len(pr)] == pr and len(seq) == len(pr) + n_new
            logits = plain_llama.forward(seq[:-1], p, pc)
            noise = plain_llama.forward(seq[:-1], p, pc, act=torch.bfloat16) - logits
            for j in range(len(pr) - 1, len(seq) - 1):
                margin = 1e-3 if dtype == "float32" else 4 * float(noise[j].abs().max())
                assert logits[j, seq[j + 1]] >= logits[j].max() - margin, f"{dtype}: new token {j + 1 - len(pr)}"


@pytest.mark.parametrize("hidden,heads,n_prompt", [(2048, 16, 4800), (4096, 32, 7296)])
def test_long_prompt_and_decoding_behind_it(hidden, heads, n_prompt):
    """A long prompt and four decoded places behind it (the decode step cuts the cache into many slices), one layer
    with head_dim 128 and 8 key/value heads: the last places of the prompt and the decoded places against the plain
    implementation, judged like the test above.  4,800 tokens at 16 heads: every block of the one-tile prefill
    attention kernel walks through several tiles, up to 38 key blocks deep.  7,296 tokens at 32 heads: enough work
    for the kernel that takes two query tiles per block."""
    cfg = gf.config_from_name("llama-3.1-8b")
    cfg.update(hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=8, intermediate_size=1024,
               num_hidden_layers=1, vocab_size=512, max_position_embeddings=8192)
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        gf.write_model_folder(d, cfg, seed=11)
        p, pc = plain_llama.load_folder(d)
        toks = traces.make_requests(cfg["vocab_size"], [n_prompt + 4], seed=2)["r0"]
        want = plain_llama.forward(toks, p, pc)[-8:]
        noise = plain_llama.forward(toks, p, pc, act=torch.bfloat16)[-8:] - want
        model = gf.load(d, dtype="bfloat16", device="cuda")
        with torch.no_grad():
            cache = model.new_cache(max_tokens=n_prompt + 64, max_seqs=1)
            st = gf.Stepper(model, cache)
            slot = cache.begin(1)
            rows = [st.step(slot, [toks[:n_prompt]], [[n_prompt - 4, n_prompt - 3, n_prompt - 2, n_prompt - 1]]).cpu()]
            for t in toks[n_prompt:]:
                rows.append(st.step(slot, [[t]], "last").cpu())
            st.check()
            cache.end(slot)
        got = torch.cat(rows)
        err = got - want
        rms = lambda t: float(t.pow(2).mean().sqrt())
        assert rms(err) <= 1.5 * rms(noise), f"rms error {rms(err):.4f}, bfloat16 noise {rms(noise):.4f}"
        assert float(err.abs().max()) <= 2.0 * float(noise.abs().max())
