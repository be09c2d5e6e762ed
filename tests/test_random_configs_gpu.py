"""Random small Llama configurations through the engine, in 32-bit and in bfloat16, against the plain
implementation: head sizes in steps of 16 up to 256, any number of heads and groups (one to eight query heads per
key/value head, prime counts among them), widths, feed-forward sizes and vocabularies that are no power of two (down
to 8 and 17), tied and untied output, one to three layers.  Every request is prefilled in one batch of unequal
lengths (all places wanted) and then decoded for two steps.  The two tiny named configurations pin two points of
this space; this walks through more of it with a fixed seed."""
import random
import tempfile

import pytest
import torch

import gpt_fast_b200 as gf
import plain_llama
import traces

pytestmark = pytest.mark.gpu


def random_config(rng):
    d_head = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256])
    groups = rng.choice([1, 2, 3, 5, 8])
    heads = groups * rng.choice([1, 2, 3, 4, 7, 8])
    return {"model_type": "llama", "architectures": ["LlamaForCausalLM"], "hidden_size": heads * d_head,
            "num_attention_heads": heads, "num_key_value_heads": groups, "num_hidden_layers": rng.choice([1, 2, 3]),
            "intermediate_size": rng.choice([8, 24, 100, 172, 384, 1000, 1536]),
            "vocab_size": rng.choice([17, 100, 257, 1000, 4099]), "max_position_embeddings": 512,
            "rope_theta": rng.choice([10000.0, 500000.0]), "rms_norm_eps": rng.choice([1e-5, 1e-6]), "rope_scaling": None,
            "tie_word_embeddings": rng.choice([True, False]), "hidden_act": "silu"}


def run_engine(folder, dtype, reqs):
    """Prompts (all but the last two tokens of each request) in one step, then two decode steps; logits by (request, place)."""
    model = gf.load(folder, dtype=dtype, device="cuda")
    ids = list(reqs)
    got = {}
    with torch.no_grad():
        cache = model.new_cache(max_tokens=sum(-(-len(reqs[i]) // 64) * 64 for i in ids) + 64, max_seqs=len(ids))
        st = gf.Stepper(model, cache)
        slots = cache.begin(len(ids))
        cut = {i: max(1, len(reqs[i]) - 2) for i in ids}
        out = st.step(slots, [reqs[i][:cut[i]] for i in ids], "all").cpu()
        r = 0
        for i in ids:
            for j in range(cut[i]):
                got[(i, j)] = out[r]
                r += 1
        for n in range(2):
            live = [k for k in range(len(ids)) if cut[ids[k]] + n < len(reqs[ids[k]])]
            if not live:
                break
            out = st.step([slots[k] for k in live], [[reqs[ids[k]][cut[ids[k]] + n]] for k in live], "last").cpu()
            for row, k in enumerate(live):
                got[(ids[k], cut[ids[k]] + n)] = out[row]
        st.check()
        cache.end(slots)
    return got


@pytest.mark.parametrize("seed", range(8))
def test_random_configuration(seed):
    rng = random.Random(1000 + seed)
    cfg = random_config(rng)
    lens = [rng.choice([1, 2, 5, 33, 64, 65, 130, 200]) for _ in range(rng.choice([1, 2, 4]))]
    what = f"{cfg['num_attention_heads']} heads in {cfg['num_key_value_heads']} groups of head_dim " \
           f"{cfg['hidden_size'] // cfg['num_attention_heads']}, feed-forward {cfg['intermediate_size']}, vocabulary " \
           f"{cfg['vocab_size']}, {cfg['num_hidden_layers']} layers, lengths {lens}"
    with tempfile.TemporaryDirectory() as d:
        gf.write_model_folder(d, cfg, seed=seed)
        p, pc = plain_llama.load_folder(d)
        reqs = traces.make_requests(cfg["vocab_size"], lens, seed=seed)
        keys = [(rid, j) for rid, toks in reqs.items() for j in range(len(toks))]
        ref = {rid: plain_llama.forward(toks, p, pc) for rid, toks in reqs.items()}
        emu = {rid: plain_llama.forward(toks, p, pc, act=torch.bfloat16) for rid, toks in reqs.items()}
        want = torch.stack([ref[r][j] for r, j in keys])
        noise = torch.stack([emu[r][j] for r, j in keys]) - want
        for dtype in ("float32", "bfloat16"):
            got = run_engine(d, dtype, reqs)
            assert set(got) == set(keys), what
            have = torch.stack([got[k] for k in keys])
            if dtype == "float32":
                torch.testing.assert_close(have, want, rtol=1e-3, atol=2e-4, msg=lambda m: f"{what}\n{m}")
            else:
                # judged as at the 8B layer sizes: against the noise of the format on this model, which the plain
                # implementation with bfloat16 activations measures, over all places together
                err = have - want
                rms = lambda t: float(t.pow(2).mean().sqrt())
                assert rms(err) <= 1.5 * rms(noise), f"{what}: rms error {rms(err):.4f}, bfloat16 noise {rms(noise):.4f}"
                assert float(err.abs().max()) <= 2.0 * float(noise.abs().max()), \
                    f"{what}: max error {float(err.abs().max()):.4f}, bfloat16 noise {float(noise.abs().max()):.4f}"
