"""The plain implementation against gpt-fast's own model.py: logits that
tests/golden/make_golden.py computed once with gpt-fast's code on the CPU."""
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_llama
from golden import make_golden

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_gptfast_golden(name):
    c = make_golden.CONFIGS[name]
    gold = load_file(os.path.join(GOLDEN, f"{name}.safetensors"))
    p = make_golden.random_gptfast_weights(c)
    if not torch.allclose(make_golden.weights_checksum(p), gold["checksum"], rtol=1e-12):
        pytest.skip("this torch draws other random numbers than the one that made the golden files")
    for j, toks in enumerate(make_golden.tokens_for(c)):
        mine = plain_llama.forward(toks, p, make_golden.plain_cfg(c))
        torch.testing.assert_close(mine, gold[f"ref_whole_{j}"], rtol=1e-5, atol=2e-6)
        torch.testing.assert_close(mine, gold[f"ref_stepped_{j}"], rtol=1e-5, atol=2e-6)


def test_plain_sampling_formulas():
    logits = torch.tensor([[1.0, 3.0, 3.0, 2.0, -1.0]])
    p = plain_llama.logits_to_probs(logits, temperature=0.5, top_k=2)
    assert p[0, 0] == 0 and p[0, 3] == 0 and p[0, 4] == 0          # below the 2nd largest value
    assert torch.isclose(p[0, 1], torch.tensor(0.5)) and torch.isclose(p[0, 2], torch.tensor(0.5))   # the tie is kept
    cold = plain_llama.logits_to_probs(logits, temperature=0.0)     # clamped to 1e-5: nearly one-hot over the tie
    assert torch.isclose(cold[0, 1] + cold[0, 2], torch.tensor(1.0))
    noise = torch.tensor([[1.0, 4.0, 1.0, 1.0, 1.0]])
    assert int(plain_llama.exponential_race(p, noise)) == 2


def test_plain_rope_scaling_bands():
    f = plain_llama.rope_frequencies(24, 500000.0)
    s = plain_llama.rope_frequencies(24, 500000.0, dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                         original_max_position_embeddings=32))
    wavelen = 2 * torch.pi / f
    assert torch.equal(s[wavelen < 8], f[wavelen < 8])                              # short waves stay
    torch.testing.assert_close(s[wavelen > 32], f[wavelen > 32] / 8.0)              # long waves are divided
    mid = (wavelen >= 8) & (wavelen <= 32)
    assert mid.any() and ((s[mid] <= f[mid]) & (s[mid] >= f[mid] / 8.0)).all()
