"""Greedy generation through the entry point on random requests (numbers of prompts, lengths around the page
edge, batch sizes, stop tokens, with and without the captured decode step), in 32-bit on the GPU, against greedy
decoding with the plain implementation, token by token.  A near-tie between the plain implementation's two best
logits ends the comparison of that request: either token is right there."""
import random
import tempfile

import pytest
import torch

import gpt_fast_b200 as gf
import plain_llama

pytestmark = pytest.mark.gpu


def plain_greedy(prompt, p, pc, max_new, stops):
    """(tokens, certain): greedy continuation; certain is False from the first near-tie on."""
    seq = list(prompt)
    for _ in range(max_new):
        logits = plain_llama.forward(seq, p, pc)[-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) < 1e-4:
            return seq, False
        seq.append(int(logits.argmax()))
        if seq[-1] in stops:
            break
    return seq, True


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_random_requests_match_plain_greedy_decoding(name):
    rng = random.Random(7 if name == "tiny-a" else 8)
    with tempfile.TemporaryDirectory() as d:
        gf.write_model_folder(d, name, seed=3)
        p, pc = plain_llama.load_folder(d)
        vocab = gf.config_from_name(name)["vocab_size"]
        model = gf.load(d, dtype="float32", device="cuda")
        for trial in range(6):
            prompts = [[rng.randrange(vocab) for _ in range(rng.choice([1, 2, 7, 30, 63, 64, 65, 80]))]
                       for _ in range(rng.choice([1, 2, 3, 5, 9]))]
            max_new = rng.choice([1, 2, 5, 17, 40])
            stops = rng.sample(range(vocab), rng.choice([0, 3, 40]))
            batch_size = rng.choice([None, 1, 2, 4])
            out, _ = gf.generate(model, prompts, max_new, batch_size=batch_size, temperature=0.0, stop_tokens=stops,
                                 use_graph=rng.choice([True, False]))
            for i, prompt in enumerate(prompts):
                want, certain = plain_greedy(prompt, p, pc, max_new, stops)
                what = f"trial {trial}, request {i} of {len(prompts)}, batch size {batch_size}, {max_new} new tokens, {len(stops)} stop tokens"
                if certain:
                    assert out[i] == want, what
                else:
                    assert out[i][:len(want)] == want, what
