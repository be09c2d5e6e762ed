"""Random batches one after another through `generate`: every request keeps its prompt, ends within its budget,
and the same batch run a second time gives the same tokens (the kernels add in a fixed order), with slots and pages
of earlier batches in use again.  A small model whose sizes take the tensor-core paths (head_dim 128, pages of 64)."""
import random

import pytest
import torch

import gpt_fast_b200 as gf

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    cfg = gf.config_from_name("tiny-b")
    cfg.update(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, intermediate_size=512, num_hidden_layers=2,
               vocab_size=1000, max_position_embeddings=2048)
    cfg.pop("head_dim", None)
    folder = str(tmp_path_factory.mktemp("small128"))
    gf.write_model_folder(folder, cfg, seed=5)
    return gf.load(folder, dtype="bfloat16", device="cuda"), cfg["vocab_size"]


def test_random_batches_reproduce(model):
    model, V = model
    rng = random.Random(11)
    for n in range(40):
        B = rng.choice([1, 2, 3, 8, 17, 40])
        prompts = [[rng.randrange(V) for _ in range(rng.choice([1, 5, 63, 64, 65, 130, 300, 700]))] for _ in range(B)]
        n_new = rng.choice([1, 2, 17, 70])
        temperature, top_k, stop = rng.choice([0.0, 0.8]), rng.choice([None, 1, 50, 200]), [rng.randrange(V)]
        runs = []
        for _ in range(2):
            out, _ = gf.generate(model, prompts, n_new, temperature=temperature, top_k=top_k, stop_tokens=stop, seed=n)
            runs.append([list(o) for o in out])
        assert runs[0] == runs[1], f"batch {n}: the same requests gave other tokens the second time"
        for o, p in zip(runs[0], prompts):
            assert o[:len(p)] == p and 1 <= len(o) - len(p) <= n_new
            assert all(0 <= t < V for t in o)
    torch.cuda.synchronize()
