"""Makes tests/golden/*.safetensors: logits of pytorch-labs/gpt-fast's own
`model.py`, run on the CPU in 32-bit on two tiny random Llama models, with the
logits of tests/plain_llama.py beside them for the record.

Run once, by hand, where gpt-fast's sources can be imported:

    python tests/golden/make_golden.py --reference /path/to/gpt-fast

`tests/test_plain.py` rebuilds the same weights from the same seeds, runs the
plain implementation and compares it with the stored logits of gpt-fast; a
checksum of the weights is stored too, so that a changed random stream is
told apart from a changed formula.
"""
import argparse
import os
import sys

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_llama  # noqa: E402

# Two configurations that differ in every size and option.
CONFIGS = {
    "tiny_a": dict(block_size=128, vocab_size=256, n_layer=2, n_head=4, dim=64, intermediate_size=172,
                   n_local_heads=4, rope_base=10000.0, norm_eps=1e-5, rope_scaling=None, tied=False,
                   seed=11, lengths=[5, 11, 17]),
    "tiny_b": dict(block_size=192, vocab_size=320, n_layer=3, n_head=6, dim=144, intermediate_size=384,
                   n_local_heads=2, rope_base=500000.0, norm_eps=1e-6,
                   rope_scaling=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                     original_max_position_embeddings=32),
                   tied=True, seed=12, lengths=[1, 7, 30, 64]),
}


def random_gptfast_weights(c):
    """Seeded weights by gpt-fast name: matrices N(0, 0.02), norms 1 + N(0, 0.1)."""
    g = torch.Generator().manual_seed(c["seed"])
    D, H, G, I, V = c["dim"], c["n_head"], c["n_local_heads"], c["intermediate_size"], c["vocab_size"]
    d = D // H

    def mat(*shape):
        return torch.randn(*shape, generator=g) * 0.02

    def norm():
        return 1.0 + torch.randn(D, generator=g) * 0.1

    p = {"tok_embeddings.weight": mat(V, D)}
    for i in range(c["n_layer"]):
        pre = f"layers.{i}."
        p[pre + "attention.wqkv.weight"] = mat((H + 2 * G) * d, D)
        p[pre + "attention.wo.weight"] = mat(D, D)
        p[pre + "feed_forward.w1.weight"] = mat(I, D)
        p[pre + "feed_forward.w2.weight"] = mat(D, I)
        p[pre + "feed_forward.w3.weight"] = mat(I, D)
        p[pre + "attention_norm.weight"] = norm()
        p[pre + "ffn_norm.weight"] = norm()
    p["norm.weight"] = norm()
    p["output.weight"] = p["tok_embeddings.weight"] if c["tied"] else mat(V, D)
    return p


def weights_checksum(p):
    return torch.stack([v.double().abs().sum() for k, v in sorted(p.items())]).sum().reshape(1)


def tokens_for(c):
    g = torch.Generator().manual_seed(c["seed"] + 1000)
    return [torch.randint(0, c["vocab_size"], (n,), generator=g) for n in c["lengths"]]


def plain_cfg(c):
    return dict(n_layer=c["n_layer"], n_head=c["n_head"], n_local_heads=c["n_local_heads"],
                head_dim=c["dim"] // c["n_head"], norm_eps=c["norm_eps"], rope_base=c["rope_base"],
                rope_scaling=c["rope_scaling"])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="folder holding gpt-fast's model.py")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    import model as ref  # gpt-fast's model.py

    for name, c in CONFIGS.items():
        p = random_gptfast_weights(c)
        args = ref.ModelArgs(block_size=c["block_size"], vocab_size=c["vocab_size"], n_layer=c["n_layer"],
                             n_head=c["n_head"], dim=c["dim"], intermediate_size=c["intermediate_size"],
                             n_local_heads=c["n_local_heads"], rope_base=c["rope_base"],
                             norm_eps=c["norm_eps"], rope_scaling=c["rope_scaling"])
        m = ref.Transformer(args).float().eval()
        sd = {k: v.clone() for k, v in p.items()}
        m.load_state_dict(sd, strict=True)
        out = {"checksum": weights_checksum(p)}
        worst = 0.0
        with torch.no_grad():
            for j, toks in enumerate(tokens_for(c)):
                m.max_seq_length = -1
                m.setup_caches(1, c["block_size"])
                S = toks.shape[0]
                whole = m(toks.view(1, S), torch.arange(S))[0]
                # the same tokens one at a time through gpt-fast's cache
                m.max_seq_length = -1
                m.setup_caches(1, c["block_size"])
                steps = [m(toks[t].view(1, 1), torch.tensor([t]))[0, 0] for t in range(S)]
                stepped = torch.stack(steps)
                mine = plain_llama.forward(toks, p, plain_cfg(c))
                out[f"ref_whole_{j}"] = whole.contiguous()
                out[f"ref_stepped_{j}"] = stepped.contiguous()
                out[f"plain_{j}"] = mine.contiguous()
                worst = max(worst, (whole - mine).abs().max().item(), (stepped - mine).abs().max().item())
        save_file(out, os.path.join(HERE, f"{name}.safetensors"))
        print(f"{name}: max |gpt-fast - plain| = {worst:.3e}")


if __name__ == "__main__":
    main()
