"""Plain, slow Llama 2/3 decoder used as the oracle of the test-suite.

Whole sequences only: no cache, no packing, no kernels, one function per part.
It shares no code with the package under test and runs on the CPU.  Every
function restates a formula of pytorch-labs/gpt-fast (cited as file:line of
that project).  `tests/golden/make_golden.py` compared it once with gpt-fast's
own `model.py` on tiny random models; the outputs are kept under
`tests/golden/`.

Tensors are named as in gpt-fast's checkpoints after conversion
(`tok_embeddings.weight`, `layers.N.attention.wqkv.weight`, ...), i.e. with
q, k and v fused and q/k rows already in interleaved-pair order.
"""
import math

import torch


def rounded(x, act):
    """Round-trip through the activation type `act` (None: leave as is).  With
    act = bfloat16 the functions below round where the library's bfloat16 path
    stores an activation: norm output, qkv, rotated q and k, attention output,
    SwiGLU output; sums, softmax and the residual stream stay 32-bit."""
    return x if act is None else x.to(act).to(x.dtype)


def rms_norm(x, weight, eps, act=None):
    """model.py:236-241: statistics in 32-bit, cast back, then the weight."""
    x32 = x.float()
    n = x32 * torch.rsqrt(torch.mean(x32 * x32, dim=-1, keepdim=True) + eps)
    return rounded(n.type_as(x) * weight.to(x.dtype), act)


def rope_frequencies(head_dim, base, rope_scaling=None):
    """model.py:271-273 (base frequencies) and model.py:244-263 (llama3 rule)."""
    freqs = 1.0 / (base ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    if rope_scaling is None:
        return freqs
    factor = rope_scaling["factor"]
    low = rope_scaling["low_freq_factor"]
    high = rope_scaling["high_freq_factor"]
    old_len = rope_scaling["original_max_position_embeddings"]
    low_wavelen = old_len / low
    high_wavelen = old_len / high
    out = []
    for f in freqs:
        wavelen = 2 * math.pi / f
        if wavelen < high_wavelen:
            out.append(f)
        elif wavelen > low_wavelen:
            out.append(f / factor)
        else:
            smooth = (old_len / wavelen - low) / (high - low)
            out.append((1 - smooth) * f / factor + smooth * f)
    return torch.tensor(out, dtype=freqs.dtype)


def rope_angles(positions, freqs):
    """model.py:274-277: angle[p, i] = p * f_i, as (cos, sin) in 32-bit."""
    ang = torch.outer(positions.to(torch.int64), freqs)
    cis = torch.polar(torch.ones_like(ang), ang)
    return cis.real, cis.imag


def apply_rope(x, cos, sin):
    """model.py:281-293: rotation of the pairs (2i, 2i+1).  x: [S, heads, d]."""
    x32 = x.float().reshape(*x.shape[:-1], -1, 2)
    c = cos[:, None, :]
    s = sin[:, None, :]
    out = torch.stack(
        [x32[..., 0] * c - x32[..., 1] * s, x32[..., 1] * c + x32[..., 0] * s], dim=-1
    )
    return out.flatten(-2).type_as(x)


def causal_attention(q, k, v, n_head, n_kv):
    """model.py:209-211: query head h reads key/value head h // (H/G); key j is
    visible to the query at place p iff j <= p; scores are scaled by
    1/sqrt(head_dim); softmax in 32-bit.  q: [S, H, d], k, v: [S, G, d]."""
    S, H, d = q.shape
    rep = n_head // n_kv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    qh = q.transpose(0, 1).float()
    kh = k.transpose(0, 1).float()
    vh = v.transpose(0, 1).float()
    scores = qh @ kh.transpose(1, 2) / math.sqrt(d)
    mask = torch.tril(torch.ones(S, S, dtype=torch.bool))
    scores = scores.masked_fill(~mask, float("-inf"))
    p = torch.softmax(scores, dim=-1)
    y = p @ vh
    return y.transpose(0, 1).reshape(S, H * d).type_as(q)


def attention(x, wqkv, wo, cos, sin, n_head, n_kv, head_dim, act=None):
    """model.py:191-216 without the cache: x [S, D] -> [S, D]."""
    S = x.shape[0]
    qkv = x @ wqkv.T
    q, k, v = qkv.split([n_head * head_dim, n_kv * head_dim, n_kv * head_dim], dim=-1)
    q = rounded(apply_rope(q.view(S, n_head, head_dim), cos, sin), act)
    k = rounded(apply_rope(k.view(S, n_kv, head_dim), cos, sin), act)
    v = rounded(v.view(S, n_kv, head_dim), act)
    y = rounded(causal_attention(q, k, v, n_head, n_kv), act)
    return y @ wo.T


def feed_forward(x, w1, w2, w3, act=None):
    """model.py:226-227: w2(silu(w1 x) * w3 x)."""
    return rounded(torch.nn.functional.silu(x @ w1.T) * (x @ w3.T), act) @ w2.T


def block(x, p, prefix, cos, sin, cfg, act=None):
    """model.py:161-164: h = x + attn(norm(x)); out = h + ffn(norm(h))."""
    a = rms_norm(x, p[prefix + "attention_norm.weight"], cfg["norm_eps"], act)
    h = x + attention(a, p[prefix + "attention.wqkv.weight"], p[prefix + "attention.wo.weight"],
                      cos, sin, cfg["n_head"], cfg["n_local_heads"], cfg["head_dim"], act)
    f = rms_norm(h, p[prefix + "ffn_norm.weight"], cfg["norm_eps"], act)
    return h + feed_forward(f, p[prefix + "feed_forward.w1.weight"],
                            p[prefix + "feed_forward.w2.weight"], p[prefix + "feed_forward.w3.weight"], act)


def forward(tokens, p, cfg, act=None):
    """model.py:136-146 for one whole sequence: token ids [S] -> logits [S, V].
    act=torch.bfloat16 rounds the activations where the library's bfloat16 path stores them.

    cfg keys: n_layer, n_head, n_local_heads, head_dim, norm_eps, rope_base,
    rope_scaling.  p: tensors by gpt-fast name; `output.weight` may be the
    same tensor as `tok_embeddings.weight` (tied)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    freqs = rope_frequencies(cfg["head_dim"], cfg["rope_base"], cfg.get("rope_scaling"))
    cos, sin = rope_angles(torch.arange(tokens.shape[0]), freqs)
    x = p["tok_embeddings.weight"][tokens]
    for i in range(cfg["n_layer"]):
        x = block(x, p, f"layers.{i}.", cos, sin, cfg, act)
    x = rms_norm(x, p["norm.weight"], cfg["norm_eps"], act)
    return x @ p["output.weight"].T


# ---- sampling (generate.py:40-57) -------------------------------------------

def logits_to_probs(logits, temperature=1.0, top_k=None):
    """generate.py:44-52: divide by max(T, 1e-5); keep what is >= the k-th
    largest value (ties kept); softmax."""
    logits = logits / max(temperature, 1e-5)
    if top_k is not None:
        v, _ = torch.topk(logits, min(top_k, logits.size(-1)))
        pivot = v.select(-1, -1).unsqueeze(-1)
        logits = torch.where(logits < pivot, -float("inf"), logits)
    return torch.softmax(logits, dim=-1)


def exponential_race(probs, noise):
    """generate.py:40-42: argmax(probs / q) with q ~ Exp(1) given as `noise`."""
    return torch.argmax(probs / noise, dim=-1)


def greedy_generate(prompt, n_new, p, cfg, stop_tokens=()):
    """Greedy continuation by re-running the whole sequence for each token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(seq, p, cfg)
        nxt = int(torch.argmax(logits[-1].float()))
        out.append(nxt)
        seq.append(nxt)
        if nxt in stop_tokens:
            break
    return out


# ---- checkpoint names (scripts/convert_hf_checkpoint.py:58-115) --------------

def hf_to_gptfast(hf, n_layer, n_head, n_kv, head_dim, tied):
    """Rename config.json-style tensors to gpt-fast's names, permute q/k rows
    from half-split to interleaved pairs (convert_hf_checkpoint.py:75-81) and
    fuse q, k, v (convert_hf_checkpoint.py:105-115)."""
    def permute(w, heads):
        dim = w.shape[1]
        return w.view(heads, 2, head_dim // 2, dim).transpose(1, 2).reshape(heads * head_dim, dim)

    p = {"tok_embeddings.weight": hf["model.embed_tokens.weight"],
         "norm.weight": hf["model.norm.weight"]}
    p["output.weight"] = p["tok_embeddings.weight"] if tied else hf["lm_head.weight"]
    for i in range(n_layer):
        s, d = f"model.layers.{i}.", f"layers.{i}."
        q = permute(hf[s + "self_attn.q_proj.weight"], n_head)
        k = permute(hf[s + "self_attn.k_proj.weight"], n_kv)
        v = hf[s + "self_attn.v_proj.weight"]
        p[d + "attention.wqkv.weight"] = torch.cat([q, k, v])
        p[d + "attention.wo.weight"] = hf[s + "self_attn.o_proj.weight"]
        p[d + "feed_forward.w1.weight"] = hf[s + "mlp.gate_proj.weight"]
        p[d + "feed_forward.w3.weight"] = hf[s + "mlp.up_proj.weight"]
        p[d + "feed_forward.w2.weight"] = hf[s + "mlp.down_proj.weight"]
        p[d + "attention_norm.weight"] = hf[s + "input_layernorm.weight"]
        p[d + "ffn_norm.weight"] = hf[s + "post_attention_layernorm.weight"]
    return p


def load_folder(folder, dtype=torch.float32):
    """Read a model folder (config.json + model.safetensors) for the oracle:
    returns (p, cfg) with every tensor cast to `dtype`."""
    import json
    import os
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    hf = {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    n_head = c["num_attention_heads"]
    n_kv = c.get("num_key_value_heads", n_head)
    head_dim = c["hidden_size"] // n_head
    tied = bool(c.get("tie_word_embeddings", False))
    rs = c.get("rope_scaling")
    cfg = dict(n_layer=c["num_hidden_layers"], n_head=n_head, n_local_heads=n_kv, head_dim=head_dim,
               norm_eps=c.get("rms_norm_eps", 1e-5), rope_base=c.get("rope_theta", 10000.0),
               rope_scaling=None if rs is None else {k: rs[k] for k in (
                   "factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")},
               vocab_size=c["vocab_size"])
    return hf_to_gptfast(hf, cfg["n_layer"], n_head, n_kv, head_dim, tied), cfg
