"""The Llama 2/3 dense decoder as data: which parts each layer has, in which
order layers run, and which checkpoint tensors fill which parameter.

The formulas live in the parts; this file only wires them as gpt-fast's
model.py does (model.py:102-164): token embedding, n_layer pre-norm blocks of
(RMSNorm, attention with RoPE, RMSNorm, SwiGLU), final RMSNorm, output linear.
Tensor names and the q/k row permutation follow gpt-fast's checkpoint
conversion (scripts/convert_hf_checkpoint.py:58-115).
"""
from ..config.args import ModelArgs
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..weights.plan import Recipe, Source, WeightPlan


def build_spec(a: ModelArgs) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(dim=a.dim, eps=a.norm_eps))
    rope = PartSpec("rope", dict(head_dim=a.head_dim, base=a.rope_base, scaling=a.rope_scaling,
                                 pairing="interleaved"))
    layer = LayerSpec(
        block="prenorm",
        parts=dict(mixer=PartSpec("attention", dict(dim=a.dim, n_head=a.n_head, n_kv=a.n_local_heads,
                                                    head_dim=a.head_dim, window=None)),
                   feed_forward=PartSpec("swiglu", dict(dim=a.dim, hidden=a.intermediate_size)),
                   mixer_norm=norm, ffn_norm=norm),
        position=rope,
    )
    spec = ModelSpec(
        architecture="llama", dim=a.dim, vocab_size=a.vocab_size,
        layers=[layer] * a.n_layer,
        schedule=[ScheduleEntry(layer=i, cache=i) for i in range(a.n_layer)],
        final_norm=norm, tie_embeddings=a.tie_embeddings, max_position=a.block_size,
        stop_tokens=tuple(a.eos_token_ids), bos_token=a.bos_token_id,
    )
    spec.validate()
    return spec


def interleave_rotary_rows(n_heads: int, head_dim: int):
    """Rows of a q or k projection stored for half-split rotary pairs
    (i, i + d/2) reordered for interleaved pairs (2i, 2i+1): new row
    h*d + 2i + j is old row h*d + j*d/2 + i
    (scripts/convert_hf_checkpoint.py:75-81)."""
    def combine(w):
        cols = w.shape[1]
        return w.view(n_heads, 2, head_dim // 2, cols).transpose(1, 2).reshape(n_heads * head_dim, cols)
    return combine


def half_split_rotary_rows(n_heads: int, head_dim: int):
    """Inverse of `interleave_rotary_rows`: the recipe's `split`, used when a model is written to a folder."""
    def split(w):
        cols = w.shape[1]
        return [w.view(n_heads, head_dim // 2, 2, cols).transpose(1, 2).reshape(n_heads * head_dim, cols)]
    return split


def weight_plan(a: ModelArgs) -> WeightPlan:
    D, H, G, d, I, V = a.dim, a.n_head, a.n_local_heads, a.head_dim, a.intermediate_size, a.vocab_size
    r = [Recipe("embed.weight", [Source("model.embed_tokens.weight", (V, D))]),
         Recipe("final_norm.weight", [Source("model.norm.weight", (D,), "norm")])]
    for i in range(a.n_layer):
        s, t = f"model.layers.{i}.", f"layers.{i}."
        r += [
            Recipe(t + "mixer.wq", [Source(s + "self_attn.q_proj.weight", (H * d, D))], interleave_rotary_rows(H, d),
                   half_split_rotary_rows(H, d)),
            Recipe(t + "mixer.wk", [Source(s + "self_attn.k_proj.weight", (G * d, D))], interleave_rotary_rows(G, d),
                   half_split_rotary_rows(G, d)),
            Recipe(t + "mixer.wv", [Source(s + "self_attn.v_proj.weight", (G * d, D))]),
            Recipe(t + "mixer.wo", [Source(s + "self_attn.o_proj.weight", (D, H * d))]),
            Recipe(t + "feed_forward.w1", [Source(s + "mlp.gate_proj.weight", (I, D))]),
            Recipe(t + "feed_forward.w3", [Source(s + "mlp.up_proj.weight", (I, D))]),
            Recipe(t + "feed_forward.w2", [Source(s + "mlp.down_proj.weight", (D, I))]),
            Recipe(t + "mixer_norm.weight", [Source(s + "input_layernorm.weight", (D,), "norm")]),
            Recipe(t + "ffn_norm.weight", [Source(s + "post_attention_layernorm.weight", (D,), "norm")]),
        ]
    plan = WeightPlan(recipes=r, ignored=(r"model\.layers\.\d+\.self_attn\.rotary_emb\.inv_freq",))
    if a.tie_embeddings:
        plan.aliases["head.weight"] = "embed.weight"
        plan.forbidden["lm_head.weight"] = "config.json sets tie_word_embeddings, so the output shares the embedding"
    else:
        plan.recipes.append(Recipe("head.weight", [Source("lm_head.weight", (V, D))]))
    return plan


LLAMA = register_architecture(Architecture(
    name="llama", aliases=("LlamaForCausalLM",),
    parse=ModelArgs.from_json, build_spec=build_spec, weight_plan=weight_plan,
))
