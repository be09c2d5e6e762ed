"""Schedules and seams that the Llama architecture itself does not use, run through the whole engine:
a schedule entry that reads another entry's cache (`owns_cache=False`), an attention layer with a
window, a decode graph that is reused for a much longer request, and an architecture that is
registered from this file, written as a model folder and loaded by `gf.load` like any other."""
import json
import math

import pytest
import torch

import gpt_fast_b200 as gf
from gpt_fast_b200 import ops, parts
from gpt_fast_b200.config.registry import Architecture, register_architecture
from gpt_fast_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from gpt_fast_b200.engine.model import Transformer
from gpt_fast_b200.parts.residual import as_residual
from gpt_fast_b200.weights.plan import Recipe, Source, WeightPlan
import plain_llama
import plain_ops
from conftest import assert_within_bf16_noise

BACKENDS = [
    pytest.param(("cpu", torch.float32), id="cpu-standin-f32"),
    pytest.param(("cuda", torch.float32), id="cuda-f32", marks=pytest.mark.gpu),
    pytest.param(("cuda", torch.bfloat16), id="cuda-bf16", marks=pytest.mark.gpu),
]


@pytest.fixture(params=BACKENDS)
def backend(request):
    device, dtype = request.param
    prev = ops.use_kernels(plain_ops.PlainOps()) if device == "cpu" else None
    yield device, dtype
    if device == "cpu":
        ops.use_kernels(prev)


def rnd(*shape, scale=1.0, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def judge(got, want, emu, dtype, where):
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=1e-4, atol=2e-5, msg=lambda m: f"{where}\n{m}")
    else:
        assert_within_bf16_noise(got, want, emu, where)


# ---- a plain restatement of attention layers with a window and with a cache read from another run ----------------

def windowed_attention(q, k, v, n_head, n_kv, window):
    """`plain_llama.causal_attention` with the keys further back than `window` places masked too:
    key j is visible to the query at place p iff p - window < j <= p."""
    S, H, d = q.shape
    rep = n_head // n_kv
    kh = k.repeat_interleave(rep, dim=1).transpose(0, 1).float()
    vh = v.repeat_interleave(rep, dim=1).transpose(0, 1).float()
    scores = q.transpose(0, 1).float() @ kh.transpose(1, 2) / math.sqrt(d)
    place = torch.arange(S)
    seen = place[None, :] <= place[:, None]
    if window:
        seen &= place[None, :] > place[:, None] - window
    p = torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)
    return (p @ vh).transpose(0, 1).reshape(S, H * d)


def schedule_plain(tokens, P, spec, geo, act=None):
    """The model of `schedule_spec` on one whole sequence.  geo: (n_head, n_kv, head_dim, rope base)."""
    H, G, d, base = geo
    R = plain_llama.rounded
    S = len(tokens)
    x = P["embed.weight"].float()[tokens]
    cos, sin = plain_llama.rope_angles(torch.arange(S), plain_llama.rope_frequencies(d, base))
    kept = {}
    for e in spec.schedule:
        pre = f"layers.{e.layer}."
        window = spec.layers[e.layer].parts["mixer"].params.get("window")
        h = plain_llama.rms_norm(x, P[pre + "mixer_norm.weight"].float(), 1e-5, act)
        q = R(plain_llama.apply_rope((h @ P[pre + "mixer.wq"].float().T).view(S, H, d), cos, sin), act)
        if e.owns_cache:
            k = R(plain_llama.apply_rope((h @ P[pre + "mixer.wk"].float().T).view(S, G, d), cos, sin), act)
            v = R((h @ P[pre + "mixer.wv"].float().T).view(S, G, d), act)
            kept[e.cache] = (k, v)
        else:
            k, v = kept[e.cache]                     # what the owner of this cache entry wrote in the same step
        x = x + R(windowed_attention(q, k, v, H, G, window), act) @ P[pre + "mixer.wo"].float().T
        f = plain_llama.rms_norm(x, P[pre + "ffn_norm.weight"].float(), 1e-5, act)
        x = x + plain_llama.feed_forward(f, P[pre + "feed_forward.w1"].float(), P[pre + "feed_forward.w2"].float(),
                                         P[pre + "feed_forward.w3"].float(), act)
    return plain_llama.rms_norm(x, P["final_norm.weight"].float(), 1e-5, act) @ P["head.weight"].float().T


def schedule_spec(dim, H, G, d, base, window, vocab=97):
    norm = PartSpec("rmsnorm", dict(dim=dim, eps=1e-5))
    rope = PartSpec("rope", dict(head_dim=d, base=base))
    ff = PartSpec("swiglu", dict(dim=dim, hidden=160))

    def layer(win):
        return LayerSpec("prenorm", dict(mixer=PartSpec("attention", dict(dim=dim, n_head=H, n_kv=G, head_dim=d, window=win)),
                                         feed_forward=ff, mixer_norm=norm, ffn_norm=norm), rope)
    # layer 0 writes cache entry 0; layer 1 (other weights) only READS entry 0; layer 2 has a window and its own
    # entry; layer 1 runs once more at the end, again on entry 0, across the windowed layer
    return ModelSpec("scheduled", dim, vocab, [layer(None), layer(None), layer(window)],
                     [ScheduleEntry(0, 0), ScheduleEntry(1, 0, owns_cache=False), ScheduleEntry(2, 1),
                      ScheduleEntry(1, 0, owns_cache=False)], norm, max_position=512)


def random_params(model, seed):
    P = {}
    for i, (name, ps) in enumerate(sorted(model.param_specs().items())):
        t = rnd(*ps.shape, scale=0.05, seed=seed + i)
        P[name] = (1 + t if ps.role == "vector" else t).bfloat16().float()
    model.load_params({k: v.to(model.dtype if model.param_specs()[k].role == "matrix" else torch.float32).to(model.device)
                       for k, v in P.items()})
    return P


@pytest.mark.parametrize("geometry", [
    pytest.param((192, 4, 2, 128, 10000.0, 40), id="head128-fused-kernels"),
    pytest.param((144, 6, 2, 24, 500000.0, 40), id="head24-generic-kernels"),
    pytest.param((128, 8, 1, 64, 10000.0, 70), id="head64-window-over-a-page-edge"),
])
def test_shared_cache_and_window_whole_stepped_and_in_the_decode_graph(backend, geometry):
    device, dtype = backend
    dim, H, G, d, base, window = geometry
    spec = schedule_spec(dim, H, G, d, base, window)
    model = Transformer(spec, dtype, device)
    P = random_params(model, 300)
    assert sorted(model.cache_needs()) == [0, 1]                 # the reader asks for no cache of its own
    geo = (H, G, d, base)
    g = torch.Generator().manual_seed(6)
    seqs = [torch.randint(0, spec.vocab_size, (n,), generator=g).tolist() for n in (150, 40, 77)]
    want = [schedule_plain(s, P, spec, geo) for s in seqs]
    emu = [schedule_plain(s, P, spec, geo, act=torch.bfloat16) for s in seqs] if dtype == torch.bfloat16 else want
    tail = 32
    with torch.no_grad():
        cache = model.new_cache(max_tokens=3 * 192)
        st = gf.Stepper(model, cache)
        # whole, as one batch of unequal lengths
        slots = cache.begin(3)
        whole = st.step(slots, seqs, "all").cpu()
        cache.end(slots)
        o = 0
        for i, s in enumerate(seqs):
            judge(whole[o:o + len(s)], want[i], emu[i], dtype, f"whole, sequence {i}")
            o += len(s)
        # heads in one step, then the last 32 tokens one by one: eagerly, and through the captured decode step
        for use_graph in ([False, True] if device == "cuda" else [False]):
            slots = cache.begin(3)
            for s_, q in zip(slots, seqs):
                cache.reserve(s_, len(q))
            st.step(slots, [s[:-tail] for s in seqs], "none")
            dec = gf.DecodeBatch(st, slots, use_graph)
            rows = [[] for _ in seqs]
            for k in range(tail):
                dec.tokens.copy_(torch.tensor([s[len(s) - tail + k] for s in seqs], dtype=torch.int32))
                out = dec.run().cpu()
                for i in range(3):
                    rows[i].append(out[i].clone())
            st.check()
            cache.end(slots)
            assert use_graph == (dec.graph is not None)
            for i, s in enumerate(seqs):
                judge(torch.stack(rows[i]), want[i][-tail:], emu[i][-tail:], dtype,
                      f"last {tail} one by one ({'graph' if use_graph else 'eager'}), sequence {i}")
        # from the very first token one by one on used slots and pages: with one, two, three keys in all, the key
        # that the owner stored in this very step carries most of the reader's answer, so a reader that copied its
        # page before the owner's store landed would be off by the size of the answer, not by noise
        slots = cache.begin(2)
        rows = [st.step([slots[1]], [[t]], "last")[0].cpu() for t in seqs[1]]
        cache.end(slots)
        judge(torch.stack(rows), want[1], emu[1], dtype, "from the first token, one by one, on a used slot")
        assert cache.slots.n_free == cache.n_slots and cache.pages_free == cache.n_pages


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_kept_cache_and_its_decode_graphs_serve_a_much_longer_request_later(tmp_path, dtype):
    """generate() keeps the decode steps it captured on the cache.  The first call's sequences are short (one
    slice per sequence in the decode attention); the second call, on the same cache and slots, has prompts a
    hundred times longer (several slices), across many pages that the first call never touched.  Its tokens are
    judged against the plain implementation, not against another run of the library."""
    cfg = gf.config_from_name("llama-3.1-8b")
    cfg.update(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, intermediate_size=320,
               num_hidden_layers=2, vocab_size=160, max_position_embeddings=2048)
    folder = gf.write_model_folder(str(tmp_path / "m"), cfg, seed=17)
    p, pc = plain_llama.load_folder(folder)
    g = torch.Generator().manual_seed(12)
    short = [torch.randint(0, 160, (n,), generator=g).tolist() for n in (6, 9)]
    long = [torch.randint(0, 160, (n,), generator=g).tolist() for n in (700, 1100)]
    model = gf.load(folder, dtype=dtype, device="cuda")
    cache = model.new_cache(max_tokens=2 * 1152, max_seqs=2, max_seq_len=1152)
    n_new = 6
    first, _ = gf.generate(model, short, n_new, temperature=0.0, cache=cache)
    stepper = gf.Stepper.of(model, cache)
    assert len(stepper._decode_batches) == 1
    again, _ = gf.generate(model, long, n_new, temperature=0.0, cache=cache)
    assert gf.Stepper.of(model, cache) is stepper and len(stepper._decode_batches) == 2     # a step of its own for the longer reach
    repeat, _ = gf.generate(model, short, n_new, temperature=0.0, cache=cache)
    assert repeat == first and len(stepper._decode_batches) == 2                            # and the short one is found again
    for pr, seq in zip(long + short, again + repeat):
        assert seq[:len(pr)] == pr and len(seq) == len(pr) + n_new
        logits = plain_llama.forward(seq[:-1], p, pc)
        if dtype == "float32":
            margin = [1e-4] * len(seq)
        else:
            noise = plain_llama.forward(seq[:-1], p, pc, act=torch.bfloat16) - logits
            margin = [4 * float(noise[j].abs().max()) for j in range(len(seq) - 1)]
        for j in range(len(pr) - 1, len(seq) - 1):
            assert logits[j, seq[j + 1]] >= logits[j].max() - margin[j], f"prompt of {len(pr)}: token {j + 1 - len(pr)}"


# ---- a whole architecture registered from here: config.json -> spec -> weight plan -> folder -> gf.load -> steps ----

class SharedNormBlock:
    """x += mixer(n(x)) + feed_forward(n(x)) with ONE norm for both branches: an arrangement with other roles
    than the built-in pre-norm block."""
    roles = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    def __init__(self, parts, dim, dtype):
        self.p, self.dim, self.dtype = parts, dim, dtype

    def parts(self):
        return dict(self.p)

    def cache_needs(self):
        return self.p["mixer"].cache_needs()

    def forward(self, x, batch, view, append=True):
        x = as_residual(x)
        h = torch.empty(x.x.shape[0], self.dim, dtype=self.dtype, device=x.x.device)
        self.p["norm"].forward(x, h)
        self.p["mixer"].forward(h, batch, view, residual=x, append=append)
        self.p["feed_forward"].forward(h, residual=x)


def toy_arch_parse(cfg):
    need = ("width", "heads", "kv_heads", "head_size", "inner", "depth", "vocab", "eps", "theta", "longest", "embed_scale",
            "logit_cap")
    missing = [k for k in need if k not in cfg]
    if missing:
        raise gf.ConfigError(f"config.json: keys {missing} are required")
    return {k: cfg[k] for k in need}


def toy_arch_spec(a):
    norm = PartSpec("rmsnorm", dict(dim=a["width"], eps=a["eps"]))
    layer = LayerSpec("shared_norm", dict(
        norm=norm,
        mixer=PartSpec("attention", dict(dim=a["width"], n_head=a["heads"], n_kv=a["kv_heads"], head_dim=a["head_size"])),
        feed_forward=PartSpec("swiglu", dict(dim=a["width"], hidden=a["inner"]))),
        PartSpec("rope", dict(head_dim=a["head_size"], base=a["theta"], pairing="half")))
    return ModelSpec("parallel-toy", a["width"], a["vocab"], [layer] * a["depth"],
                     [ScheduleEntry(i, i) for i in range(a["depth"])], norm, tie_embeddings=True, max_position=a["longest"],
                     embed_scale=a["embed_scale"], logit_cap=a["logit_cap"])


def toy_arch_plan(a):
    D, H, G, d, I, V = a["width"], a["heads"], a["kv_heads"], a["head_size"], a["inner"], a["vocab"]
    r = [Recipe("embed.weight", [Source("wte", (V, D))]), Recipe("final_norm.weight", [Source("ln_f", (D,), "norm")])]
    for i in range(a["depth"]):
        s, t = f"h.{i}.", f"layers.{i}."
        r += [Recipe(t + "mixer.wq", [Source(s + "q", (H * d, D))]), Recipe(t + "mixer.wk", [Source(s + "k", (G * d, D))]),
              Recipe(t + "mixer.wv", [Source(s + "v", (G * d, D))]), Recipe(t + "mixer.wo", [Source(s + "o", (D, H * d))]),
              Recipe(t + "feed_forward.w1", [Source(s + "gate", (I, D))]), Recipe(t + "feed_forward.w3", [Source(s + "up", (I, D))]),
              Recipe(t + "feed_forward.w2", [Source(s + "down", (D, I))]), Recipe(t + "norm.weight", [Source(s + "ln", (D,), "norm")])]
    return WeightPlan(recipes=r, aliases={"head.weight": "embed.weight"})


def rope_half(x, cos, sin):
    """Rotation of the pairs (i, i + d/2) (the checkpoint layout this toy keeps, unlike gpt-fast's interleaved pairs)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half].float(), x[..., half:].float()
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def toy_arch_plain(tokens, T, a, act=None):
    R = plain_llama.rounded
    D, H, G, d = a["width"], a["heads"], a["kv_heads"], a["head_size"]
    S = len(tokens)
    x = T["wte"].float()[tokens] * a["embed_scale"]
    cos, sin = plain_llama.rope_angles(torch.arange(S), plain_llama.rope_frequencies(d, a["theta"]))
    for i in range(a["depth"]):
        s = f"h.{i}."
        h = plain_llama.rms_norm(x, T[s + "ln"].float(), a["eps"], act)
        q = R(rope_half((h @ T[s + "q"].float().T).view(S, H, d), cos, sin), act)
        k = R(rope_half((h @ T[s + "k"].float().T).view(S, G, d), cos, sin), act)
        v = R((h @ T[s + "v"].float().T).view(S, G, d), act)
        y = R(windowed_attention(q, k, v, H, G, None), act) @ T[s + "o"].float().T
        x = x + y + plain_llama.feed_forward(h, T[s + "gate"].float(), T[s + "down"].float(), T[s + "up"].float(), act)
    logits = plain_llama.rms_norm(x, T["ln_f"].float(), a["eps"], act) @ T["wte"].float().T
    return a["logit_cap"] * torch.tanh(logits / a["logit_cap"])


def test_an_architecture_registered_from_a_test_loads_from_its_folder_and_steps(backend, tmp_path):
    device, dtype = backend
    if "shared_norm" not in parts.BLOCKS:
        parts.register_block("shared_norm", SharedNormBlock)
        register_architecture(Architecture(name="parallel-toy", aliases=("ParallelToyLM",), parse=toy_arch_parse,
                                           build_spec=toy_arch_spec, weight_plan=toy_arch_plan))
    assert "parallel-toy" in gf.architecture_names()
    cfg = dict(model_type="parallel-toy", width=80, heads=5, kv_heads=5, head_size=16, inner=136, depth=2, vocab=89,
               eps=1e-6, theta=3000.0, longest=160, embed_scale=8.0, logit_cap=0.5)
    folder = gf.write_model_folder(str(tmp_path / "toy"), cfg, seed=21)
    with open(tmp_path / "toy" / "config.json") as f:
        assert json.load(f)["model_type"] == "parallel-toy"
    from safetensors.torch import load_file
    T = load_file(str(tmp_path / "toy" / "model.safetensors"))
    assert set(T) == {"wte", "ln_f"} | {f"h.{i}.{n}" for i in range(2) for n in ("q", "k", "v", "o", "gate", "up", "down", "ln")}
    model = gf.load(folder, dtype=dtype, device=device)
    assert model.spec.architecture == "parallel-toy" and model.head_weight.data_ptr() == model.embed_weight.data_ptr()
    a = toy_arch_parse(cfg)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, 89, (n,), generator=g).tolist() for n in (70, 9)]
    want = [toy_arch_plain(s, T, a) for s in seqs]
    emu = [toy_arch_plain(s, T, a, act=torch.bfloat16) for s in seqs]
    with torch.no_grad():
        cache = model.new_cache(max_tokens=192)
        st = gf.Stepper(model, cache)
        slots = cache.begin(2)
        heads = [len(s) - 4 for s in seqs]
        out = st.step(slots, [s[:h] for s, h in zip(seqs, heads)], "all").cpu()
        rows = [list(out[:heads[0]]), list(out[heads[0]:])]
        for k in range(4):
            out = st.step(slots, [[s[h + k]] for s, h in zip(seqs, heads)], "last").cpu()
            for i in range(2):
                rows[i].append(out[i])
        st.check()
        cache.end(slots)
    for i in range(2):
        judge(torch.stack(rows[i]), want[i], emu[i], dtype, f"sequence {i}")
    if device == "cuda":                       # generation runs on it like on any model
        out, stats = gf.generate(model, [seqs[1]], 5, temperature=0.0)
        assert len(out[0]) == len(seqs[1]) + 5 and stats.decode_steps == 4
    # the loader's one error names this architecture's tensors
    from safetensors.torch import save_file
    del T["h.1.up"]
    T["h.1.extra"] = torch.zeros(3)
    save_file(T, str(tmp_path / "toy" / "model.safetensors"))
    with pytest.raises(gf.WeightError) as e:
        gf.load(folder, dtype=dtype, device=device)
    assert "h.1.up" in str(e.value) and "h.1.extra" in str(e.value)
