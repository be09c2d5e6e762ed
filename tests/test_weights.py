"""Weights by tensor name: the loader's mapping, precision rules and its one error."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import gpt_fast_b200 as gf
from gpt_fast_b200.architectures.llama import half_split_rotary_rows, interleave_rotary_rows
from gpt_fast_b200.config.registry import architecture_for, read_config
from gpt_fast_b200.engine.model import Transformer
from gpt_fast_b200.weights.loader import SafetensorsCheckpoint, load_parameters
import plain_llama


def load_cpu(folder, dtype=torch.float32):
    cfg = read_config(folder)
    arch = architecture_for(cfg)
    args = arch.parse(cfg)
    model = Transformer(arch.build_spec(args), dtype, "cpu")
    params = load_parameters(arch.weight_plan(args), SafetensorsCheckpoint(folder), model.param_specs(), dtype, "cpu")
    model.load_params(params)
    return model, params


def rewrite(folder, tmp_path, edit):
    t = load_file(os.path.join(folder, "model.safetensors"))
    edit(t)
    out = tmp_path / "edited"
    out.mkdir()
    save_file(t, str(out / "model.safetensors"))
    (out / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    return str(out)


def test_names_permutation_and_fusing_match_gptfasts_converter(tiny_folders):
    for name in ("tiny-a", "tiny-b"):
        model, params = load_cpu(tiny_folders[name])
        p, cfg = plain_llama.load_folder(tiny_folders[name])          # convert_hf_checkpoint.py's map, restated
        for i, b in enumerate(model.blocks):
            assert torch.equal(b.mixer.wqkv, p[f"layers.{i}.attention.wqkv.weight"])
            assert torch.equal(b.mixer.wo, p[f"layers.{i}.attention.wo.weight"])
            assert torch.equal(b.feed_forward.w13[0::2], p[f"layers.{i}.feed_forward.w1.weight"])
            assert torch.equal(b.feed_forward.w13[1::2], p[f"layers.{i}.feed_forward.w3.weight"])
            assert torch.equal(b.feed_forward.w2, p[f"layers.{i}.feed_forward.w2.weight"])
            assert torch.equal(b.mixer_norm.weight.float(), p[f"layers.{i}.attention_norm.weight"])
        assert torch.equal(model.embed_weight, p["tok_embeddings.weight"])


def test_rotary_row_permutation_is_the_stated_index_map():
    H, d = 3, 8
    w = torch.arange(H * d, dtype=torch.float32)[:, None].repeat(1, 5)
    out = interleave_rotary_rows(H, d)(w)
    for h in range(H):
        for i in range(d // 2):
            for j in range(2):
                assert out[h * d + 2 * i + j, 0] == h * d + j * d // 2 + i
    assert torch.equal(half_split_rotary_rows(H, d)(out)[0], w)


def test_tied_output_is_one_buffer_and_untied_is_two(tiny_folders):
    tied, _ = load_cpu(tiny_folders["tiny-b"])
    assert tied.head_weight.data_ptr() == tied.embed_weight.data_ptr()
    untied, _ = load_cpu(tiny_folders["tiny-a"])
    assert untied.head_weight.data_ptr() != untied.embed_weight.data_ptr()


def test_precision_rules(tiny_folders):
    # tiny-a stores its norm weights in 32-bit: they stay so in a bfloat16 model; matrices are bfloat16
    m, _ = load_cpu(tiny_folders["tiny-a"], torch.bfloat16)
    assert m.blocks[0].mixer_norm.weight.dtype == torch.float32 and m.final_norm.weight.dtype == torch.float32
    assert m.blocks[0].mixer.wqkv.dtype == torch.bfloat16 and m.embed_weight.dtype == torch.bfloat16
    # tiny-b stores them in bfloat16: kept in a bfloat16 model, widened exactly in a 32-bit model
    m, _ = load_cpu(tiny_folders["tiny-b"], torch.bfloat16)
    assert m.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    m32, _ = load_cpu(tiny_folders["tiny-b"], torch.float32)
    assert m32.blocks[0].mixer.wo.dtype == torch.float32
    assert torch.equal(m32.blocks[0].mixer.wo, m.blocks[0].mixer.wo.float())


def test_one_error_lists_everything_wrong(tiny_folders, tmp_path):
    def edit(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(4)
        t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(3, 5, dtype=torch.bfloat16)
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)          # known and dropped
    folder = rewrite(tiny_folders["tiny-a"], tmp_path, edit)
    with pytest.raises(gf.WeightError) as e:
        load_cpu(folder)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [(n, tuple(f)) for n, w, f in err.wrong_shape] == [("model.layers.0.mlp.down_proj.weight", (3, 5))]
    text = str(err)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shape", "expected (64, 172), found (3, 5)"):
        assert word in text


def test_tied_model_refuses_an_lm_head_and_untied_needs_one(tiny_folders, tmp_path):
    def add_head(t):
        t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    with pytest.raises(gf.WeightError, match="tie_word_embeddings"):
        load_cpu(rewrite(tiny_folders["tiny-b"], tmp_path, add_head))
    (tmp_path / "edited" / "model.safetensors").unlink()
    (tmp_path / "edited" / "config.json").unlink()
    (tmp_path / "edited").rmdir()
    with pytest.raises(gf.WeightError, match="lm_head.weight"):
        load_cpu(rewrite(tiny_folders["tiny-a"], tmp_path, lambda t: t.pop("lm_head.weight")))


def test_shards_and_their_errors(tiny_folders, tmp_path):
    t = load_file(os.path.join(tiny_folders["tiny-a"], "model.safetensors"))
    names = sorted(t)
    a, b = names[: len(names) // 2], names[len(names) // 2:]
    save_file({k: t[k] for k in a}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({k: t[k] for k in b}, str(tmp_path / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {**{k: "model-00001-of-00002.safetensors" for k in a},
                            **{k: "model-00002-of-00002.safetensors" for k in b}}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    (tmp_path / "config.json").write_text(open(os.path.join(tiny_folders["tiny-a"], "config.json")).read())
    sharded, _ = load_cpu(str(tmp_path))
    whole, _ = load_cpu(tiny_folders["tiny-a"])
    assert torch.equal(sharded.blocks[1].mixer.wqkv, whole.blocks[1].mixer.wqkv)
    save_file({k: t[k] for k in b + a[:1]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    with pytest.raises(gf.WeightError, match="is in both"):
        load_cpu(str(tmp_path))
    empty = tmp_path / "empty"
    empty.mkdir()
    (empty / "config.json").write_text((tmp_path / "config.json").read_text())
    with pytest.raises(gf.WeightError, match="no model.safetensors"):
        load_cpu(str(empty))


def test_random_weights_mode_is_seeded_per_tensor(tmp_path):
    a = gf.write_model_folder(str(tmp_path / "a"), "tiny-a", seed=5)
    b = gf.write_model_folder(str(tmp_path / "b"), "tiny-a", seed=5)
    c = gf.write_model_folder(str(tmp_path / "c"), "tiny-a", seed=6)
    ta, tb, tc = (load_file(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"])
    assert ta["lm_head.weight"].dtype == torch.bfloat16
    assert abs(ta["model.embed_tokens.weight"].float().std() - 0.02) < 0.002
    assert abs(ta["model.norm.weight"].float().mean() - 1.0) < 0.05
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["hidden_size"] == 64 and cfg["model_type"] == "llama"


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_a_loaded_model_written_back_is_the_same_folder(tiny_folders, tmp_path, name):
    """load -> save_folder -> load: the same tensors under the same checkpoint names (q/k rows back in half-split
    order, gate/up and q/k/v taken apart again, the tied output not written twice), bit for bit, and the same
    model parameters after loading the written folder."""
    folder = tiny_folders[name]
    model = gf.load(folder, dtype="bfloat16", device="cpu")
    out = gf.save_folder(model, str(tmp_path / "written"))
    a = load_file(os.path.join(folder, "model.safetensors"))
    b = load_file(os.path.join(out, "model.safetensors"))
    assert sorted(a) == sorted(b)
    for k in a:
        want = a[k] if a[k].dtype == torch.float32 and a[k].ndim == 1 else a[k].to(torch.bfloat16)
        assert b[k].dtype == want.dtype and torch.equal(b[k], want), k
    assert json.load(open(os.path.join(out, "config.json")))["num_hidden_layers"] == read_config(folder)["num_hidden_layers"]
    again = gf.load(out, dtype="bfloat16", device="cpu")
    pa, pb = model.export_params(), again.export_params()
    assert sorted(pa) == sorted(pb) and all(torch.equal(pa[k], pb[k]) for k in pa)
    # a model that was not made by load() cannot be written: it has no plan
    bare = Transformer(model.spec, torch.bfloat16, "cpu")
    with pytest.raises(ValueError, match="made by load"):
        gf.save_folder(bare, str(tmp_path / "bare"))
