"""Typed configuration of the Llama 2/3 dense decoder, read from the keys of the
architecture's own config.json.

Field names follow gpt-fast's `ModelArgs` (model.py:21-42); gpt-fast picks a
size by directory name and never reads config.json, so the key mapping is
this library's.  Every value comes from the file (or from the default the
file format itself implies); no size is fixed in code.
"""
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

ROPE_SCALING_KEYS = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")


class ConfigError(ValueError):
    """A config.json this library cannot run; the message names the key."""


def find_multiple(n: int, k: int) -> int:
    """Round n up to a multiple of k (gpt-fast model.py:16-19)."""
    return n if n % k == 0 else n + k - (n % k)


def _positive_int(cfg: Dict[str, Any], key: str, default=None) -> int:
    if key not in cfg or cfg[key] is None:
        if default is None:
            raise ConfigError(f"config.json: key '{key}' is required")
        return default
    v = cfg[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: '{key}' must be a positive integer, found {v!r}")
    return v


@dataclass(frozen=True)
class ModelArgs:
    block_size: int                      # max_position_embeddings
    vocab_size: int
    n_layer: int                         # num_hidden_layers
    n_head: int                          # num_attention_heads
    dim: int                             # hidden_size
    intermediate_size: int
    n_local_heads: int                   # num_key_value_heads
    head_dim: int
    rope_base: float                     # rope_theta
    norm_eps: float                      # rms_norm_eps
    rope_scaling: Optional[Dict[str, float]] = None
    tie_embeddings: bool = False         # tie_word_embeddings
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    source: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_json(cls, cfg) -> "ModelArgs":
        """Parse a config.json (path of the file, of its folder, or the dict)."""
        if isinstance(cfg, (str, os.PathLike)):
            path = os.fspath(cfg)
            if os.path.isdir(path):
                path = os.path.join(path, "config.json")
            if not os.path.isfile(path):
                raise ConfigError(f"no config.json at {path}")
            with open(path) as f:
                cfg = json.load(f)
        if not isinstance(cfg, dict):
            raise ConfigError("config.json must hold one JSON object")

        dim = _positive_int(cfg, "hidden_size")
        n_head = _positive_int(cfg, "num_attention_heads")
        n_kv = _positive_int(cfg, "num_key_value_heads", n_head)
        if dim % n_head:
            raise ConfigError(f"config.json: hidden_size {dim} is not a multiple of num_attention_heads {n_head}")
        head_dim = _positive_int(cfg, "head_dim", dim // n_head)
        if head_dim != dim // n_head:
            raise ConfigError(f"config.json: head_dim {head_dim} differs from hidden_size/num_attention_heads "
                              f"= {dim // n_head}; this decoder cannot express that")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even for rotary pairs")
        if n_head % n_kv:
            raise ConfigError(f"config.json: num_attention_heads {n_head} is not a multiple of "
                              f"num_key_value_heads {n_kv}")
        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (only 'silu')")
        for key in ("attention_bias", "mlp_bias"):
            if cfg.get(key):
                raise ConfigError(f"config.json: '{key}' is set; this decoder has no biases")

        scaling = cfg.get("rope_scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError("config.json: 'rope_scaling' must be an object or null")
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind != "llama3":
                raise ConfigError(f"config.json: rope_scaling type '{kind}' is not supported (only 'llama3')")
            missing = [k for k in ROPE_SCALING_KEYS if k not in scaling]
            if missing:
                raise ConfigError(f"config.json: rope_scaling lacks {missing}")
            scaling = {k: float(scaling[k]) for k in ROPE_SCALING_KEYS}
            if scaling["low_freq_factor"] == scaling["high_freq_factor"]:
                raise ConfigError("config.json: rope_scaling low_freq_factor equals high_freq_factor")

        eos = cfg.get("eos_token_id")
        if eos is None:
            eos_ids = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: eos_token_id must be an integer or a list of them, found {eos!r}")
        eps = cfg.get("rms_norm_eps", 1e-5)
        theta = cfg.get("rope_theta", 10000.0)
        if not isinstance(eps, (int, float)) or eps <= 0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, found {eps!r}")
        if not isinstance(theta, (int, float)) or theta <= 0:
            raise ConfigError(f"config.json: rope_theta must be positive, found {theta!r}")

        return cls(
            block_size=_positive_int(cfg, "max_position_embeddings"),
            vocab_size=_positive_int(cfg, "vocab_size"),
            n_layer=_positive_int(cfg, "num_hidden_layers"),
            n_head=n_head, dim=dim,
            intermediate_size=_positive_int(cfg, "intermediate_size"),
            n_local_heads=n_kv, head_dim=head_dim,
            rope_base=float(theta), norm_eps=float(eps), rope_scaling=scaling,
            tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids, bos_token_id=cfg.get("bos_token_id"),
            source=dict(cfg),
        )

    def to_json(self) -> Dict[str, Any]:
        """The config.json that parses back to this configuration."""
        out = dict(self.source)
        out.update(
            model_type=out.get("model_type", "llama"),
            architectures=out.get("architectures", ["LlamaForCausalLM"]),
            max_position_embeddings=self.block_size, vocab_size=self.vocab_size,
            num_hidden_layers=self.n_layer, num_attention_heads=self.n_head, hidden_size=self.dim,
            intermediate_size=self.intermediate_size, num_key_value_heads=self.n_local_heads,
            head_dim=self.head_dim, rope_theta=self.rope_base, rms_norm_eps=self.norm_eps,
            tie_word_embeddings=self.tie_embeddings, hidden_act="silu",
        )
        out["rope_scaling"] = None if self.rope_scaling is None else dict(self.rope_scaling, rope_type="llama3")
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out
