"""Registries of the parts a layer is made of.

A part is a small class that owns its parameters and launches kernels through
`ops`; it takes its sizes and constants as constructor arguments and never
sees the model's configuration.  Five kinds, one registry each:

    NORMS          forward(x32 [T,D], out [R,D], rows=None)
    POSITIONS      prepare(max_positions, device); what a mixer needs to place tokens
    MIXERS         cache_needs(); forward(h, batch, view, residual, append)
    FEED_FORWARDS  forward(h, residual)
    BLOCKS         roles; cache_needs(); forward(x32, batch, view, append): the arrangement of the above

Every part also has `param_specs()` (name -> weights.loader.ParamSpec) and
`load(tensors)`.  Mixers and feed-forwards ADD their result into `residual`, the
step's residual stream (`parts.residual.Residual`, float32):
`residual.add_linear(a, w)` folds the sum into the product's kernel (or defers
it to the next norm), `residual.add(y)` is for parts that cannot fuse.

`register_*` adds a class under a name; a `config.spec.PartSpec` names it.
"""
from typing import Any, Callable, Dict

from ..config.spec import PartSpec

NORMS: Dict[str, Callable] = {}
POSITIONS: Dict[str, Callable] = {}
MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}

# kind of part -> registry; a block arrangement names a kind for each of its roles
REGISTRIES: Dict[str, Dict[str, Callable]] = {"norm": NORMS, "position": POSITIONS, "mixer": MIXERS,
                                              "feed_forward": FEED_FORWARDS}


def _registrar(table: Dict[str, Callable], kind: str):
    def register(name: str, factory: Callable = None):
        """`register(name, cls)` or `@register(name)` above a class."""
        def put(f):
            if name in table and table[name] is not f:
                raise ValueError(f"{kind} '{name}' is already registered")
            table[name] = f
            return f
        return put(factory) if factory is not None else put
    return register


register_norm = _registrar(NORMS, "norm")
register_position = _registrar(POSITIONS, "position encoding")
register_mixer = _registrar(MIXERS, "mixer")
register_feed_forward = _registrar(FEED_FORWARDS, "feed-forward")
register_block = _registrar(BLOCKS, "block")


def build_block(layer, dim: int, dtype, position):
    """Construct the block arrangement a `LayerSpec` names, with one part per declared role."""
    if layer.block not in BLOCKS:
        raise KeyError(f"no block arrangement named '{layer.block}'; known: {sorted(BLOCKS)}")
    cls = BLOCKS[layer.block]
    roles = dict(cls.roles)
    optional = set(getattr(cls, "optional_roles", ()))
    unknown = sorted(set(layer.parts) - set(roles))
    missing = sorted(set(roles) - set(layer.parts) - optional)
    if unknown or missing:
        raise ValueError(f"block '{layer.block}' takes the parts {sorted(roles)}"
                         + (f"; not given: {missing}" if missing else "") + (f"; not known to it: {unknown}" if unknown else ""))
    built = {}
    for role, kind in roles.items():
        if role not in layer.parts:
            continue
        if kind not in REGISTRIES:
            raise KeyError(f"block '{layer.block}' asks for a part of kind '{kind}'; kinds: {sorted(REGISTRIES)}")
        extra = {"position": position} if kind == "mixer" else {}
        built[role] = build_part(REGISTRIES[kind], layer.parts[role], dtype=dtype, **extra)
    return cls(parts=built, dim=dim, dtype=dtype)


def build_part(table: Dict[str, Callable], spec: PartSpec, **extra: Any):
    """Construct the part that `spec` names, with the spec's parameters plus
    what the model adds (dtype, a position encoding, ...)."""
    if spec.kind not in table:
        raise KeyError(f"no part named '{spec.kind}' is registered; known: {sorted(table)}")
    return table[spec.kind](**spec.params, **extra)


from . import norm, rope, attention, feed_forward, block  # noqa: E402,F401  (register the built-in parts)
