"""Dokulorn: typed configuration and its description as parts.

A decoder-only model whose layers are listed one by one in config.json.  Every layer norms AFTER the sum,
    x <- norm1(alpha x + mixer(x));   x <- norm2(alpha x + ff(x))      (alpha = `postln_alpha`),
with scale-only root-mean-square norms whose weight holds the scale minus one (y = x / rms * (1 + w)); a layer whose
`mlp` is null ends after the first sublayer.  A layer's `type` names its mixer:

  "retention"  linear attention with a fixed decay per head (`parts/decay_attention.py`): rotary positions on q and
               k, k times dim^(-1/2), every head's output divided by its root mean square, gate silu(W_g x);
  "parallel"   two mixers side by side on the same input (`parts/mixer_pair.py`), each result normed over the model
               width with a plain weight, the mixer's result half their sum.  Left: softmax attention with grouped
               key/value heads, rotary positions, q and k divided by their root mean square after rotation, a score
               scale, a tanh soft-cap, a learned sink per head in the softmax's denominator and an element-wise
               sigmoid gate (`parts/attention.py`).  Right: decay attention on silu(q), silu(k), silu(v), the heads
               normed together with a plain weight, gate sigmoid(W_g x).

The feed-forward is the gated form with tanh-GELU.  The embedding is multiplied by `embedding.scale`; logits are the
final norm's rows times the embedding table (without that scale).

What the design fixes stands here (which norm has which offset, which activation gates what, k's constant, the
factor 1/2); every size and every other constant is read from config.json.  The design names no longest context;
tables of the position encodings are built for `max_positions` (an optional key of this library, default 32,768).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import Architecture, ConfigReader, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

ARCHITECTURE_NAME = "Dokulorn"
MODEL_TYPE = "dokulorn"
DEFAULT_MAX_POSITIONS = 32768


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int


@dataclass(frozen=True)
class DecayMixerConfig:
    """A retention mixer, or the right half of a parallel mixer (which has no rotation)."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[RotaryConfig]


@dataclass(frozen=True)
class SoftmaxMixerConfig:
    """The left half of a parallel mixer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    rot: RotaryConfig


@dataclass(frozen=True)
class DokulornLayer:
    type: str                                   # "retention" or "parallel"
    retention: Optional[DecayMixerConfig]
    left: Optional[SoftmaxMixerConfig]
    right: Optional[DecayMixerConfig]
    ff: Optional[int]                           # the dense feed-forward's inner size; None: no feed-forward


@dataclass(frozen=True)
class DokulornConfig:
    width: int
    vocab: int
    eps: float
    alpha: float
    embedding_scale: float
    max_positions: int
    layers: Tuple[DokulornLayer, ...]

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "DokulornConfig":
        r = ConfigReader(raw, "Dokulorn config")
        width = r.integer("width", minimum=1)
        vocab = r.integer("vocab", minimum=1)
        alpha = r.number("postln_alpha")
        maxpos = r.integer("max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1)
        eps = _sub_number(r, raw, "norm", "eps", positive=True)
        scale = _sub_number(r, raw, "embedding", "scale")
        layers = []
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            r.problems.append("key 'layers' must list at least one layer")
            listed = []
        for i, entry in enumerate(listed):
            layer, problems = _parse_layer(entry)
            r.problems += [f"layers[{i}]: {p}" for p in problems]
            if layer is not None:
                layers.append(layer)
        r.finish()
        return DokulornConfig(width, vocab, eps, alpha, scale, maxpos, tuple(layers))


def _sub_number(r: ConfigReader, raw, outer: str, key: str, positive: bool = False):
    if isinstance(raw.get(outer), dict):
        rr = ConfigReader(raw[outer], outer)
        v = rr.number(key, positive=positive)
        r.problems += [f"{outer}: {p}" for p in rr.problems]
        return v
    r.problems.append(f"missing key '{outer}' (an object with '{key}')")
    return None


def _parse_rot(m, rm: ConfigReader, dim) -> Optional[RotaryConfig]:
    if not isinstance(m.get("rot"), dict):
        rm.problems.append("missing key 'rot' (an object with 'base' and 'dims')")
        return None
    rr = ConfigReader(m["rot"], "rot")
    base = rr.number("base", positive=True)
    dims = rr.integer("dims", minimum=2)
    if dims is not None and dim is not None:
        rr.check(dims % 2 == 0 and dims <= dim, f"dims ({dims}) must be even and at most dim ({dim})")
    rm.problems += [f"rot: {p}" for p in rr.problems]
    return None if rr.problems else RotaryConfig(base, dims)


def _parse_decay_mixer(m, what: str, with_rot: bool):
    """-> (DecayMixerConfig or None, problems)"""
    if not isinstance(m, dict):
        return None, [f"{what} must be an object"]
    rm = ConfigReader(m, what)
    heads = rm.integer("heads", minimum=1)
    dim = rm.integer("dim", minimum=1)
    vdim = rm.integer("vdim", minimum=1)
    decay = m.get("decay")
    if not isinstance(decay, list) or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
        rm.problems.append("key 'decay' must list a number per head")
        decay = None
    elif heads is not None:
        rm.check(len(decay) == heads, f"'decay' lists {len(decay)} numbers for {heads} heads")
        rm.check(all(0.0 <= float(d) <= 1.0 for d in decay), "every decay must lie in [0, 1]")
    rot = _parse_rot(m, rm, dim) if with_rot else None
    if rm.problems:
        return None, [f"{what}: {p}" for p in rm.problems]
    return DecayMixerConfig(heads, dim, vdim, tuple(float(d) for d in decay), rot), []


def _parse_softmax_mixer(m, what: str):
    if not isinstance(m, dict):
        return None, [f"{what} must be an object"]
    rm = ConfigReader(m, what)
    heads = rm.integer("heads", minimum=1)
    kv_heads = rm.integer("kv_heads", minimum=1)
    dim = rm.integer("dim", minimum=1)
    vdim = rm.integer("vdim", minimum=1)
    scale = rm.number("scale")
    softcap = rm.number("softcap", positive=True)
    if heads is not None and kv_heads is not None:
        rm.check(heads % kv_heads == 0, f"{heads} heads cannot share {kv_heads} key/value heads")
    rot = _parse_rot(m, rm, dim)
    if rm.problems:
        return None, [f"{what}: {p}" for p in rm.problems]
    return SoftmaxMixerConfig(heads, kv_heads, dim, vdim, scale, softcap, rot), []


def _parse_layer(entry):
    if not isinstance(entry, dict):
        return None, ["must be an object"]
    r = ConfigReader(entry, "layer")
    kind = r.string("type")
    retention = left = right = None
    m = entry.get("mixer")
    if kind == "retention":
        retention, problems = _parse_decay_mixer(m, "mixer", with_rot=True)
        r.problems += problems
    elif kind == "parallel":
        if not isinstance(m, dict):
            r.problems.append("missing key 'mixer' (an object with 'left' and 'right')")
        else:
            left, problems = _parse_softmax_mixer(m.get("left"), "mixer.left")
            r.problems += problems
            right, problems = _parse_decay_mixer(m.get("right"), "mixer.right", with_rot=False)
            r.problems += problems
    elif kind is not None:
        r.problems.append(f"type '{kind}' is not known (known: 'retention', 'parallel')")
    ff = None
    if entry.get("mlp") is not None:
        f = entry["mlp"]
        if not isinstance(f, dict):
            r.problems.append("key 'mlp' must be an object or null")
        else:
            rf = ConfigReader(f, "mlp")
            fk = rf.string("kind", default="dense")
            if fk is not None and fk != "dense":
                rf.problems.append(f"kind '{fk}' is not known (known: 'dense')")
            ff = rf.integer("ff", minimum=1)
            r.problems += [f"mlp: {p}" for p in rf.problems]
    if r.problems:
        return None, r.problems
    return DokulornLayer(kind, retention, left, right, ff), []


def _rotary(rot: RotaryConfig, dim: int, max_positions: int) -> PartSpec:
    return PartSpec("rotary", {"theta": rot.base, "head_dim": dim, "rotary_dim": rot.dims, "max_positions": max_positions,
                               "pairing": "half"})


def _decay_mixer(cfg: DokulornConfig, m: DecayMixerConfig, prefix: str, retention: bool) -> PartSpec:
    W, H = cfg.width, m.heads
    tensors = {"q": TensorSpec(prefix + "q", (H * m.dim, W)), "k": TensorSpec(prefix + "k", (H * m.dim, W)),
               "v": TensorSpec(prefix + "v", (H * m.vdim, W)), "g": TensorSpec(prefix + "g", (H * m.vdim, W)),
               "o": TensorSpec(prefix + "o", (W, H * m.vdim))}
    params = {"hidden_size": W, "n_heads": H, "dim": m.dim, "vdim": m.vdim, "decay": m.decay, "eps": cfg.eps}
    if retention:
        params.update(activation=None, k_scale=m.dim ** -0.5, position=_rotary(m.rot, m.dim, cfg.max_positions),
                      out_norm="per_head", gate="silu")
    else:
        params.update(activation="silu", k_scale=1.0, position=None, out_norm="all_heads", gate="sigmoid")
        tensors["norm"] = TensorSpec(prefix + "norm", (H * m.vdim,), "vector", init_std=0.1, init_mean=1.0)
    return PartSpec("decay_attention", params, tensors)


def _softmax_mixer(cfg: DokulornConfig, m: SoftmaxMixerConfig, prefix: str) -> PartSpec:
    W, H, G = cfg.width, m.heads, m.kv_heads
    tensors = {"q": TensorSpec(prefix + "q", (H * m.dim, W)), "k": TensorSpec(prefix + "k", (G * m.dim, W)),
               "v": TensorSpec(prefix + "v", (G * m.vdim, W)), "g": TensorSpec(prefix + "g", (H * m.vdim, W)),
               "o": TensorSpec(prefix + "o", (W, H * m.vdim)),
               "sinks": TensorSpec(prefix + "sink", (H,), "vector", init_std=1.0)}
    return PartSpec("attention", {
        "hidden_size": W, "n_heads": H, "n_kv_heads": G, "head_dim": m.dim, "value_dim": m.vdim, "score_scale": m.scale,
        "softcap": m.softcap, "window": None, "qk_norm_eps": cfg.eps, "gate": "sigmoid",
        "position": _rotary(m.rot, m.dim, cfg.max_positions)}, tensors)


def build_spec(cfg: DokulornConfig) -> ModelSpec:
    """The model as parts; tensor names are the checkpoint's own ('l<i>.' + 'norm1', 'mix.q', 'mix.left.q', 'mlp.gate', ...)."""
    W, V = cfg.width, cfg.vocab

    def norm(name):     # the weight holds the scale minus one (offset 1)
        return PartSpec("rms_norm", {"size": W, "eps": cfg.eps, "offset": 1.0},
                        {"weight": TensorSpec(name, (W,), "vector", init_std=0.1)})

    def plain_weight(name):
        return TensorSpec(name, (W,), "vector", init_std=0.1, init_mean=1.0)

    layers: List[LayerSpec] = []
    ignored: List[str] = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        if layer.type == "retention":
            mixer = _decay_mixer(cfg, layer.retention, p + "mix.", retention=True)
        else:
            mixer = PartSpec("mixer_pair", {
                "left": _softmax_mixer(cfg, layer.left, p + "mix.left."),
                "right": _decay_mixer(cfg, layer.right, p + "mix.right.", retention=False),
                "eps": cfg.eps, "factor": 0.5},
                {"left_out": plain_weight(p + "mix.left.out"), "right_out": plain_weight(p + "mix.right.out")})
        norms = {"post_mixer": norm(p + "norm1")}
        ff = None
        if layer.ff is not None:
            ff = PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": layer.ff, "activation": "gelu_tanh"},
                          {"gate": TensorSpec(p + "mlp.gate", (layer.ff, W)), "up": TensorSpec(p + "mlp.up", (layer.ff, W)),
                           "down": TensorSpec(p + "mlp.down", (W, layer.ff))})
            norms["post_feed_forward"] = norm(p + "norm2")
        else:
            ignored.append(p + "norm2")       # a file may carry it; a layer without a feed-forward does not read it
        layers.append(LayerSpec("postnorm", mixer, ff, norms, {"alpha": cfg.alpha}))

    table = TensorSpec("embed", (V, W), init_std=0.05)
    spec = ModelSpec(
        architecture=ARCHITECTURE_NAME, hidden_size=W, vocab_size=V, max_positions=cfg.max_positions,
        embedding=PartSpec("scaled_embedding", {"vocab_size": V, "hidden_size": W, "scale": cfg.embedding_scale}, {"table": table}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": W, "softcap": None, "scale": 1.0}, {"weight": table}),
        ignored_tensors=tuple(ignored))
    spec.validate()
    return spec


register_architecture(Architecture(ARCHITECTURE_NAME, MODEL_TYPE, DokulornConfig.from_dict, build_spec), replace=True)
