"""Ligirax: typed configuration and its description as parts.

A decoder-only model of layers listed one by one in config.json: every layer names its mixer (`type`; the
one kind is "latent_attention", `parts/latent_attention.py`) with the mixer's own sizes, and its
feed-forward (`mlp`: a routed mixture of small gated feed-forwards, `parts/routed_experts.py`, or null for
none).  Around each sublayer stand a norm before and a norm after (scale-only root-mean-square norms with
a plain weight), and the normed branch is multiplied by `residual_mult` before it joins the stream:
    x <- x + m * norm1b(mixer(norm1(x)));   x <- x + m * norm2b(ff(norm2(x))).
The embedding table is also the output matrix; logits are multiplied by `logit_scale`.

What the design fixes stands here: the four-norm arrangement, interleaved rotary pairs with YaRN-blended
frequencies on the rotated part of queries and of the shared key part, the gated form of the experts
(`swish_limit`: min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1)), softmax scores with a correction
added for the choice only and weights that are not renormalised, identity experts at the end of the
router's outputs.  Every size and every other constant is read from config.json.  A mixer with `kv_from: j`
has no compression of its own and reads the cached latent rows of layer j.

The design names no longest context; tables of the position encoding are built for `max_positions`
(an optional key of this library, default 32,768).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import Architecture, ConfigError, ConfigReader, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

ARCHITECTURE_NAME = "Ligirax"
MODEL_TYPE = "ligirax"
DEFAULT_MAX_POSITIONS = 32768


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]]     # YaRN: factor, original, fast, slow; None: plain frequencies


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot: RotaryConfig
    kv_from: Optional[int]


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    identity: int
    top: int
    ff: int
    limit: float


@dataclass(frozen=True)
class LigiraxLayer:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[MoEConfig]


@dataclass(frozen=True)
class LigiraxConfig:
    width: int
    vocab: int
    eps: float
    residual_mult: float
    logit_scale: float
    max_positions: int
    layers: Tuple[LigiraxLayer, ...]
    raw: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "LigiraxConfig":
        r = ConfigReader(raw, "Ligirax config")
        width = r.integer("width", minimum=1)
        vocab = r.integer("vocab", minimum=1)
        mult = r.number("residual_mult")
        logit_scale = r.number("logit_scale")
        maxpos = r.integer("max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1)
        eps = None
        if isinstance(raw.get("norm"), dict):
            rn = ConfigReader(raw["norm"], "norm")
            eps = rn.number("eps", positive=True)
            r.problems += [f"norm: {p}" for p in rn.problems]
        else:
            r.problems.append("missing key 'norm' (an object with 'eps')")
        layers = []
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            r.problems.append("key 'layers' must list at least one layer")
            listed = []
        for i, entry in enumerate(listed):
            layer, problems = _parse_layer(entry, i, len(listed))
            r.problems += [f"layers[{i}]: {p}" for p in problems]
            if layer is not None:
                layers.append(layer)
        if not r.problems:
            for i, layer in enumerate(layers):
                j = layer.mixer.kv_from
                if j is None:
                    continue
                if not 0 <= j < i:
                    r.problems.append(f"layers[{i}]: kv_from names layer {j}, which does not come before it")
                    continue
                src = layers[j].mixer
                if src.kv_from is not None:
                    r.problems.append(f"layers[{i}]: kv_from names layer {j}, which has no latent rows of its own")
                elif (src.kv_rank, src.rot_dim, src.rot) != (layer.mixer.kv_rank, layer.mixer.rot_dim, layer.mixer.rot):
                    r.problems.append(f"layers[{i}]: kv_rank, rot_dim and rot must equal those of layer {j}, whose rows it reads")
        r.finish()
        return LigiraxConfig(width, vocab, eps, mult, logit_scale, maxpos, tuple(layers))


def _parse_layer(entry, i, n_layers):
    if not isinstance(entry, dict):
        return None, ["must be an object"]
    r = ConfigReader(entry, "layer")
    kind = r.string("type")
    if kind is not None and kind != "latent_attention":
        r.problems.append(f"type '{kind}' is not known (known: 'latent_attention')")
    mixer = None
    if isinstance(entry.get("mixer"), dict):
        m = entry["mixer"]
        rm = ConfigReader(m, "mixer")
        heads = rm.integer("heads", minimum=1)
        dim = rm.integer("dim", minimum=1)
        rot_dim = rm.integer("rot_dim", minimum=2)
        vdim = rm.integer("vdim", minimum=1)
        kv_rank = rm.integer("kv_rank", minimum=1)
        scale = rm.number("scale")
        kv_from = rm.integer("kv_from", default=None, minimum=0)
        window = None
        if m.get("mask") is not None:
            if isinstance(m["mask"], dict):
                rk = ConfigReader(m["mask"], "mask")
                window = rk.integer("size", minimum=1)
                rm.problems += [f"mask: {p}" for p in rk.problems]
            else:
                rm.problems.append("key 'mask' must be an object with 'size'")
        rot = None
        if isinstance(m.get("rot"), dict):
            rr = ConfigReader(m["rot"], "rot")
            base = rr.number("base", positive=True)
            dims = rr.integer("dims", minimum=2)
            scaling = None
            if m["rot"].get("scaling") is not None:
                if isinstance(m["rot"]["scaling"], dict):
                    rs = ConfigReader(m["rot"]["scaling"], "scaling")
                    vals = [(k, rs.number(k, positive=True)) for k in ("factor", "original", "fast", "slow")]
                    rr.problems += [f"scaling: {p}" for p in rs.problems]
                    scaling = tuple(vals)
                else:
                    rr.problems.append("key 'scaling' must be an object")
            if dims is not None and rot_dim is not None:
                rr.check(dims % 2 == 0 and dims <= rot_dim, f"dims ({dims}) must be even and at most rot_dim ({rot_dim})")
            if base is not None:
                rr.check(base != 1.0, "base must not be 1")
            rm.problems += [f"rot: {p}" for p in rr.problems]
            if not rr.problems:
                rot = RotaryConfig(base, dims, scaling)
        else:
            rm.problems.append("missing key 'rot' (an object)")
        r.problems += [f"mixer: {p}" for p in rm.problems]
        if not rm.problems:
            mixer = LatentMixerConfig(heads, dim, rot_dim, vdim, kv_rank, scale, window, rot, kv_from)
    else:
        r.problems.append("missing key 'mixer' (an object)")
    mlp = None
    if entry.get("mlp") is not None:
        f = entry["mlp"]
        if not isinstance(f, dict):
            r.problems.append("key 'mlp' must be an object or null")
        else:
            rf = ConfigReader(f, "mlp")
            fk = rf.string("kind", default="moe")
            if fk is not None and fk != "moe":
                rf.problems.append(f"kind '{fk}' is not known (known: 'moe')")
            ff = limit = experts = identity = top = None
            if isinstance(f.get("expert"), dict):
                re_ = ConfigReader(f["expert"], "expert")
                ff = re_.integer("ff", minimum=1)
                limit = re_.number("limit", positive=True)
                rf.problems += [f"expert: {p}" for p in re_.problems]
            else:
                rf.problems.append("missing key 'expert' (an object)")
            if isinstance(f.get("router"), dict):
                rr = ConfigReader(f["router"], "router")
                experts = rr.integer("experts", minimum=0)
                identity = rr.integer("identity", default=0, minimum=0)
                top = rr.integer("top", minimum=1)
                if None not in (experts, identity, top):
                    rr.check(experts + identity >= 1 and top <= experts + identity,
                             f"top ({top}) of {experts} + {identity} experts cannot be chosen")
                rf.problems += [f"router: {p}" for p in rr.problems]
            else:
                rf.problems.append("missing key 'router' (an object)")
            r.problems += [f"mlp: {p}" for p in rf.problems]
            if not rf.problems:
                mlp = MoEConfig(experts, identity, top, ff, limit)
    if r.problems:
        return None, r.problems
    return LigiraxLayer(kind, mixer, mlp), []


def build_spec(cfg: LigiraxConfig) -> ModelSpec:
    """The model as parts; tensor names are the checkpoint's own ('l<i>.' + 'norm1', 'mix.q', 'mlp.e<k>.gate', ...)."""
    W, V = cfg.width, cfg.vocab

    def norm(name, scale=1.0):
        return PartSpec("rms_norm", {"size": W, "eps": cfg.eps, "offset": 0.0, "scale": scale},
                        {"weight": TensorSpec(name, (W,), "vector", init_std=0.1, init_mean=1.0)})

    # the window the cached rows of a layer are kept for: the widest of the layers that read them
    keep: Dict[int, Optional[int]] = {}
    unlimited = set()
    for i, layer in enumerate(cfg.layers):
        owner = layer.mixer.kv_from if layer.mixer.kv_from is not None else i
        if layer.mixer.window is None:
            unlimited.add(owner)
        keep[owner] = max(keep.get(owner) or 0, layer.mixer.window or 0)

    layers, ignored = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        H, d, rd, vd, r = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
        owner = m.kv_from if m.kv_from is not None else i
        position = PartSpec("rotary", {
            "theta": m.rot.base, "head_dim": rd, "rotary_dim": m.rot.dims, "max_positions": cfg.max_positions,
            "pairing": "interleaved", "scaling": dict(m.rot.scaling, kind="yarn") if m.rot.scaling else None})
        tensors = {"q": TensorSpec(p + "mix.q", (H * (d + rd), W)),
                   "uk": TensorSpec(p + "mix.uk", (H * d, r), init_std=0.08),
                   "uv": TensorSpec(p + "mix.uv", (H * vd, r), init_std=0.08),
                   "g": TensorSpec(p + "mix.g", (H, W)),
                   "o": TensorSpec(p + "mix.o", (W, H * vd))}
        if m.kv_from is None:
            tensors["dkv"] = TensorSpec(p + "mix.dkv", (r + rd, W))
            tensors["dkv_norm"] = TensorSpec(p + "mix.dkv.norm", (r,), "vector", init_std=0.1, init_mean=1.0)
        mixer = PartSpec("latent_attention", {
            "hidden_size": W, "n_heads": H, "dim": d, "rot_dim": rd, "vdim": vd, "kv_rank": r, "score_scale": m.scale,
            "window": m.window, "cache_window": None if owner in unlimited else keep[owner], "eps": cfg.eps,
            "position": position}, tensors)
        norms = {"pre_mixer": norm(p + "norm1"), "post_mixer": norm(p + "norm1b", cfg.residual_mult)}
        ff = None
        if layer.mlp is not None:
            f = layer.mlp
            total = f.experts + f.identity
            ft = {"router": TensorSpec(p + "mlp.router", (total, W), init_std=0.5),
                  "correction": TensorSpec(p + "mlp.correction", (total,), "vector", init_std=0.2)}
            for e in range(f.experts):
                ft[f"gate{e}"] = TensorSpec(p + f"mlp.e{e}.gate", (f.ff, W))
                ft[f"up{e}"] = TensorSpec(p + f"mlp.e{e}.up", (f.ff, W))
                ft[f"down{e}"] = TensorSpec(p + f"mlp.e{e}.down", (W, f.ff))
            ff = PartSpec("routed_experts", {"hidden_size": W, "expert_size": f.ff, "n_experts": f.experts, "n_identity": f.identity,
                                             "top": f.top, "form": "swish_limit", "form_param": f.limit}, ft)
            norms["pre_feed_forward"] = norm(p + "norm2")
            norms["post_feed_forward"] = norm(p + "norm2b", cfg.residual_mult)
        else:
            ignored += [p + "norm2", p + "norm2b"]      # a file may carry them; a layer without a feed-forward reads neither
        layers.append(LayerSpec("sandwich", mixer, ff, norms))

    table = TensorSpec("embed", (V, W), init_std=0.5)
    spec = ModelSpec(
        architecture=ARCHITECTURE_NAME, hidden_size=W, vocab_size=V, max_positions=cfg.max_positions,
        embedding=PartSpec("scaled_embedding", {"vocab_size": V, "hidden_size": W, "scale": 1.0}, {"table": table}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, layer.mixer.kv_from) for i, layer in enumerate(cfg.layers)),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": W, "softcap": None, "scale": cfg.logit_scale}, {"weight": table}),
        ignored_tensors=tuple(ignored))
    spec.validate()
    return spec


register_architecture(Architecture(ARCHITECTURE_NAME, MODEL_TYPE, LigiraxConfig.from_dict, build_spec), replace=True)
