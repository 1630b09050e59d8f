"""Tiny Ligirax configurations for the tests.  They differ from each other in every size and option:
  LA  three layers: one with rows of its own and YaRN scaling, one that reads them through a wider window and with
      other head sizes, one without window and without feed-forward; identity experts
  LB  ten heads (more than a decode block takes), rot.dims below rot_dim, values wider than keys, a cached row whose
      size is no multiple of 16, one expert of three and no identity expert, multipliers of 1
  LC  sizes the fast kernels take (cached rows of 64 values, heads padded to 64), a window of 40
  LD  as LC with every expert chosen (no choice can flip between number formats), for long runs in bfloat16
"""
import copy


def _rot(base, dims, scaling=None):
    return {"base": base, "dims": dims, **({"scaling": scaling} if scaling else {})}


def _mixer(heads, dim, rot_dim, vdim, kv_rank, scale, rot, window=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, identity, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}


_ROT_A = _rot(5000.0, 8, {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0})
LA = {
    "architecture": "Ligirax", "width": 64, "vocab": 200, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_scale": 2.0,
    "max_positions": 512,
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(3, 16, 8, 16, 24, 0.2, _ROT_A, window=8), "mlp": _moe(5, 2, 3, 24, 1.0)},
        {"type": "latent_attention", "mixer": _mixer(2, 24, 8, 8, 24, 0.15, _ROT_A, window=12, kv_from=0), "mlp": _moe(4, 1, 2, 40, 0.7)},
        {"type": "latent_attention", "mixer": _mixer(4, 8, 8, 16, 16, 0.3, _rot(100.0, 8)), "mlp": None},
    ],
}
_ROT_B = _rot(300.0, 8)
LB = {
    "architecture": "Ligirax", "width": 72, "vocab": 131, "norm": {"eps": 1e-4}, "residual_mult": 1.0, "logit_scale": 1.0,
    "max_positions": 300,
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(10, 8, 16, 24, 40, 0.25, _ROT_B, window=5), "mlp": _moe(3, 0, 1, 16, 2.0)},
        {"type": "latent_attention", "mixer": _mixer(10, 8, 16, 24, 40, 0.25, _ROT_B, window=5), "mlp": None},
        {"type": "latent_attention", "mixer": _mixer(5, 16, 16, 8, 40, 0.1, _ROT_B, window=3, kv_from=1), "mlp": _moe(2, 3, 2, 8, 0.5)},
    ],
}
_ROT_C = _rot(20000.0, 16, {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 2.0})
LC = {
    "architecture": "Ligirax", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "residual_mult": 0.4, "logit_scale": 0.7,
    "max_positions": 1024,
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(4, 32, 16, 32, 48, 0.14, _ROT_C, window=40), "mlp": _moe(8, 1, 2, 64, 1.5)},
        {"type": "latent_attention", "mixer": _mixer(4, 32, 16, 32, 48, 0.14, _ROT_C, window=40, kv_from=0), "mlp": _moe(8, 1, 2, 64, 1.5)},
    ],
}
LD = copy.deepcopy(LC)
for _layer in LD["layers"]:
    _layer["mlp"] = _moe(3, 1, 4, 32, 1.5)

CONFIGS = {"LA": (LA, 21), "LB": (LB, 22), "LC": (LC, 23), "LD": (LD, 24)}


def config(name):
    cfg, seed = CONFIGS[name]
    return copy.deepcopy(cfg), seed
