"""Tiny Dokulorn configurations for the tests.  They differ from each other in every size, constant and in the order
of their layers:
  DA  a pair first (4 query heads on 2 key/value heads, heads of 32, rotation on half of a head), then two retention
      layers (one with decay 1: nothing is forgotten; values wider than keys); sizes the tensor-core kernels take
  DB  sizes no fast kernel takes: heads of 12 and 20 values, an odd number of rotated pairs, as many key/value heads as
      query heads, values wider than keys in the softmax half (the heads are zero-padded), rotation on the whole head,
      one lightning head, alpha and the embedding's scale 1, a pair without feed-forward and a retention layer with one
  DC  heads of 64 and 128 (the tcgen05 prefill attention; two column blocks of a state), one key/value head for all
      query heads, a head with decay 0
"""
import copy


def _rot(base, dims):
    return {"base": base, "dims": dims}


def _ret(heads, dim, vdim, decay, rot):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rot}


def _left(heads, kv_heads, dim, vdim, rot, scale, softcap):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale, "softcap": softcap}


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


DA = {
    "architecture": "Dokulorn", "width": 64, "vocab": 180, "norm": {"eps": 1e-5}, "postln_alpha": 1.7, "embedding": {"scale": 3.0},
    "max_positions": 1024,
    "layers": [
        {"type": "parallel", "mixer": {"left": _left(4, 2, 32, 32, _rot(500.0, 16), 0.9, 8.0), "right": _right(2, 32, 48, [0.9, 0.99])},
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "retention", "mixer": _ret(2, 32, 64, [0.95, 1.0], _rot(10000.0, 32)), "mlp": None},
        {"type": "retention", "mixer": _ret(3, 16, 16, [0.7, 0.97, 0.999], _rot(100.0, 8)), "mlp": {"kind": "dense", "ff": 40}},
    ],
}
DB = {
    "architecture": "Dokulorn", "width": 72, "vocab": 131, "norm": {"eps": 1e-4}, "postln_alpha": 1.0, "embedding": {"scale": 1.0},
    "max_positions": 600,
    "layers": [
        {"type": "retention", "mixer": _ret(5, 12, 20, [0.5, 0.8, 0.9, 0.99, 0.9999], _rot(30.0, 6)), "mlp": {"kind": "dense", "ff": 50}},
        {"type": "parallel", "mixer": {"left": _left(3, 3, 24, 40, _rot(2000.0, 24), 1.3, 30.0), "right": _right(1, 8, 72, [0.93])},
         "mlp": None},
        {"type": "parallel", "mixer": {"left": _left(6, 1, 8, 8, _rot(50.0, 2), 2.0, 5.0), "right": _right(3, 20, 12, [0.6, 0.98, 1.0])},
         "mlp": {"kind": "dense", "ff": 33}},
    ],
}
DC = {
    "architecture": "Dokulorn", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "postln_alpha": 3.0, "embedding": {"scale": 7.5},
    "max_positions": 2048,
    "layers": [
        {"type": "retention", "mixer": _ret(2, 64, 128, [0.98, 0.9995], _rot(5e5, 64)), "mlp": None},
        {"type": "parallel", "mixer": {"left": _left(4, 1, 64, 64, _rot(10000.0, 32), 1.1, 15.0), "right": _right(2, 128, 32, [0.0, 0.96])},
         "mlp": {"kind": "dense", "ff": 192}},
        {"type": "retention", "mixer": _ret(1, 128, 64, [0.999], _rot(777.0, 128)), "mlp": None},
    ],
}

CONFIGS = {"DA": (DA, 31), "DB": (DB, 32), "DC": (DC, 33)}


def config(name):
    cfg, seed = CONFIGS[name]
    return copy.deepcopy(cfg), seed
