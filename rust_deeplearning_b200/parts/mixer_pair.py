"""Two mixers side by side: both read the same input, each result is normed over the model width with a plain
weight of its own, and the mixer's result is `factor` times their sum:
    y = factor * (rms_norm(left(x); w_left) + rms_norm(right(x); w_right)).
The two are built through the mixer registry from their own descriptions (`params["left"]`, `params["right"]`:
`PartSpec`s of any registered kinds), so any pair can stand side by side as long as at most one of them keeps
keys and values and at most one keeps state: a layer run has one key/value store and one state row.
The sum is formed in float32 (one kernel for both norms and the sum).
"""
from __future__ import annotations

from ..cache.cache import RunCache
from ..kernels import ops
from .registry import BuildContext, build_part, register_part
from .spec import PartSpec


class MixerPair:
    def __init__(self, left, right, w_left, w_right, eps: float, factor: float):
        self.left, self.right = left, right
        self.w_left, self.w_right, self.eps, self.factor = w_left, w_right, float(eps), float(factor)
        (lk, ls), (rk, rs) = left.needs(), right.needs()
        if lk is not None and rk is not None:
            raise ValueError("mixer_pair: both mixers keep keys and values; a layer run has one store")
        if ls is not None and rs is not None:
            raise ValueError("mixer_pair: both mixers keep state; a layer run has one state row")
        self._needs = (lk if lk is not None else rk, ls if ls is not None else rs)
        # the step's batch description is cut into query tiles for whichever of the two asks
        self.query_tile_rows = max(getattr(left, "query_tile_rows", 0) or 0, getattr(right, "query_tile_rows", 0) or 0)

    def needs(self):
        return self._needs

    def forward(self, x, batch, cache: RunCache, run: int):
        a = self.left.forward(x, batch, cache, run)
        b = self.right.forward(x, batch, cache, run)
        return ops.norm_pair(a, b, self.w_left, self.w_right, self.eps, self.factor)


def _build_mixer_pair(spec: PartSpec, ctx: BuildContext) -> MixerPair:
    p, t = spec.params, spec.tensors
    left = build_part("mixer", p["left"], ctx)
    right = build_part("mixer", p["right"], ctx)
    return MixerPair(left, right, ctx.tensor(t["left_out"]), ctx.tensor(t["right_out"]), p["eps"], p.get("factor", 0.5))


register_part("mixer", "mixer_pair", _build_mixer_pair, replace=True)
