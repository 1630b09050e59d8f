"""A routed feed-forward: a router chooses, per token, a few of many small gated feed-forwards.

Per row x (`csrc/moe.cu`):
    z = W_r x                      float32 logits over all experts, identity experts included
    s = softmax(z)
    the `top` experts with the largest s + correction are taken; their weights are s itself, not renormalised
    y = sum_k s[e_k] * expert_{e_k}(x)
A real expert is W_down gated(W_gate x, W_up x) without biases, with the gated form and its parameter as
parameters (`ops.GATED_FORMS`); the last `n_identity` outputs of the router are identity experts, whose
output is x itself.  Rows are independent of each other, so packing and batching never concern the part.
Interface: `forward(x [rows, hidden] normed) -> [rows, hidden]`.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .registry import BuildContext, register_part
from .spec import PartSpec


class RoutedExperts:
    def __init__(self, *, hidden_size, expert_size, n_experts, n_identity, top, form, form_param, w_router, correction,
                 gates, ups, downs):
        if form not in ops.GATED_FORMS:
            raise ValueError(f"routed_experts: unknown gated form '{form}', known: {sorted(ops.GATED_FORMS)}")
        if not 1 <= top <= n_experts + n_identity:
            raise ValueError(f"routed_experts: {top} of {n_experts + n_identity} experts cannot be chosen")
        self.hidden_size, self.expert_size = hidden_size, expert_size
        self.n_experts, self.n_identity, self.top = n_experts, n_identity, top
        self.form, self.form_param = form, float(form_param)
        self.w_router = w_router.to(torch.float32).contiguous()
        self.correction = correction.to(torch.float32).contiguous() if correction is not None else None
        # [experts, 2 ff, hidden]: an expert's gate rows, then its up rows; [experts, hidden, ff]
        self.w_gate_up = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]).contiguous() if n_experts else None
        self.w_down = torch.stack(list(downs)).contiguous() if n_experts else None

    def forward(self, x):
        sel, sel_w = ops.moe_route(x, self.w_router, self.correction, self.top)
        return ops.moe_experts(x, sel, sel_w, self.w_gate_up, self.w_down, self.n_experts, self.form, self.form_param)


def _build_routed_experts(spec: PartSpec, ctx: BuildContext) -> RoutedExperts:
    p, t = spec.params, spec.tensors
    E = p["n_experts"]
    return RoutedExperts(hidden_size=p["hidden_size"], expert_size=p["expert_size"], n_experts=E, n_identity=p.get("n_identity", 0),
                         top=p["top"], form=p["form"], form_param=p.get("form_param", 0.0),
                         w_router=ctx.tensor(t["router"]), correction=ctx.tensor(t["correction"]) if "correction" in t else None,
                         gates=[ctx.tensor(t[f"gate{e}"]) for e in range(E)], ups=[ctx.tensor(t[f"up{e}"]) for e in range(E)],
                         downs=[ctx.tensor(t[f"down{e}"]) for e in range(E)])


register_part("feed_forward", "routed_experts", _build_routed_experts, replace=True)
