"""The decay-attention mixer: linear attention with a fixed decay per head and a state of fixed size.

Per head h with decay d_h, over a sequence's tokens t = 0, 1, ...:
    S_t = d_h S_(t-1) + k_t v_t^T        (S [dim, vdim], float32, zero before the first token)
    o_t = S_t^T q_t
There is no softmax and no denominator, so a sequence needs no keys of earlier tokens, only S: the mixer
declares a `StateRequirement` and the cache keeps one state row per slot (`cache.state`, zeroed when the slot
is handed out).  Retention layers and "lightning" layers are this mixer with different parameters:

  activation   None, or "silu" applied to q, k and v before they enter the recurrence
  position     a rotary part applied to q and k (None: no rotation)
  k_scale      a constant on k (after rotation)
  out_norm     "per_head": every head's o is divided by its root mean square, no weight;
               "all_heads": the concatenated heads are normed together, times the weight `norm`
  gate         "silu" or "sigmoid": the normed output is multiplied by gate_fn(W_g x), element by element

One product makes q, k, v and the gate's logits ([W_q; W_k; W_v; W_g]); rotation, activation, the constant on
k, the recurrence and its products with q run in float from those rows (`ops.decay_attention`); norm and gate
are one kernel over the float result; then the output product.
"""
from __future__ import annotations

import torch

from ..cache.cache import RunCache, StateRequirement
from ..kernels import ops
from .registry import BuildContext, build_part, register_part
from .spec import PartSpec


class DecayAttention:
    def __init__(self, *, hidden_size, n_heads, dim, vdim, decay, activation, k_scale, position, out_norm, norm_weight, eps,
                 gate, wq, wk, wv, wg, wo, device):
        if len(decay) != n_heads:
            raise ValueError(f"decay_attention: {len(decay)} decays for {n_heads} heads")
        if any(not 0.0 <= float(d) <= 1.0 for d in decay):
            raise ValueError("decay_attention: a decay lies outside [0, 1]")
        if activation not in (None, "silu"):
            raise ValueError(f"decay_attention: unknown activation '{activation}' (known: None, 'silu')")
        if out_norm not in ("per_head", "all_heads"):
            raise ValueError(f"decay_attention: out_norm '{out_norm}' is not one of 'per_head', 'all_heads'")
        if gate not in ops.GATES:
            raise ValueError(f"decay_attention: unknown gate '{gate}', known: {sorted(ops.GATES)}")
        if position is not None and not (hasattr(position, "tables") and getattr(position, "pairing", "half") == "half"):
            raise ValueError("decay_attention: the position part must offer tables() of half-split pairs")
        self.hidden_size, self.n_heads, self.dim, self.vdim = hidden_size, n_heads, dim, vdim
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32, device=device)
        self.silu, self.k_scale, self.position = activation == "silu", float(k_scale), position
        self.out_norm, self.norm_weight, self.eps, self.gate = out_norm, norm_weight, float(eps), gate
        self.w_in = torch.cat([wq, wk, wv, wg], dim=0).contiguous()
        self.w_o = wo
        self.q_col, self.k_col = 0, n_heads * dim
        self.v_col, self.g_col = 2 * n_heads * dim, 2 * n_heads * dim + n_heads * vdim

    def needs(self):
        return None, StateRequirement((self.n_heads, self.dim, self.vdim), "float32")

    def forward(self, x, batch, cache: RunCache, run: int):
        H, vd = self.n_heads, self.vdim
        rows = ops.linear(x, self.w_in)
        cos = sin = None
        rot_n = 0
        if self.position is not None:
            (cos, sin), rot_n = self.position.tables(), self.position.rotary_dim
        o = ops.decay_attention(rows, q_col=self.q_col, k_col=self.k_col, v_col=self.v_col, n_heads=H, dim=self.dim, vdim=vd,
                                decay=self.decay, state=cache.state, tok_pos=batch.tok_pos, seq_start=batch.seq_start,
                                slots=batch.slots, n_seqs=batch.n_seqs, silu=self.silu, k_scale=self.k_scale,
                                cos=cos, sin=sin, rot_n=rot_n)
        y = ops.group_norm_gate(o, H if self.out_norm == "per_head" else 1, eps=self.eps, weight=self.norm_weight,
                                gate=rows[:, self.g_col:self.g_col + H * vd], gate_kind=self.gate, out_dtype=x.dtype)
        return ops.linear(y, self.w_o)


def _build_decay_attention(spec: PartSpec, ctx: BuildContext) -> DecayAttention:
    p, t = spec.params, spec.tensors
    position = build_part("position", p["position"], ctx) if p.get("position") is not None else None
    return DecayAttention(hidden_size=p["hidden_size"], n_heads=p["n_heads"], dim=p["dim"], vdim=p["vdim"], decay=p["decay"],
                          activation=p.get("activation"), k_scale=p.get("k_scale", 1.0), position=position,
                          out_norm=p.get("out_norm", "per_head"),
                          norm_weight=ctx.tensor(t["norm"]) if "norm" in t else None, eps=p["eps"], gate=p.get("gate", "sigmoid"),
                          wq=ctx.tensor(t["q"]), wk=ctx.tensor(t["k"]), wv=ctx.tensor(t["v"]), wg=ctx.tensor(t["g"]),
                          wo=ctx.tensor(t["o"]), device=ctx.device)


register_part("mixer", "decay_attention", _build_decay_attention, replace=True)
