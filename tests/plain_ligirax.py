"""Plain, slow Ligirax in numpy: the oracle the engine is compared with.

Whole sequences, no cache, no batching, float64, one function per mechanism, written from the design's
equations; it shares no code with the package (only the safetensors reader of the other oracle).

    layer:   x <- x + m * norm(mixer(norm(x; n1)); n1b);   x <- x + m * norm(ff(norm(x; n2)); n2b)   (ff may be absent)
    norm:    x / sqrt(mean(x^2) + eps) * w
    mixer:   latent attention (below); feed-forward: routed experts (below)
    output:  logits = E norm(x; final) * logit_scale, E the embedding table
"""
from __future__ import annotations

import math

import numpy as np

from plain_gemma2 import read_config, read_safetensors  # noqa: F401  (file formats only)
import os


def load_folder(folder):
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    return read_config(folder), {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def rotary_frequencies(rot):
    """Frequencies of the n/2 pairs and the factor on cos and sin.  Plain: f_i = base^(-2i/n).  With scaling
    (factor F, original L, fast, slow): d(t) = n ln(L / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), n - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    f_i <- f_i / F * ramp_i + f_i (1 - ramp_i), and cos, sin are multiplied by 0.1 ln F + 1."""
    n, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / n) for i in range(n // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    d = lambda t: n * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(d(sc["fast"])), 0), min(math.ceil(d(sc["slow"])), n - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1 - ramp))
    return np.array(out), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(v, pos, rot):
    """One vector at position pos: pairs (2i, 2i+1) of its first rot['dims'] values turn by pos * f_i; the rest pass."""
    f, mag = rotary_frequencies(rot)
    out = np.array(v, dtype=np.float64)
    for i, fi in enumerate(f):
        a = pos * fi
        c, s = math.cos(a) * mag, math.sin(a) * mag
        u, w = v[2 * i], v[2 * i + 1]
        out[2 * i], out[2 * i + 1] = u * c - w * s, w * c + u * s
    return out


def latent_rows(h, w, prefix, m, eps):
    """Per token: the normed latent c and the rotated shared key part."""
    r = m["kv_rank"]
    dk = h @ w[prefix + "dkv"].T
    c = rms_norm(dk[:, :r], w[prefix + "dkv.norm"], eps)
    kr = np.stack([rotate(dk[t, r:], t, m["rot"]) for t in range(h.shape[0])])
    return c, kr


def latent_attention(h, w, prefix, m, eps, rows):
    """rows: (c, kr) of this layer or of the layer it reads.  Query by query, key by key."""
    T = h.shape[0]
    H, d, rd, vd = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = rows
    q = (h @ w[prefix + "q"].T).reshape(T, H, d + rd)
    k_un = (c @ w[prefix + "uk"].T).reshape(T, H, d)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, vd)
    gate = 1.0 / (1.0 + np.exp(-(h @ w[prefix + "g"].T)))
    window = m["mask"]["size"] if m.get("mask") else None
    out = np.zeros((T, H, vd))
    for i in range(T):
        first = 0 if window is None else max(0, i - window + 1)
        for hh in range(H):
            q_rot = rotate(q[i, hh, d:], i, m["rot"])
            s = np.array([(q[i, hh, :d] @ k_un[j, hh] + q_rot @ kr[j]) * m["scale"] for j in range(first, i + 1)])
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, hh] = (p[:, None] * v[first:i + 1, hh]).sum(axis=0) * gate[i, hh]
    return out.reshape(T, H * vd) @ w[prefix + "o"].T


def router(h, w, prefix, f):
    """Chosen experts [T, top], their weights, and each token's margin: the gap between the last chosen and the
    first not chosen choice score (inf when every expert is chosen)."""
    z = h @ w[prefix + "router"].T
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    s = e / e.sum(axis=-1, keepdims=True)
    choice = s + w[prefix + "correction"]
    top = f["router"]["top"]
    order = np.argsort(-choice, axis=-1, kind="stable")
    chosen = order[:, :top]
    srt = np.take_along_axis(choice, order, axis=-1)
    gaps = [srt[:, k] - srt[:, k + 1] for k in range(min(top, srt.shape[1] - 1))]     # a swap inside the chosen set reorders a sum only
    margin = gaps[-1] if top < srt.shape[1] else np.full(h.shape[0], np.inf)
    return chosen, np.take_along_axis(s, chosen, axis=-1), margin


def expert(x, w, prefix, e, limit):
    g = np.minimum(x @ w[prefix + f"e{e}.gate"].T, limit)
    u = np.clip(x @ w[prefix + f"e{e}.up"].T, -limit, limit)
    return (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)) @ w[prefix + f"e{e}.down"].T


def routed_experts(h, w, prefix, f, margins=None):
    chosen, weight, margin = router(h, w, prefix, f)
    if margins is not None:
        margins.append(margin)
    n_real = f["router"]["experts"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for k, e in enumerate(chosen[t]):
            y = h[t] if e >= n_real else expert(h[t], w, prefix, int(e), f["expert"]["limit"])
            out[t] += weight[t, k] * y
    return out


def forward(cfg, w, ids, margins=None, streams=None):
    """float64 logits [T, vocab]; margins: list that receives every routed layer's per-token margin;
    streams: list that receives the residual stream after every layer."""
    x = w["embed"][np.asarray(ids)]
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    rows = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mx = layer["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        src = mx.get("kv_from")
        if src is None:
            rows[i] = latent_rows(h, w, p + "mix.", mx, eps)
            src = i
        x = x + m * rms_norm(latent_attention(h, w, p + "mix.", mx, eps, rows[src]), w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            x = x + m * rms_norm(routed_experts(h, w, p + "mlp.", layer["mlp"], margins), w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.copy())
    return (rms_norm(x, w["final.norm"], eps) @ w["embed"].T) * cfg["logit_scale"]


def min_margin(cfg, w, ids):
    margins = []
    forward(cfg, w, ids, margins)
    return min((float(m.min()) for m in margins), default=math.inf)


def generate_greedy(cfg, w, prompt, max_new_tokens):
    ids = list(prompt)
    for _ in range(max_new_tokens):
        ids.append(int(np.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
