"""Plain, slow Dokulorn in numpy: the oracle the engine is compared with.

Whole sequences, no cache, no batching, float64, one function per mechanism, token by token and key by key; it
shares no code with the package (only the file readers of the other oracle).

    layer:    x <- n1(a x + mixer(x));  x <- n2(a x + ff(x))  (ff may be absent);  n(v) = v / sqrt(mean(v^2) + eps) (1 + w)
    mixers:   retention, or a pair (softmax attention with a sink | lightning attention), see the functions
    output:   logits = E n_final(x), E the embedding table; the embedding itself is E[id] * scale
"""
from __future__ import annotations

import math
import os

import numpy as np

from plain_gemma2 import read_config, read_safetensors  # noqa: F401  (file formats only)


def load_folder(folder):
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    return read_config(folder), {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


def unit_rms(v, eps):
    """v divided by its root mean square, eps inside the root."""
    return v / math.sqrt(float(np.mean(v * v)) + eps)


def turn(v, pos, rot):
    """One head's vector at position pos: value i and value i + n/2 of its first n = rot['dims'] values form a pair
    that turns by pos * base^(-2i/n); the rest pass."""
    n, out = rot["dims"], np.array(v, dtype=np.float64)
    for i in range(n // 2):
        ang = pos * rot["base"] ** (-2.0 * i / n)
        c, s = math.cos(ang), math.sin(ang)
        u, w = v[i], v[i + n // 2]
        out[i], out[i + n // 2] = u * c - w * s, w * c + u * s
    return out


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def decay_recurrence(q, k, v, decay):
    """One head: S_t = decay S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t.  q, k [T, d], v [T, e] -> [T, e]."""
    S = np.zeros((q.shape[1], v.shape[1]))
    out = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        S = decay * S + np.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out


def retention(w, p, m, h, eps):
    """q, k rotated, k times dim^-1/2, the recurrence per head, each head's o divided by its root mean square,
    times silu(W_g h), then W_o."""
    T, H, d, e = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    o = np.zeros((T, H * e))
    for a in range(H):
        qa = np.stack([turn(q[t, a * d:(a + 1) * d], t, m["rot"]) for t in range(T)])
        ka = np.stack([turn(k[t, a * d:(a + 1) * d], t, m["rot"]) for t in range(T)]) * d ** -0.5
        oa = decay_recurrence(qa, ka, v[:, a * e:(a + 1) * e], m["decay"][a])
        for t in range(T):
            o[t, a * e:(a + 1) * e] = unit_rms(oa[t], eps)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def sink_attention(w, p, m, h, eps):
    """Grouped-query softmax attention: q, k rotated and then divided by their root mean square, score times
    `scale`, soft-capped, causal; the denominator also holds exp(sink) of the head; the heads times sigmoid(W_g h),
    then W_o."""
    T, H, G, d, e = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    cap = m["softcap"]
    o = np.zeros((T, H * e))
    kn = [[unit_rms(turn(k[t, g * d:(g + 1) * d], t, m["rot"]), eps) for t in range(T)] for g in range(G)]
    for a in range(H):
        g = a // (H // G)
        sink = float(w[p + "sink"][a])
        for t in range(T):
            qa = unit_rms(turn(q[t, a * d:(a + 1) * d], t, m["rot"]), eps)
            s = np.array([cap * math.tanh(float(qa @ kn[g][j]) * m["scale"] / cap) for j in range(t + 1)])
            top = max(float(s.max()), sink)
            ex = np.exp(s - top)
            den = ex.sum() + math.exp(sink - top)
            o[t, a * e:(a + 1) * e] = (ex / den) @ v[:t + 1, g * e:(g + 1) * e]
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def lightning(w, p, m, h, eps):
    """silu on q, k, v, the recurrence per head, the concatenated heads normed together with a plain weight, times
    sigmoid(W_g h), then W_o."""
    T, H, d, e = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q, k, v = silu(h @ w[p + "q"].T), silu(h @ w[p + "k"].T), silu(h @ w[p + "v"].T)
    o = np.concatenate([decay_recurrence(q[:, a * d:(a + 1) * d], k[:, a * d:(a + 1) * d], v[:, a * e:(a + 1) * e], m["decay"][a])
                        for a in range(H)], axis=1)
    o = np.stack([unit_rms(o[t], eps) for t in range(T)]) * w[p + "norm"]
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def pair(w, p, m, h, eps):
    """Half the sum of the two mixers' results, each normed over the width with its plain weight."""
    left, right = sink_attention(w, p + "left.", m["left"], h, eps), lightning(w, p + "right.", m["right"], h, eps)
    return np.stack([0.5 * (unit_rms(left[t], eps) * w[p + "left.out"] + unit_rms(right[t], eps) * w[p + "right.out"])
                     for t in range(h.shape[0])])


def feed_forward(w, p, h):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def norm_after_sum(x, branch, alpha, weight, eps):
    return np.stack([unit_rms(alpha * x[t] + branch[t], eps) * (1.0 + weight) for t in range(x.shape[0])])


def forward(cfg, w, ids, layers_out=None):
    """Logits [T, vocab] of one whole sequence."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][np.asarray(ids)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "retention":
            a = retention(w, p + "mix.", layer["mixer"], x, eps)
        else:
            a = pair(w, p + "mix.", layer["mixer"], x, eps)
        x = norm_after_sum(x, a, alpha, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = norm_after_sum(x, feed_forward(w, p + "mlp.", x), alpha, w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    x = np.stack([unit_rms(x[t], eps) * (1.0 + w["final.norm"]) for t in range(x.shape[0])])
    return x @ w["embed"].T


def generate_greedy(cfg, w, ids, n):
    ids = list(ids)
    for _ in range(n):
        ids.append(int(np.argmax(forward(cfg, w, ids)[-1])))
    return ids
