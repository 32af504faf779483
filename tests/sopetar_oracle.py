"""Plain, slow restatement of the Sopetar design in float64 numpy: one function per mechanism, a whole sequence at a time with explicit
visibility masks. Test infrastructure only: it shares no code with the product package and is written for clarity, not speed.

Notation: T tokens of one sequence at positions 0 .. T-1, d model width; weights arrive as a dict name -> float64 array with the names
of the weight file; ``cfg`` is the parsed config.json.
"""
from __future__ import annotations

import math

import numpy as np

GLU_ALPHA = 1.702        # the feed-forward's gate is g * sigmoid(GLU_ALPHA * g)
SLOPE_SPAN = 8.0         # head h of H is charged 2^(-SLOPE_SPAN (h+1) / H) per position of distance


# ---------------------------------------------------------------- element-wise helpers and norms
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def layer_norm(x, w, b, eps):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


# ---------------------------------------------------------------- positions
def rotate_pairs(x, pos, dims, base):
    """x [T, ..., n]: the first `dims` entries of the last axis are rotated pairwise ((0,1), (2,3), ...) by pos * base^(-2i/dims)."""
    out = np.array(x, dtype=np.float64, copy=True)
    i = np.arange(dims // 2, dtype=np.float64)
    angle = np.asarray(pos, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)          # [T, dims/2]
    angle = angle.reshape((x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,))
    c, s = np.cos(angle), np.sin(angle)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T, size=None, keep_first=0):
    """[T, T] booleans: query i sees key j when j <= i and (i - j < size or j < keep_first); size None = no window."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    see = j <= i
    if size is not None:
        see &= (i - j < size) | (j < keep_first)
    return see


def distance_slopes(heads):
    return np.array([2.0 ** (-SLOPE_SPAN * (h + 1) / heads) for h in range(heads)])


# ---------------------------------------------------------------- mixers
def capped_biased_attention(h, W, pre, m, eps, v_first=None):
    """The 'attention' mixer: biased projections, q / k / v scaled to unit rms per head, scores capped by tanh and charged a slope per
    position of distance, a sliding window that keeps the first tokens. Returns (output [T, d], the values that were attended [T, G, vdim])."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).reshape(T, H, dk)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).reshape(T, G, dk)
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).reshape(T, G, dv)
    q, k, v = unit_rms(q, eps), unit_rms(k, eps), unit_rms(v, eps)
    if v_first is not None:
        lam = float(W[pre + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    mask = m.get("mask") or {}
    see = visible(T, mask.get("size"), mask.get("keep_first", 0))
    dist = (np.arange(T)[:, None] - np.arange(T)[None, :]).astype(np.float64)
    slopes = distance_slopes(H)
    cap = m.get("softcap")
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * np.tanh(s / cap)
        s = s - slopes[hd] * dist
        s = np.where(see, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[:, hd] = p @ v[:, g]
    return out.reshape(T, H * dv) @ W[pre + "o"].T, v


def latent_attention(h, W, pre, m, eps):
    """The 'latent_attention' mixer: keys and values are expanded from one normed latent vector per token; a rotated key part is shared
    by the heads; the softmax's denominator holds one more term exp(sink) per head; a sigmoid gate per head."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    q = (h @ W[pre + "q"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], pos, m["rot"]["dims"], m["rot"]["base"])
    low = h @ W[pre + "dkv"].T
    c = unit_rms(low[:, :R], eps) * W[pre + "dkv.norm"]
    k_rot = rotate_pairs(low[:, R:], pos, m["rot"]["dims"], m["rot"]["base"])                # [T, dr], one for all heads
    k_plain = (c @ W[pre + "uk"].T).reshape(T, H, dn)
    v = (c @ W[pre + "uv"].T).reshape(T, H, dv)
    mask = m.get("mask") or {}
    see = visible(T, mask.get("size"), mask.get("keep_first", 0))
    gate = sigmoid(h @ W[pre + "g"].T)                                                       # [T, H]
    out = np.zeros((T, H, dv))
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        s = np.where(see, s, -np.inf)
        sink = float(W[pre + "sink"][hd])
        top = np.maximum(s.max(axis=1, keepdims=True), sink)
        p = np.exp(s - top)
        p /= p.sum(axis=1, keepdims=True) + np.exp(sink - top)
        out[:, hd] = (p @ v[:, hd]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * dv) @ W[pre + "o"].T


# ---------------------------------------------------------------- feed-forward
def clamped_glu(h, W, pre, mlp):
    lim = mlp["limit"]
    g = np.minimum(h @ W[pre + "gate"].T + W[pre + "gate.b"], lim)
    u = np.clip(h @ W[pre + "up"].T + W[pre + "up.b"], -lim, lim)
    return (g * sigmoid(GLU_ALPHA * g) * (u + 1.0)) @ W[pre + "down"].T + W[pre + "down.b"]


# ---------------------------------------------------------------- the model
def forward(cfg, W, tokens, taps=None):
    """Logits [T, vocab] of one sequence. ``taps``, if a list, receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    history = [x]                                 # the embedding output and every layer's own result
    v_first = None
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        if l["type"] == "attention":
            share = bool(l["mixer"].get("v_mix"))
            y, v = capped_biased_attention(h, W, p + "mix.", l["mixer"], eps, v_first if share else None)
            if share and v_first is None:
                v_first = v
        elif l["type"] == "latent_attention":
            y = latent_attention(h, W, p + "mix.", l["mixer"], eps)
        else:
            raise ValueError(l["type"])
        if l.get("mlp") is not None:
            y = y + clamped_glu(h, W, p + "mlp.", l["mlp"])
        history.append(x + y)
        coef = W[p + "dwa"]
        x = sum(coef[j] * history[j] for j in range(i + 2))
        if taps is not None:
            taps.append(x)
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return x @ W["head"].T
