"""Plain, slow restatement of the Munazen design in float64 numpy: one function per mechanism, token by token where the design is
recurrent. Test infrastructure only: it shares no code with the product package and is written for clarity, not speed.

Notation: T tokens of one sequence, d model width; weights arrive as a dict name -> float64 array with the names of the weight file.
"""
from __future__ import annotations

import math

import numpy as np


# ---------------------------------------------------------------- element-wise helpers
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """Rows of x divided by their root mean square (eps inside the root)."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


# ---------------------------------------------------------------- norms
def group_rms_norm(x, w, groups, eps):
    """x [T, d] cut into `groups` consecutive parts, each part scaled to unit rms, then the whole times w."""
    T, d = x.shape
    parts = x.reshape(T, groups, d // groups)
    return unit_rms(parts, eps).reshape(T, d) * w


# ---------------------------------------------------------------- rotary angles
def rotary_frequencies(dims, base, scaling=None):
    """Returns (freq [dims/2], magnitude): the angle of pair i at position p is p * freq[i]; cos and sin are multiplied by magnitude."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, angle, magnitude=1.0, layout="interleaved"):
    """x [..., n] with n = 2 * angle.shape[-1]: every pair (u, v) -> (u cos - v sin, v cos + u sin)."""
    c, s = np.cos(angle) * magnitude, np.sin(angle) * magnitude
    out = np.empty_like(x)
    if layout == "interleaved":
        u, v = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = u * c - v * s
        out[..., 1::2] = v * c + u * s
    else:
        half = x.shape[-1] // 2
        u, v = x[..., :half], x[..., half:]
        out[..., :half] = u * c - v * s
        out[..., half:] = v * c + u * s
    return out


# ---------------------------------------------------------------- softmax attention with rotated values and a head gate
def gated_rotary_attention(h, W, pre, cfg, layout="interleaved"):
    """The left half of the parallel mixer. h [T, d]; returns [T, d]."""
    T = h.shape[0]
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    rot = cfg["rot"]
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).reshape(T, H, dk)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).reshape(T, G, dk)
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).reshape(T, G, dv)
    gate = sigmoid(h @ W[pre + "g"].T)                                     # [T, H]
    pos = np.arange(T, dtype=np.float64)
    rd = rot["dims"]
    f, mag = rotary_frequencies(rd, rot["base"], rot.get("scaling"))
    ang = pos[:, None, None] * f[None, None, :]
    q[..., :rd] = rotate(q[..., :rd], ang, mag, layout)
    k[..., :rd] = rotate(k[..., :rd], ang, mag, layout)
    fv = rot["base"] ** (-2.0 * np.arange(dv // 2, dtype=np.float64) / dv)
    angv = pos[:, None, None] * fv[None, None, :]
    v = rotate(v, angv, 1.0, layout)                                       # what the cache holds
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * cfg["scale"]
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[:, hd] = p @ v[:, g]
    out = rotate(out, -angv, 1.0, layout)                                  # turned back by the query's own position
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ W[pre + "o"].T + W[pre + "o.b"]


# ---------------------------------------------------------------- gated linear recurrent unit with a short convolution
def causal_conv(x, w, b):
    """x [T, C]; w [C, taps], the last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    out = np.zeros((T, C))
    for t in range(T):
        out[t] = (padded[t:t + taps].T * w).sum(axis=1) + b
    return out


def gated_linear_recurrent(h, W, pre, cfg):
    """The right half of the parallel mixer. h [T, d]; returns [T, d]."""
    T = h.shape[0]
    width, blocks = cfg["width"], cfg["blocks"]
    y = gelu_tanh(h @ W[pre + "y"].T + W[pre + "y.b"])
    u = causal_conv(h @ W[pre + "x"].T + W[pre + "x.b"], W[pre + "conv"], W[pre + "conv.b"])
    ub = u.reshape(T, blocks, width // blocks)
    r = sigmoid(np.einsum("tbi,boi->tbo", ub, W[pre + "ra"]) + W[pre + "ra.b"]).reshape(T, width)
    i = sigmoid(np.einsum("tbi,boi->tbo", ub, W[pre + "ri"]) + W[pre + "ri.b"]).reshape(T, width)
    a = np.exp(-8.0 * r * softplus(W[pre + "lam"]))
    S = np.zeros(width)
    out = np.zeros((T, width))
    for t in range(T):
        S = a[t] * S + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ W[pre + "o"].T


# ---------------------------------------------------------------- gated linear attention
def gated_linear_attention(h, W, pre, cfg, eps):
    T = h.shape[0]
    H, dk, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ W[pre + "k"].T).reshape(T, H, dk)
    v = (h @ W[pre + "v"].T).reshape(T, H, dv)
    z = (h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / cfg["tau"])).reshape(T, H, dk)
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    o = unit_rms(o, eps) * W[pre + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T


# ---------------------------------------------------------------- feed-forward
def polynorm_ff(h, W, pre, eps):
    z = h @ W[pre + "up"].T
    a, b, c, e = W[pre + "act"]
    act = a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e
    return act @ W[pre + "down"].T


# ---------------------------------------------------------------- the model
def layer_runs(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def mixer(h, W, li, layer, cfg, layout):
    m, pre = layer["mixer"], f"l{li}.mix."
    if layer["type"] == "gla":
        return gated_linear_attention(h, W, pre, m, cfg["norm"]["eps"])
    if layer["type"] == "parallel":
        return (m["left_scale"] * gated_rotary_attention(h, W, pre + "left.", m["left"], layout)
                + m["right_scale"] * gated_linear_recurrent(h, W, pre + "right.", m["right"]))
    raise ValueError(layer["type"])


def forward(cfg, W, tokens, layout="interleaved", want_layers=False):
    """Whole-sequence forward of one request. Returns logits [T, vocab] (and the stream sum after every layer run)."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps, groups, ns = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["streams"]
    x0 = W["embed"][np.asarray(tokens)]
    xs = [x0.copy() for _ in range(ns)]
    after = []
    for li in layer_runs(cfg):
        layer = cfg["layers"][li]
        subs = [(1, lambda h: mixer(h, W, li, layer, cfg, layout))]
        if layer.get("mlp"):
            subs.append((2, lambda h: polynorm_ff(h, W, f"l{li}.mlp.", eps)))
        for q, fn in subs:
            hc = f"l{li}.hc{q}."
            u = sum(W[hc + "in"][s] * xs[s] for s in range(ns))
            y = fn(group_rms_norm(u, W[f"l{li}.norm{q}"], groups, eps))
            xs = [sum(W[hc + "mix"][s, t] * xs[s] for s in range(ns)) + W[hc + "out"][t] * y for t in range(ns)]
        after.append(sum(xs))
    x = group_rms_norm(sum(xs), W["final.norm"], groups, eps)
    logits = x @ W["head"].T
    return (logits, np.stack(after)) if want_layers else logits
