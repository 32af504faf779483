"""Test helpers for the Munazen design: small random configurations, random weights written as a model folder (config.json +
model.safetensors in bf16), and the error measure the tests share. Nothing here is used by the product package."""
from __future__ import annotations

import json
import os
import struct

import numpy as np


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_round(a: np.ndarray) -> np.ndarray:
    return (to_bf16_bits(a).astype(np.uint32) << 16).view(np.float32).reshape(np.shape(a))


def parallel_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, base=10000.0, scaling=None, scale=0.25, width=32, blocks=2, conv=3,
                   left_scale=0.9, right_scale=1.3, ff=48):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot},
                      "right": {"width": width, "blocks": blocks, "conv": conv}, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def gla_layer(heads=2, dim=20, vdim=12, tau=8.0, ff=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_config(layers, vocab=97, width=48, streams=3, groups=2, eps=1e-5, loop=None):
    return {"architecture": "Munazen", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps, "groups": groups},
            "layers": layers, "loop": loop or {"start": 0, "stop": 0, "times": 1}}


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """name -> float32 array of bf16-representable values (so that both storage types hold the same numbers)."""
    rng = np.random.default_rng(seed)
    d, s = cfg["width"], cfg["streams"]
    w = {}

    def mat(n_out, n_in, gain=1.0):
        return bf16_round(rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in))

    def vec(n, mean=0.0, std=0.1):
        return bf16_round(mean + std * rng.standard_normal(n))

    w["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], d)))
    w["head"] = mat(cfg["vocab"], d)
    w["final.norm"] = vec(d, 1.0)
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [1] + ([2] if l.get("mlp") else [])
        for q in subs:
            w[f"{p}norm{q}"] = vec(d, 1.0)
            w[f"{p}hc{q}.in"] = vec(s, 1.0 / s, 0.2)
            w[f"{p}hc{q}.out"] = vec(s, 1.0, 0.3)
            w[f"{p}hc{q}.mix"] = bf16_round(np.eye(s) + 0.2 * rng.standard_normal((s, s)))
        m = l["mixer"]
        if l["type"] == "parallel":
            a, r = m["left"], m["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            w[p + "mix.left.q"], w[p + "mix.left.q.b"] = mat(H * dk, d, 1.5), vec(H * dk)
            w[p + "mix.left.k"], w[p + "mix.left.k.b"] = mat(G * dk, d, 1.5), vec(G * dk)
            w[p + "mix.left.v"], w[p + "mix.left.v.b"] = mat(G * dv, d), vec(G * dv)
            w[p + "mix.left.g"] = mat(H, d)
            w[p + "mix.left.o"], w[p + "mix.left.o.b"] = mat(d, H * dv), vec(d)
            W, B, taps = r["width"], r["blocks"], r["conv"]
            w[p + "mix.right.y"], w[p + "mix.right.y.b"] = mat(W, d), vec(W)
            w[p + "mix.right.x"], w[p + "mix.right.x.b"] = mat(W, d), vec(W)
            w[p + "mix.right.conv"], w[p + "mix.right.conv.b"] = bf16_round(rng.standard_normal((W, taps)) * 0.5), vec(W)
            w[p + "mix.right.ra"], w[p + "mix.right.ra.b"] = bf16_round(rng.standard_normal((B, W // B, W // B)) / np.sqrt(W // B)), vec(W).reshape(B, W // B)
            w[p + "mix.right.ri"], w[p + "mix.right.ri.b"] = bf16_round(rng.standard_normal((B, W // B, W // B)) / np.sqrt(W // B)), vec(W).reshape(B, W // B)
            w[p + "mix.right.lam"] = vec(W, -1.0, 1.5)
            w[p + "mix.right.o"] = mat(d, W)
        else:
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"] = mat(H * dk, d), mat(H * dk, d)
            w[p + "mix.v"], w[p + "mix.g"] = mat(H * dv, d), mat(H * dv, d)
            w[p + "mix.o"] = mat(d, H * dv)
            w[p + "mix.norm"] = vec(dv, 1.0)
            rank = 4
            w[p + "mix.a1"], w[p + "mix.a2"], w[p + "mix.a2.b"] = mat(rank, d), mat(H * dk, rank, 2.0), vec(H * dk, 1.0, 1.0)
        if l.get("mlp"):
            ff = l["mlp"]["ff"]
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, d), mat(d, ff)
            w[p + "mlp.act"] = bf16_round(np.array([0.6, 0.3, -0.2, 0.05]) + 0.05 * rng.standard_normal(4))
    return {k: np.asarray(v, dtype=np.float32) for k, v in w.items()}


def write_model(folder: str, cfg: dict, w: dict) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, a in w.items():
        raw = to_bf16_bits(a).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    return folder


def logit_error(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: rms over the vocabulary of the difference with its mean taken off, relative to the rms of the wanted logits."""
    d = np.asarray(got, dtype=np.float64) - np.asarray(want, dtype=np.float64)
    d = d - d.mean(axis=-1, keepdims=True)
    w = np.asarray(want, dtype=np.float64)
    scale = np.sqrt(((w - w.mean(axis=-1, keepdims=True)) ** 2).mean())
    return np.sqrt((d ** 2).mean(axis=-1)) / scale
