"""Test helpers for the Sopetar design: small configurations, random weights written as a model folder (config.json + model.safetensors in
bf16) and the error measure the tests share. Nothing here is used by the product package."""
from __future__ import annotations

import numpy as np

from munazen_testlib import bf16_round, logit_error, to_bf16_bits, write_model  # noqa: F401  (the file format and the measure are the same)


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, softcap=30.0, size=20, keep_first=3, v_mix=False, ff=40, limit=1.25):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if softcap:
        m["softcap"] = softcap
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep_first}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def latent_layer(heads=3, dim=8, rot_dim=12, vdim=20, kv_rank=40, scale=0.2, rot_dims=None, base=1000.0, size=20, keep_first=None, ff=40, limit=1.25):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}
    if size is not None:
        m["mask"] = {"size": size}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def make_config(layers, vocab=83, width=48, eps=1e-5, embedding_scale=2.5):
    return {"architecture": "Sopetar", "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale}, "norm": {"eps": eps}, "layers": layers}


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """name -> float32 array of bf16-representable values (so that both storage types hold the same numbers)."""
    rng = np.random.default_rng(seed)
    d = cfg["width"]
    w = {}

    def mat(n_out, n_in, gain=1.0):
        return bf16_round(rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in))

    def vec(n, mean=0.0, std=0.1):
        return bf16_round(mean + std * rng.standard_normal(n))

    w["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], d)))
    w["head"] = mat(cfg["vocab"], d)
    w["final.norm"], w["final.norm.b"] = vec(d, 1.0), vec(d)
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"], w[p + "norm1.b"] = vec(d, 1.0), vec(d)
        m = l["mixer"]
        if l["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.q.b"] = mat(H * dk, d, 1.5), vec(H * dk)
            w[p + "mix.k"], w[p + "mix.k.b"] = mat(G * dk, d, 1.5), vec(G * dk)
            w[p + "mix.v"], w[p + "mix.v.b"] = mat(G * dv, d), vec(G * dv)
            w[p + "mix.vmix"] = bf16_round(np.array(0.3 + 0.1 * rng.standard_normal()))
            w[p + "mix.o"] = mat(d, H * dv)
        else:
            H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "mix.q"] = mat(H * (dn + dr), d, 2.0)
            w[p + "mix.dkv"] = mat(R + dr, d, 2.0)
            w[p + "mix.dkv.norm"] = vec(R, 1.0, 0.2)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * dn, R), mat(H * dv, R)
            w[p + "mix.sink"] = vec(H, 2.0, 1.0)          # large enough to take a visible share of the denominator
            w[p + "mix.g"] = mat(H, d, 2.0)
            w[p + "mix.o"] = mat(d, H * dv)
        if l.get("mlp"):
            ff = l["mlp"]["ff"]
            w[p + "mlp.gate"], w[p + "mlp.gate.b"] = mat(ff, d, 2.0), vec(ff)       # wide enough that the clamps bite
            w[p + "mlp.up"], w[p + "mlp.up.b"] = mat(ff, d, 2.0), vec(ff)
            w[p + "mlp.down"], w[p + "mlp.down.b"] = mat(d, ff), vec(d)
        w[p + "dwa"] = bf16_round(np.concatenate([0.15 * rng.standard_normal(i + 1), [1.0 + 0.1 * rng.standard_normal()]]))
    return {k: np.asarray(v, dtype=np.float32) for k, v in w.items()}
