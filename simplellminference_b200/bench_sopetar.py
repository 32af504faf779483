"""Throughput of the Sopetar design at layer sizes of real models (random weights), beside the Llama engine at equal width, depth,
feed-forward width and head geometry: prompt tokens per second of one whole prompt, and decoded tokens per second of 1 and 4 requests
stepping together at a context of the prompt's length. Used by ``bench.py --sopetar``; prints one JSON object per size.

Timing and roofline fractions as in ``bench_hybrid`` (CUDA events on the launching stream, 3 warm-ups, medians; prefill = algorithmic
matrix-product flops against the measured sustained bf16 rate, decode = every matrix once + the cache rows inside the windows against the
measured copy bandwidth)."""
from __future__ import annotations

import json

import numpy as np

from .bench_hybrid import _matrix_params, _time, bench_llama

SIZES = {
    # name: width, layer pattern repeats ([attention, latent, latent, latent] each), prompt length
    "w1024": dict(width=1024, repeats=2, prompt=2048),
    "w2048": dict(width=2048, repeats=2, prompt=2048),
    "w4096": dict(width=4096, repeats=1, prompt=2048),
}
WINDOW = 1024


def sopetar_config(width: int, repeats: int, vocab: int = 32000) -> dict:
    heads = width // 128
    ff = ((8 * width // 3) + 255) // 256 * 256
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 50.0, "v_mix": True,
                     "mask": {"size": WINDOW, "keep_first": 4}}}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": heads, "dim": 64, "rot_dim": 64, "vdim": 64, "kv_rank": 128, "scale": 128 ** -0.5, "rot": {"dims": 64, "base": 10000.0},
                     "mask": {"size": WINDOW}}}
    return {"architecture": "Sopetar", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "layers": [att, lat, lat, lat] * repeats}


def random_sopetar_weights(cfg: dict, device, seed: int = 0) -> dict:
    """Random bf16 tensors under the design's tensor names, made on the device."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    d = cfg["width"]

    def mat(n_out, n_in, gain=1.0):
        return (torch.randn(n_out, n_in, generator=g, device=device) * (gain / n_in ** 0.5)).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)

    w = {"embed": torch.randn(cfg["vocab"], d, generator=g, device=device).to(torch.bfloat16), "head": mat(cfg["vocab"], d), "final.norm": vec(d, 1.0),
         "final.norm.b": vec(d)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        w[p + "norm1"], w[p + "norm1.b"] = vec(d, 1.0), vec(d)
        if l["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                w[p + f"mix.{n}"], w[p + f"mix.{n}.b"] = mat(rows, d), vec(rows)
            w[p + "mix.vmix"], w[p + "mix.o"] = torch.tensor(0.3, device=device).to(torch.bfloat16), mat(d, H * dv)
        else:
            H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "mix.q"], w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(H * (dn + dr), d), mat(R + dr, d), vec(R, 1.0)
            w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.sink"] = mat(H * dn, R), mat(H * dv, R), vec(H, 0.0, 1.0)
            w[p + "mix.g"], w[p + "mix.o"] = mat(H, d), mat(d, H * dv)
        ff = l["mlp"]["ff"]
        w[p + "mlp.gate"], w[p + "mlp.gate.b"], w[p + "mlp.up"], w[p + "mlp.up.b"] = mat(ff, d), vec(ff), mat(ff, d), vec(ff)
        w[p + "mlp.down"], w[p + "mlp.down.b"] = mat(d, ff), vec(d)
        w[p + "dwa"] = torch.cat([0.05 * torch.randn(i + 1, generator=g, device=device), torch.ones(1, device=device)]).to(torch.bfloat16)
    return w


def bench_sopetar(name: str, hbm_gbs: float, tflops: float) -> dict:
    import torch

    from .config import BF16, SopetarConfig
    from .models.sopetar import SopetarModel
    from .seqengine import SequenceEngine
    from .seqops import Ops
    size = SIZES[name]
    dev = torch.device("cuda")
    cfg = sopetar_config(size["width"], size["repeats"])
    w = random_sopetar_weights(cfg, dev)
    params = _matrix_params(w)
    ops = Ops(BF16)
    model = SopetarModel(SopetarConfig.from_dict(cfg), w, ops, dev)
    T = size["prompt"]
    eng = SequenceEngine(model, max_tokens=4 * (T + 128), max_seqs=4)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg["vocab"], size=T).astype(np.int32)

    def prefill():
        s = eng.admit()
        eng.run([(s, prompt, [T - 1])])
        eng.release(s)

    l0 = ops.launches
    prefill_ms = _time(prefill, 5)
    out = {"model": f"sopetar-{name}", "width": size["width"], "layers": len(cfg["layers"]), "matrix_params": params, "prompt_len": T,
           "prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_sec": round(T / prefill_ms * 1e3, 1),
           "prefill_gemm_tflops": round(2.0 * params * T / prefill_ms / 1e9, 1), "prefill_launches": (ops.launches - l0) // 8}
    out["prefill_fraction_of_measured_bf16_peak"] = round(out["prefill_gemm_tflops"] / tflops, 3)
    # cache bytes a decoding step must read per request: the rows inside each layer's window (bf16 pools)
    cache_bytes = 0
    for l in cfg["layers"]:
        m = l["mixer"]
        rows = min(T, m["mask"]["size"] + m["mask"].get("keep_first", 0))
        cache_bytes += 2 * rows * (m["kv_heads"] * (m["dim"] + m["vdim"]) if l["type"] == "attention" else m["kv_rank"] + m["rot_dim"])
    for n in (1, 4):
        slots = [eng.admit() for _ in range(n)]
        eng.run([(s, prompt, []) for s in slots])
        tok = [int(prompt[-1])] * n

        def step():
            eng.run([(s, [t], [0]) for s, t in zip(slots, tok)])

        ms = _time(step, 30, warmup=4)
        out[f"decode{n}_ms_per_step"] = round(ms, 4)
        out[f"decode{n}_tokens_per_sec"] = round(n / ms * 1e3, 1)
        out[f"decode{n}_fraction_of_measured_hbm"] = round((2.0 * params + n * cache_bytes) / (ms * 1e-3) / (hbm_gbs * 1e9), 3)
        for s in slots:
            eng.release(s)
    out["graph_replays"] = eng.graph_replays
    return out


def main(sizes, hbm_gbs: float, tflops: float) -> list:
    res = []
    for name in sizes:
        for label, fn in (("sopetar", lambda: bench_sopetar(name, hbm_gbs, tflops)), ("llama", lambda: bench_llama(name, hbm_gbs, tflops, SIZES[name]))):
            try:
                r = fn()
            except Exception as ex:   # one size that does not fit or run must not hide the others
                r = {"model": f"{label}-{name}", "error": f"{type(ex).__name__}: {ex}"[:300]}
            print(json.dumps(r), flush=True)
            res.append(r)
    return res
