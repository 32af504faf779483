"""Throughput of the Munazen design at layer sizes of real models (random weights), beside the Llama engine at equal width, depth and
head geometry: prompt tokens per second of one whole prompt, and decoded tokens per second of 1 and 4 requests stepping together at a
context of about the prompt's length. Used by ``bench.py --hybrid``; prints one JSON object per size.

Timing: CUDA events on the launching stream around each repetition, 3 warm-ups, the median of 5 (prefill) or of 30 steps (decode); the
L2 is flushed between prefill repetitions by the run itself (weights + activations of every size exceed 126 MB). Roofline fractions use
the measured peaks (MEASURED_PEAKS.json): prefill = algorithmic matrix-product flops / time against the sustained dense bf16 rate,
decode = bytes of every weight once + the caches and states read per step / time against the copy bandwidth."""
from __future__ import annotations

import json
import statistics

import numpy as np

SIZES = {
    # name: width, layer pattern repeats ([gla, parallel, parallel, parallel] each), prompt length
    "w1024": dict(width=1024, repeats=2, prompt=2048),
    "w2048": dict(width=2048, repeats=2, prompt=2048),
    "w4096": dict(width=4096, repeats=1, prompt=2048),
}


def munazen_config(width: int, repeats: int, vocab: int = 32000) -> dict:
    heads = width // 128
    par = {"type": "parallel",
           "mixer": {"left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                              "rot": {"dims": 64, "base": 500000.0, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}},
                     "right": {"width": width, "blocks": heads, "conv": 4}, "left_scale": 1.0, "right_scale": 1.0},
           "mlp": {"kind": "dense", "ff": 4 * width}}
    gla = {"type": "gla", "mixer": {"heads": heads, "dim": 64, "vdim": 128, "tau": 16.0}, "mlp": {"kind": "dense", "ff": 4 * width}}
    return {"architecture": "Munazen", "vocab": vocab, "width": width, "streams": 2, "norm": {"eps": 1e-6, "groups": 4},
            "layers": [gla, par, par, par] * repeats, "loop": {"start": 0, "stop": 0, "times": 1}}


def random_munazen_weights(cfg: dict, device, seed: int = 0) -> dict:
    """Random bf16 tensors under the design's tensor names, made on the device."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    d, s = cfg["width"], cfg["streams"]

    def mat(n_out, n_in, gain=1.0):
        return (torch.randn(n_out, n_in, generator=g, device=device) * (gain / n_in ** 0.5)).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)

    w = {"embed": torch.randn(cfg["vocab"], d, generator=g, device=device).to(torch.bfloat16), "head": mat(cfg["vocab"], d), "final.norm": vec(d, 1.0)}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        for q in (1, 2) if l.get("mlp") else (1,):
            w[f"{p}norm{q}"] = vec(d, 1.0)
            w[f"{p}hc{q}.in"], w[f"{p}hc{q}.out"] = vec(s, 1.0 / s, 0.1), vec(s, 1.0, 0.1)
            w[f"{p}hc{q}.mix"] = (torch.eye(s, device=device) + 0.1 * torch.randn(s, s, generator=g, device=device)).to(torch.bfloat16)
        m = l["mixer"]
        if l["type"] == "parallel":
            a, r = m["left"], m["right"]
            H, G, dk, dv, W, B = a["heads"], a["kv_heads"], a["dim"], a["vdim"], r["width"], r["blocks"]
            for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                w[p + f"mix.left.{n}"], w[p + f"mix.left.{n}.b"] = mat(rows, d), vec(rows)
            w[p + "mix.left.g"], w[p + "mix.left.o"], w[p + "mix.left.o.b"] = mat(H, d), mat(d, H * dv), vec(d)
            for n in ("y", "x"):
                w[p + f"mix.right.{n}"], w[p + f"mix.right.{n}.b"] = mat(W, d), vec(W)
            w[p + "mix.right.conv"], w[p + "mix.right.conv.b"] = (0.5 * torch.randn(W, r["conv"], generator=g, device=device)).to(torch.bfloat16), vec(W)
            for n in ("ra", "ri"):
                w[p + f"mix.right.{n}"] = (torch.randn(B, W // B, W // B, generator=g, device=device) / (W // B) ** 0.5).to(torch.bfloat16)
                w[p + f"mix.right.{n}.b"] = vec(W).reshape(B, W // B)
            w[p + "mix.right.lam"], w[p + "mix.right.o"] = vec(W, -1.0, 1.5), mat(d, W)
        else:
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"] = mat(H * dk, d), mat(H * dk, d), mat(H * dv, d), mat(H * dv, d)
            w[p + "mix.o"], w[p + "mix.norm"] = mat(d, H * dv), vec(dv, 1.0)
            w[p + "mix.a1"], w[p + "mix.a2"], w[p + "mix.a2.b"] = mat(16, d), mat(H * dk, 16, 2.0), vec(H * dk, 1.0, 1.0)
        if l.get("mlp"):
            ff = l["mlp"]["ff"]
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, d), mat(d, ff)
            w[p + "mlp.act"] = torch.tensor([0.6, 0.3, -0.2, 0.05], device=device).to(torch.bfloat16)
    return w


def _matrix_params(w: dict) -> int:
    return sum(t.numel() for n, t in w.items() if t.dim() >= 2 and n != "embed")


def _time(fn, reps, warmup=3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ms.append(a.elapsed_time(b))
    return statistics.median(ms)


def _time_wall(fn, reps, warmup=1):
    """For an engine that runs on a stream of its own: wall clock around the call and a device-wide synchronisation."""
    import time

    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        ms.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(ms)


def bench_munazen(name: str, hbm_gbs: float, tflops: float) -> dict:
    import torch

    from .config import BF16, MunazenConfig
    from .models.munazen import MunazenModel
    from .seqengine import SequenceEngine
    from .seqops import Ops
    size = SIZES[name]
    dev = torch.device("cuda")
    cfg = munazen_config(size["width"], size["repeats"])
    w = random_munazen_weights(cfg, dev)
    params = _matrix_params(w)
    ops = Ops(BF16)
    model = MunazenModel(MunazenConfig.from_dict(cfg), w, ops, dev)
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
    prefill_launches = (ops.launches - l0) // 8
    out = {"model": f"munazen-{name}", "width": size["width"], "layers": len(cfg["layers"]), "matrix_params": params, "prompt_len": T,
           "prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_sec": round(T / prefill_ms * 1e3, 1),
           "prefill_gemm_tflops": round(2.0 * params * T / prefill_ms / 1e9, 1), "prefill_launches": prefill_launches}
    out["prefill_fraction_of_measured_bf16_peak"] = round(out["prefill_gemm_tflops"] / tflops, 3)
    # bytes a decoding step must read: every matrix once (bf16), the keys and values of the context, the recurrent states
    kv_bytes = sum(2 * T * l["mixer"]["left"]["kv_heads"] * (l["mixer"]["left"]["dim"] + l["mixer"]["left"]["vdim"]) for l in cfg["layers"] if l["type"] == "parallel")
    state_bytes = sum(4 * (l["mixer"]["heads"] * l["mixer"]["dim"] * l["mixer"]["vdim"] * 2 if l["type"] == "gla" else l["mixer"]["right"]["width"] * 2 * l["mixer"]["right"]["conv"])
                      for l in cfg["layers"])
    for n in (1, 4):
        slots = [eng.admit() for _ in range(n)]
        eng.run([(s, prompt, []) for s in slots])
        tok = [int(prompt[-1])] * n

        def step():
            eng.run([(s, [t], [0]) for s, t in zip(slots, tok)])

        ms = _time(step, 30, warmup=4)
        bytes_step = 2.0 * params + n * (kv_bytes + state_bytes)
        out[f"decode{n}_ms_per_step"] = round(ms, 4)
        out[f"decode{n}_tokens_per_sec"] = round(n / ms * 1e3, 1)
        out[f"decode{n}_fraction_of_measured_hbm"] = round(bytes_step / (ms * 1e-3) / (hbm_gbs * 1e9), 3)
        for s in slots:
            eng.release(s)
    out["graph_replays"] = eng.graph_replays
    return out


def bench_llama(name: str, hbm_gbs: float, tflops: float, size: dict | None = None) -> dict:
    """The closest model of the framework at the same width, depth and head geometry: its batched tensor-core prefill and its
    one-sequence decode step (device-resident greedy loop)."""
    import torch

    from .config import BF16, ModelShape
    from .engine import Engine
    size = size or SIZES[name]
    d, layers, T = size["width"], 4 * size["repeats"], size["prompt"]
    heads = d // 128
    inter = ((8 * d // 3) + 255) // 256 * 256
    ms = ModelShape(32000, 128, d, max(1, heads // 4) * 128, inter, T + 512, layers, heads, max(1, heads // 4))
    eng = Engine(ms, w_dtype=BF16, kv_dtype=BF16, mega=True, mega_v2=True, mega_fuse_down=True).load_synthetic(7)
    ids = np.random.default_rng(1).integers(1, 32000, size=T).astype(np.int32)
    params = layers * (2 * d * d + 2 * ms.kv_hidden * d + 3 * inter * d) + 32000 * d
    out = {"model": f"llama-{name}", "width": d, "layers": layers, "matrix_params": params, "prompt_len": T, "mode": eng.mode}
    if eng.prefill_supported:
        pm = _time_wall(lambda: eng.prefill(ids), 5, warmup=2)
        out.update(prefill_ms=round(pm, 3), prefill_tokens_per_sec=round(T / pm * 1e3, 1), prefill_gemm_tflops=round(2.0 * params * T / pm / 1e9, 1))
        out["prefill_fraction_of_measured_bf16_peak"] = round(out["prefill_gemm_tflops"] / tflops, 3)
    eng.prefill(ids) if eng.prefill_supported else eng.greedy(ids.tolist(), T)
    n_steps = 64

    def steps():
        eng.enqueue_steps(n_steps)

    dm = _time_wall(steps, 3, warmup=1) / n_steps
    out.update(decode1_ms_per_step=round(dm, 4), decode1_tokens_per_sec=round(1e3 / dm, 1),
               decode1_fraction_of_measured_hbm=round(ms.step_bytes(T, BF16, BF16) / (dm * 1e-3) / (hbm_gbs * 1e9), 3))
    eng.close()
    return out


def main(sizes, hbm_gbs: float, tflops: float) -> list:
    res = []
    for name in sizes:
        for fn in (bench_munazen, bench_llama):
            try:
                r = fn(name, hbm_gbs, tflops)
            except Exception as ex:   # one size that does not fit or run must not hide the others
                r = {"model": f"{fn.__name__[6:]}-{name}", "error": f"{type(ex).__name__}: {ex}"[:300]}
            print(json.dumps(r), flush=True)
            res.append(r)
    return res
