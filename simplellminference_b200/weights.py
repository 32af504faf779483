"""Weights of a config.json model: model.safetensors -> device tensors in the storage type of the run.

The file format is read here directly (8-byte little-endian header length, JSON header name -> dtype / shape / data_offsets, raw data),
like convert.read_safetensors, but the values keep their stored bits: a bf16 matrix goes to the device as bf16 (bf16 mode) or is widened
exactly to fp32 (fp32 mode); integer tables stay int32. Which tensors are matrices (kept in the storage type, operands of matrix
products) and which are small fp32 vectors is the model's business: ``load`` returns everything in the storage type and the mechanisms
call .float() on what they need in fp32."""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch

from .config import BF16


def read_raw(path: str) -> dict:
    """name -> (dtype string, shape, numpy array of the stored bits: uint16 for BF16 / F16, float32, int32)."""
    out = {}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
        for name, info in header.items():
            if name == "__metadata__":
                continue
            dt, (b0, b1) = info["dtype"], info["data_offsets"]
            np_dt = {"BF16": "<u2", "F16": "<f2", "F32": "<f4", "I32": "<i4"}.get(dt)
            if np_dt is None:
                raise ValueError(f"{name}: dtype {dt} not supported (BF16, F16, F32, I32)")
            f.seek(base + b0)
            out[name] = (dt, tuple(info["shape"]), np.frombuffer(f.read(b1 - b0), dtype=np_dt).reshape(info["shape"]))
    return out


def load(model_dir: str, w_dtype: int, device) -> dict:
    """Every tensor of model.safetensors on ``device``: floating tensors as bf16 (w_dtype BF16) or fp32, integer tensors as int32."""
    target = torch.bfloat16 if w_dtype == BF16 else torch.float32
    out = {}
    for name, (dt, _, a) in read_raw(os.path.join(model_dir, "model.safetensors")).items():
        if dt == "I32":
            out[name] = torch.from_numpy(a.copy()).to(device)
        elif dt == "BF16":
            out[name] = torch.from_numpy(a.copy().view(np.int16)).view(torch.bfloat16).to(device).to(target)
        else:
            out[name] = torch.from_numpy(a.astype(np.float32)).to(device).to(target)
    return out
