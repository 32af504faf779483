"""Model-shape presets (reference: include/model/config.h:5-17 hard-codes ONE shape; BASELINE.json names five)."""
from __future__ import annotations

from dataclasses import dataclass, asdict

F32, BF16, INT8 = 0, 1, 2
DTYPE_NAMES = {F32: "f32", BF16: "bf16", INT8: "int8"}


@dataclass(frozen=True)
class ModelShape:
    """Field-for-field the reference's model::LlamaModelConfig."""

    vocab: int
    head_dim: int
    hidden: int
    kv_hidden: int
    inter: int
    max_len: int
    layers: int
    heads: int
    kv_heads: int
    eps: float = 1e-5
    theta: float = 10000.0

    def __post_init__(self):
        if self.heads * self.head_dim != self.hidden:
            raise ValueError("heads*head_dim must equal hidden (the reference's wq/wo are d x d, model.cpp:372-378)")
        if self.kv_heads * self.head_dim != self.kv_hidden or self.heads % self.kv_heads:
            raise ValueError("inconsistent kv dims")

    def n_params(self) -> int:
        d, kv, I, L, V = self.hidden, self.kv_hidden, self.inter, self.layers, self.vocab
        return V * d + (2 * L + 1) * d + L * (2 * d * d + 2 * kv * d + 3 * I * d)

    def step_bytes(self, pos: int, w_dtype: int = BF16, kv_dtype: int = BF16, group: int = 64) -> float:
        """Algorithmic HBM bytes of one decode step at position `pos`."""
        bw = {F32: 4.0, BF16: 2.0, INT8: 1.0 + 4.0 / group}[w_dtype]
        bkv = 4.0 if kv_dtype == F32 else 2.0
        d, kv, I, L, V = self.hidden, self.kv_hidden, self.inter, self.layers, self.vocab
        return (bw * (V * d + L * (2 * d * d + 2 * kv * d + 3 * I * d)) + 4.0 * (2 * L + 1) * d + bw * d
                + bkv * 2 * L * kv * (pos + 1) + bkv * 2 * L * kv)

    def as_dict(self):
        return asdict(self)


# BASELINE.json configs (shapes only; weights are random-init)
PRESETS = {
    "stories15M": ModelShape(32000, 48, 288, 288, 768, 256, 6, 6, 6),
    "stories110M": ModelShape(32000, 64, 768, 768, 2048, 1024, 12, 12, 12),
    "tinyllama-1.1b": ModelShape(32000, 64, 2048, 256, 5632, 2048, 22, 32, 4),
    "llama2-7b": ModelShape(32000, 128, 4096, 4096, 11008, 4096, 32, 32, 32),
    # +8 positions of slack: the reference's GQA RoPE over-run limits the parity domain to pos <= S - H/KVH
    "llama3-8b": ModelShape(128256, 128, 4096, 1024, 14336, 8192 + 8, 32, 32, 8, theta=500000.0),
    # small shapes for tests
    "tiny_gqa": ModelShape(512, 32, 128, 64, 384, 48, 3, 4, 2),
    "tiny_mha_hd48": ModelShape(300, 48, 96, 96, 200, 40, 2, 2, 2),
}


# ---------------------------------------------------------------------------------------------------------------------------
# Models described by a config.json (a folder with config.json + model.safetensors). `architecture` selects the reader here and the
# model class in simplellminference_b200.models; the Llama shapes above stay what the C engine takes.
# ---------------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RotaryConfig:
    """Rotary positions on the first ``dims`` dimensions of a head; ``scaling`` = YaRN-style (factor, original, fast, slow) or None."""
    dims: int
    base: float
    scaling: dict | None = None


@dataclass(frozen=True)
class SoftmaxMixerConfig:
    heads: int
    kv_heads: int
    dim: int          # per-head query / key width
    vdim: int         # per-head value width
    scale: float
    rot: RotaryConfig


@dataclass(frozen=True)
class RecurrentMixerConfig:
    width: int
    blocks: int
    conv: int         # taps of the causal convolution


@dataclass(frozen=True)
class LinearAttentionMixerConfig:
    heads: int
    dim: int
    vdim: int
    tau: float


@dataclass(frozen=True)
class MunazenLayerConfig:
    type: str                                   # "parallel" | "gla"
    left: SoftmaxMixerConfig | None = None      # parallel
    right: RecurrentMixerConfig | None = None   # parallel
    left_scale: float = 1.0
    right_scale: float = 1.0
    gla: LinearAttentionMixerConfig | None = None
    ff: int | None = None                       # width of the dense feed-forward, None = the layer has none


@dataclass(frozen=True)
class MunazenConfig:
    """The Munazen design: every size and every constant that may differ between its models comes from config.json."""
    architecture: str
    vocab: int
    width: int
    streams: int
    norm_eps: float
    norm_groups: int
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    @staticmethod
    def from_dict(c: dict) -> "MunazenConfig":
        layers = []
        for i, l in enumerate(c["layers"]):
            m, mlp = l["mixer"], l.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
            ff = int(mlp["ff"]) if mlp is not None else None
            if l["type"] == "parallel":
                a, r = m["left"], m["right"]
                rot = a["rot"]
                layers.append(MunazenLayerConfig(
                    "parallel",
                    left=SoftmaxMixerConfig(int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"]), float(a["scale"]),
                                            RotaryConfig(int(rot["dims"]), float(rot["base"]), rot.get("scaling") or None)),
                    right=RecurrentMixerConfig(int(r["width"]), int(r["blocks"]), int(r["conv"])),
                    left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]), ff=ff))
            elif l["type"] == "gla":
                layers.append(MunazenLayerConfig("gla", gla=LinearAttentionMixerConfig(int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])),
                                                 ff=ff))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
        loop = c.get("loop") or {}
        start, stop, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
        if not (0 <= start <= stop <= len(layers)) or times < 1:
            raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        norm = c.get("norm") or {}
        return MunazenConfig(c["architecture"], int(c["vocab"]), int(c["width"]), int(c.get("streams", 1)), float(norm.get("eps", 1e-6)),
                             int(norm.get("groups", 1)), tuple(layers), start, stop, times)

    def layer_runs(self) -> list:
        """Layer indices in the order they run: the looped range repeats with the same weights (each pass has its own state)."""
        return (list(range(self.loop_start)) + list(range(self.loop_start, self.loop_stop)) * self.loop_times
                + list(range(self.loop_stop, len(self.layers))))


CONFIG_READERS = {"Munazen": MunazenConfig.from_dict}


def read_model_config(model_dir: str):
    """config.json of a model folder -> the config object of its architecture (KeyError names the architectures known here)."""
    import json
    import os
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    arch = c.get("architecture")
    if arch not in CONFIG_READERS:
        raise KeyError(f"architecture {arch!r} is not registered (known: {sorted(CONFIG_READERS)})")
    return CONFIG_READERS[arch](c)
