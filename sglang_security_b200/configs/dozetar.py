"""Configuration of the Dozetar design: a decoder-only model over a 32-bit residual whose sublayers
read the residual itself and are normed on their OUTPUT (x += r * rmsnorm(sublayer(x)) * g).  A layer's
mixer is either a matrix-memory recurrence with exponential gates ("mlstm") or two mixers side by
side ("parallel": softmax attention with a sliding window, kept first tokens and a sink, beside a
decayed linear attention); its feed-forward is a mixture of ungated experts or absent.  Every size,
the layer order and the constants a model may choose are read from config.json."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Union

from .model_config import register_config


@dataclass
class MLSTMSpec:
    heads: int
    dim: int            # query/key size per head
    vdim: int           # value size per head
    gate_cap: float     # soft cap of the gate pre-activations (0 = none)


@dataclass
class SinkAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]       # tokens a position sees, itself included; None = all before
    keep_first: int             # leading tokens that stay visible outside the window
    rope_base: float
    rope_dims: int              # rotated leading coordinates of each head (0 = no rotation)


@dataclass
class DecayedAttentionSpec:
    heads: int
    dim: int
    vdim: int
    decay: List[float]          # one constant per head


@dataclass
class ParallelSpec:
    left: SinkAttentionSpec
    right: DecayedAttentionSpec
    left_scale: float
    right_scale: float


@dataclass
class ExpertsSpec:
    experts: int
    top: int
    ff: int


@dataclass
class DozetarLayerSpec:
    type: str                                    # "mlstm" | "parallel"
    mixer: Union[MLSTMSpec, ParallelSpec]
    mlp: Optional[ExpertsSpec]


@dataclass
class DozetarConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_softcap: float                         # 0 = none
    layers: List[DozetarLayerSpec] = field(default_factory=list)

    @property
    def num_layers(self) -> int:
        return len(self.layers)


def _sink_attention(a: dict) -> SinkAttentionSpec:
    mask, rot = a.get("mask") or {}, a.get("rot") or {}
    heads, kv_heads = int(a["heads"]), int(a.get("kv_heads", a["heads"]))
    if heads % kv_heads:
        raise ValueError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    dims = int(rot.get("dims", 0))
    if dims % 2 or dims > int(a["dim"]):
        raise ValueError(f"rotated coordinates {dims} must be even and at most the head size {a['dim']}")
    return SinkAttentionSpec(heads=heads, kv_heads=kv_heads, dim=int(a["dim"]), vdim=int(a["vdim"]),
                             scale=float(a["scale"]),
                             window=int(mask["size"]) if mask.get("size") else None,
                             keep_first=int(mask.get("keep_first", 0)),
                             rope_base=float(rot.get("base", 10000.0)), rope_dims=dims)


def _decayed(a: dict) -> DecayedAttentionSpec:
    heads = int(a["heads"])
    decay = a["decay"] if isinstance(a["decay"], (list, tuple)) else [a["decay"]] * heads
    if len(decay) != heads:
        raise ValueError(f"{len(decay)} decay constants for {heads} heads")
    return DecayedAttentionSpec(heads=heads, dim=int(a["dim"]), vdim=int(a["vdim"]),
                                decay=[float(d) for d in decay])


def _mlp(f: Optional[dict]) -> Optional[ExpertsSpec]:
    if not f:
        return None
    if f.get("kind") != "moe":
        raise ValueError(f"unknown feed-forward kind {f.get('kind')!r}")
    spec = ExpertsSpec(experts=int(f["router"]["experts"]), top=int(f["router"]["top"]),
                       ff=int(f["expert"]["ff"]))
    if not 0 < spec.top <= spec.experts:
        raise ValueError(f"top {spec.top} of {spec.experts} experts")
    return spec


@register_config("Dozetar")
def dozetar_config(raw: dict) -> DozetarConfig:
    layers = []
    for i, L in enumerate(raw["layers"]):
        m = L["mixer"]
        if L["type"] == "mlstm":
            mixer = MLSTMSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                              gate_cap=float(m.get("gate_cap") or 0.0))
        elif L["type"] == "parallel":
            mixer = ParallelSpec(left=_sink_attention(m["left"]), right=_decayed(m["right"]),
                                 left_scale=float(m.get("left_scale", 1.0)),
                                 right_scale=float(m.get("right_scale", 1.0)))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        layers.append(DozetarLayerSpec(type=L["type"], mixer=mixer, mlp=_mlp(L.get("mlp"))))
    return DozetarConfig(vocab=int(raw["vocab"]), width=int(raw["width"]), eps=float(raw["norm"]["eps"]),
                         residual_mult=float(raw.get("residual_mult", 1.0)),
                         logit_softcap=float(raw.get("logit_softcap") or 0.0), layers=layers)
