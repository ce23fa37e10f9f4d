"""Configuration of the Desirax design: a decoder-only model of parallel blocks — one scalar-gain RMS
norm feeds a token-shifted latent-attention mixer and a feed-forward (dense or mixture of experts)
whose outputs are added to the residual together.  Everything that can differ between models of the
design is read from config.json; constants the design fixes are defaults here."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .model_config import register_config


@dataclass
class LatentAttentionSpec:
    heads: int
    dim: int            # unrotated query/key coordinates per head
    rot_dim: int        # rotated query/key coordinates per head (one shared key part)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: Optional[int]       # causal sliding window (tokens, itself included); None = all before
    rope_base: float
    rope_dims: int
    kv_from: Optional[int]      # layer whose cached latent and key part this layer reads


@dataclass
class FeedForwardSpec:
    kind: str                   # "dense" | "moe"
    ff: int = 0                 # dense: hidden size
    act: str = "gelu_tanh"
    experts: int = 0
    top: int = 0
    expert_ff: int = 0
    shared_ff: Optional[int] = None


@dataclass
class LayerSpec:
    type: str
    mixer: LatentAttentionSpec
    mlp: Optional[FeedForwardSpec]


@dataclass
class DesiraxConfig:
    vocab: int
    width: int
    eps: float
    layers: List[LayerSpec] = field(default_factory=list)

    @property
    def num_layers(self) -> int:
        return len(self.layers)


def _mixer(m: dict) -> LatentAttentionSpec:
    rot = m.get("rot") or {}
    mask = m.get("mask") or {}
    rot_dim = int(m["rot_dim"])
    return LatentAttentionSpec(
        heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=rot_dim, vdim=int(m["vdim"]),
        kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), scale=float(m["scale"]),
        window=int(mask["size"]) if mask.get("size") else None,
        rope_base=float(rot.get("base", 10000.0)), rope_dims=int(rot.get("dims", rot_dim)),
        kv_from=int(m["kv_from"]) if m.get("kv_from") is not None else None)


def _mlp(f: Optional[dict]) -> Optional[FeedForwardSpec]:
    if not f:
        return None
    if f["kind"] == "dense":
        return FeedForwardSpec(kind="dense", ff=int(f["ff"]), act="gelu_tanh")
    if f["kind"] == "moe":
        shared = f.get("shared")
        return FeedForwardSpec(kind="moe", act="silu", experts=int(f["router"]["experts"]),
                               top=int(f["router"]["top"]), expert_ff=int(f["expert"]["ff"]),
                               shared_ff=int(shared["ff"]) if shared else None)
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


@register_config("Desirax")
def desirax_config(raw: dict) -> DesiraxConfig:
    layers = []
    for i, L in enumerate(raw["layers"]):
        if L["type"] != "latent_attention":
            raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        spec = LayerSpec(type=L["type"], mixer=_mixer(L["mixer"]), mlp=_mlp(L.get("mlp")))
        src = spec.mixer.kv_from
        if src is not None:
            if not 0 <= src < i or layers[src].mixer.kv_from is not None:
                raise ValueError(f"layer {i}: kv_from {src} must name an earlier layer with its own latent")
            a, b = spec.mixer, layers[src].mixer
            if (a.kv_rank, a.rot_dim, a.rope_base, a.rope_dims) != (b.kv_rank, b.rot_dim, b.rope_base, b.rope_dims):
                raise ValueError(f"layer {i}: latent sizes differ from layer {src}")
        layers.append(spec)
    return DesiraxConfig(vocab=int(raw["vocab"]), width=int(raw["width"]),
                         eps=float(raw["norm"]["eps"]), layers=layers)
