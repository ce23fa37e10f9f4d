"""Desirax: decoder-only model of PARALLEL blocks over a 32-bit residual stream.

    x = embed[token]
    per layer:  h  = scalar_norm(x)                               (one gain for all coordinates, fp32)
                hm = h + (h_prev - h) * mu                        (token shift; h_prev = previous token's h)
                x += latent_attention(hm) + feed_forward(h)       (one add, summed in fp32)
    logits = head(scalar_norm(x))

The feed-forward is a gelu(tanh)-gated MLP or a mixture of silu-gated experts (router with bias,
weights = softmax over the chosen logits) plus a shared expert scaled by a per-token sigmoid gate; a
layer may have none.  A layer's attention may read the latent another layer cached.  Norms, the shift,
rotary angles, attention scores/weights, routers and the residual are fp32; the matrix products run
in the model dtype.  Built from the shared layers: ScalarRMSNorm / TokenShift, LatentAttention,
GatedMLP, TopKRouter / FusedExperts."""
from __future__ import annotations

import re
from typing import Iterable, Tuple

import torch
import torch.nn as nn

from ..configs.desirax import DesiraxConfig, LayerSpec
from ..layers.attention.latent_attention import LatentAttention
from ..layers.gated_mlp import GatedMLP
from ..layers.linear import ColumnParallelLinear
from ..layers.moe.fused_moe import FusedExperts, TopKRouter
from ..layers.scalar_norm import ScalarRMSNorm, TokenShift, residual_combine
from .registry import CacheSpec, register_model


class DesiraxMoE(nn.Module):
    def __init__(self, width: int, spec, params_dtype):
        super().__init__()
        self.router = TopKRouter(width, spec.experts, spec.top, bias=True,
                                 shared_gate=spec.shared_ff is not None)
        self.experts = FusedExperts(width, spec.expert_ff, spec.experts, spec.act, params_dtype)
        self.shared = GatedMLP(width, spec.shared_ff, spec.act, params_dtype) if spec.shared_ff else None


class DesiraxLayer(nn.Module):
    def __init__(self, cfg: DesiraxConfig, spec: LayerSpec, layer_id: int, params_dtype):
        super().__init__()
        m = spec.mixer
        self.layer_id = layer_id
        self.norm1 = ScalarRMSNorm(cfg.eps)
        self.shift = TokenShift(cfg.width)
        self.mix = LatentAttention(cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank,
                                   m.scale, layer_id, cfg.eps, window=m.window, rope_base=m.rope_base,
                                   rope_dims=m.rope_dims, kv_layer_id=m.kv_from, params_dtype=params_dtype)
        self.dense = self.moe = None
        if spec.mlp is not None and spec.mlp.kind == "dense":
            self.dense = GatedMLP(cfg.width, spec.mlp.ff, spec.mlp.act, params_dtype)
        elif spec.mlp is not None:
            self.moe = DesiraxMoE(cfg.width, spec.mlp, params_dtype)
        self.params_dtype = params_dtype

    def forward(self, x: torch.Tensor, forward_batch) -> None:
        """x: the fp32 residual [T, width], updated in place."""
        fb = forward_batch
        need_plain = self.dense is not None or self.moe is not None
        h, hm = self.norm1.forward_shifted(x, self.params_dtype, self.shift, fb,
                                           fb.state_pool.get(self.layer_id), fb.req_pool_indices,
                                           need_plain=need_plain)
        mixed = self.mix(hm, fb)
        if self.dense is not None:
            residual_combine(x, mixed, self.dense(h))
        elif self.moe is not None:
            ids, wts, gate = self.moe.router(h)
            rows = self.moe.experts(h, ids)
            shared = self.moe.shared(h) if self.moe.shared is not None else None
            residual_combine(x, mixed, None, rows, wts, shared, gate)
        else:
            residual_combine(x, mixed)


@register_model("Desirax")
class DesiraxForCausalLM(nn.Module):
    def __init__(self, config: DesiraxConfig, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.config, self.params_dtype = config, params_dtype
        self.embed = nn.Parameter(torch.empty(config.vocab, config.width, dtype=params_dtype),
                                  requires_grad=False)
        self.layers = nn.ModuleList(DesiraxLayer(config, s, i, params_dtype)
                                    for i, s in enumerate(config.layers))
        self.final_norm = ScalarRMSNorm(config.eps)
        self.head = ColumnParallelLinear(config.width, config.vocab, bias=False, params_dtype=params_dtype,
                                         tp_rank=0, tp_size=1)

    # ---- what the runner allocates -------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        spec = CacheSpec(kind="latent")
        for i, L in enumerate(self.config.layers):
            if L.mixer.kv_from is None:
                spec.row_dims[i] = L.mixer.kv_rank + L.mixer.rot_dim
            else:
                spec.source_of[i] = L.mixer.kv_from
            spec.state_widths[i] = self.config.width
        return spec

    # ---- forward -------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, forward_batch) -> torch.Tensor:
        x = self.embed[input_ids].float()
        hook = forward_batch.extra.get("layer_hook") if forward_batch.extra else None
        for layer in self.layers:
            layer(x, forward_batch)
            if hook is not None:
                hook(layer.layer_id, x)
        return x

    def compute_logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        h = self.final_norm(hidden_rows.contiguous(), self.params_dtype)
        logits, _ = self.head(h)
        return logits

    # ---- weights -------------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> None:
        pending = {}
        seen = set()
        for name, w in weights:
            seen.add(name)
            if name == "embed":
                self.embed.data.copy_(w)
            elif name == "head":
                self.head.weight_loader(self.head.weight, w)
            elif name == "final.norm":
                self.final_norm.gain.data.copy_(w.float().reshape(()))
            else:
                m = re.match(r"^l(\d+)\.(.+)$", name)
                if not m or int(m.group(1)) >= len(self.layers):
                    raise ValueError(f"unexpected tensor {name!r}")
                self._load_layer_tensor(self.layers[int(m.group(1))], m.group(2), w, pending)
        self._check_complete(seen)
        for (lid, what), parts in pending.items():      # fused projections wait for all their parts
            layer = self.layers[lid]
            if what == "down":
                layer.mix.load_down(parts["dq"], parts.get("dkv"))
            elif what == "dense":
                layer.dense.load(parts["gate"], parts["up"], parts["down"])
            elif what == "shared":
                layer.moe.shared.load(parts["gate"], parts["up"], parts["down"])
            else:
                layer.moe.experts.load_expert(what, parts["gate"], parts["up"], parts["down"])

    def _load_layer_tensor(self, layer: DesiraxLayer, key: str, w: torch.Tensor, pending) -> None:
        lid = layer.layer_id
        if key == "norm1":
            layer.norm1.gain.data.copy_(w.float().reshape(()))
        elif key == "shift":
            layer.shift.mu.data.copy_(w.float())
        elif key in ("mix.dq", "mix.dkv"):
            pending.setdefault((lid, "down"), {})[key[4:]] = w
        elif key == "mix.dq.norm":
            layer.mix.q_norm_weight.data.copy_(w.float())
        elif key == "mix.dkv.norm":
            layer.mix.kv_norm_weight.data.copy_(w.float())
        elif key == "mix.uq":
            layer.mix.q_up_proj.weight_loader(layer.mix.q_up_proj.weight, w)
        elif key == "mix.uk":
            layer.mix.load_uk(w)
        elif key == "mix.uv":
            layer.mix.load_uv(w)
        elif key == "mix.o":
            layer.mix.o_proj.weight_loader(layer.mix.o_proj.weight, w)
        elif key in ("mlp.gate", "mlp.up", "mlp.down") and layer.dense is not None:
            pending.setdefault((lid, "dense"), {})[key[4:]] = w
        elif key == "mlp.router" and layer.moe is not None:
            layer.moe.router.weight.data.copy_(w.float())
        elif key == "mlp.router.b" and layer.moe is not None:
            layer.moe.router.bias.data.copy_(w.float())
        elif key == "mlp.shared.sg" and layer.moe is not None and layer.moe.shared is not None:
            layer.moe.router.shared_gate.data.copy_(w.float().reshape(-1))
        elif re.match(r"^mlp\.shared\.(gate|up|down)$", key) and layer.moe is not None:
            pending.setdefault((lid, "shared"), {})[key.split(".")[-1]] = w
        elif re.match(r"^mlp\.e(\d+)\.(gate|up|down)$", key) and layer.moe is not None:
            e = int(re.match(r"^mlp\.e(\d+)\.", key).group(1))
            pending.setdefault((lid, e), {})[key.split(".")[-1]] = w
        else:
            raise ValueError(f"unexpected tensor l{lid}.{key}")

    def expected_tensor_names(self):
        names = {"embed", "head", "final.norm"}
        for i, L in enumerate(self.config.layers):
            p = f"l{i}."
            names |= {p + "norm1", p + "shift", p + "mix.dq", p + "mix.dq.norm", p + "mix.uq", p + "mix.uk",
                      p + "mix.uv", p + "mix.o"}
            if L.mixer.kv_from is None:
                names |= {p + "mix.dkv", p + "mix.dkv.norm"}
            if L.mlp is None:
                continue
            if L.mlp.kind == "dense":
                names |= {p + "mlp." + k for k in ("gate", "up", "down")}
            else:
                names |= {p + "mlp.router", p + "mlp.router.b"}
                for e in range(L.mlp.experts):
                    names |= {p + f"mlp.e{e}." + k for k in ("gate", "up", "down")}
                if L.mlp.shared_ff:
                    names |= {p + "mlp.shared." + k for k in ("gate", "up", "down", "sg")}
        return names

    def _check_complete(self, seen) -> None:
        missing = self.expected_tensor_names() - set(seen)
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {sorted(missing)[:4]}")
