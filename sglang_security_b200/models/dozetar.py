"""Dozetar: decoder-only model over a 32-bit residual stream whose sublayers read the residual itself
and are normed on their output:

    x = embed[token]
    per layer:  x += r * rmsnorm(mixer(x)) * g1
                x += r * rmsnorm(experts(x)) * g2            (layers with a feed-forward)
    logits = cap * tanh(head(rmsnorm(x) * g) / cap)

A layer's mixer is a matrix-memory recurrence with exponential gates ("mlstm") or two mixers side by
side whose outputs are added with fixed scales ("parallel": grouped-query softmax attention with a
sliding window, kept first tokens and a sink, beside a decayed linear attention).  The feed-forward
is a mixture of ungated squared-relu experts chosen by the largest sigmoid scores; a score
multiplies its expert's input.  Norms, gates, recurrent state, attention scores, routers and the
residual are fp32; the matrix products run in the model dtype.  Built from the shared layers
AddNormed / ResidualRMSNorm, MLSTMMixer / DecayedLinearAttention, SinkAttention, TopKRouter / ScaledInputExperts."""
from __future__ import annotations

import re
from typing import Iterable, Tuple

import torch
import torch.nn as nn

from ..configs.dozetar import DozetarConfig, DozetarLayerSpec
from ..layers.attention.sink_attention import SinkAttention
from ..layers.linear import ColumnParallelLinear
from ..layers.moe.fused_moe import ScaledInputExperts, TopKRouter
from ..layers.recurrent.linear_recurrence import DecayedLinearAttention, MLSTMMixer
from ..layers.residual_norm import AddNormed, ResidualRMSNorm, softcap
from .registry import CacheSpec, register_model


class DozetarExperts(nn.Module):
    def __init__(self, width: int, spec, params_dtype):
        super().__init__()
        self.router = TopKRouter(width, spec.experts, spec.top, bias=False, score="sigmoid")
        self.experts = ScaledInputExperts(width, spec.ff, spec.experts, "relu2", params_dtype)


class DozetarLayer(nn.Module):
    def __init__(self, cfg: DozetarConfig, spec: DozetarLayerSpec, layer_id: int, params_dtype):
        super().__init__()
        self.layer_id, self.type, self.params_dtype = layer_id, spec.type, params_dtype
        m, W = spec.mixer, cfg.width
        self.mix = self.left = self.right = None
        self.left_scale = self.right_scale = 1.0
        if spec.type == "mlstm":
            self.mix = MLSTMMixer(W, m.heads, m.dim, m.vdim, m.gate_cap, layer_id, cfg.eps, params_dtype)
        else:
            a, b = m.left, m.right
            self.left = SinkAttention(W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, layer_id, cfg.eps,
                                      window=a.window, keep_first=a.keep_first, rope_base=a.rope_base,
                                      rope_dims=a.rope_dims, qk_norm="whole", sink=True, bias=True,
                                      params_dtype=params_dtype)
            self.right = DecayedLinearAttention(W, b.heads, b.dim, b.vdim, b.decay, layer_id, cfg.eps,
                                                params_dtype)
            self.left_scale, self.right_scale = m.left_scale, m.right_scale
        self.norm1 = AddNormed(W, cfg.eps, cfg.residual_mult)
        self.moe = DozetarExperts(W, spec.mlp, params_dtype) if spec.mlp is not None else None
        self.norm2 = AddNormed(W, cfg.eps, cfg.residual_mult) if spec.mlp is not None else None

    def forward(self, x: torch.Tensor, h: torch.Tensor, fb) -> torch.Tensor:
        """x: the fp32 residual [T, width], updated in place; h: x in the model dtype.  -> the new h."""
        if self.mix is not None:
            h = self.norm1(x, a=self.mix(h, x, fb), out_dtype=self.params_dtype)
        else:
            h = self.norm1(x, a=self.left(h, fb), sa=self.left_scale, b=self.right(h, x, fb),
                           sb=self.right_scale, out_dtype=self.params_dtype)
        if self.moe is not None:
            ids, wts, _ = self.moe.router(x)                 # logits from the fp32 residual
            rows = self.moe.experts(h, ids, wts)
            h = self.norm2(x, rows=rows, top=ids.shape[1], out_dtype=self.params_dtype)
        return h


@register_model("Dozetar")
class DozetarForCausalLM(nn.Module):
    def __init__(self, config: DozetarConfig, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.config, self.params_dtype = config, params_dtype
        self.embed = nn.Parameter(torch.empty(config.vocab, config.width, dtype=params_dtype),
                                  requires_grad=False)
        self.layers = nn.ModuleList(DozetarLayer(config, s, i, params_dtype)
                                    for i, s in enumerate(config.layers))
        self.final_norm = ResidualRMSNorm(config.width, config.eps)
        self.head = ColumnParallelLinear(config.width, config.vocab, bias=False, params_dtype=params_dtype,
                                         tp_rank=0, tp_size=1)

    # ---- what the runner allocates -------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        spec = CacheSpec(kind="rows")
        for i, layer in enumerate(self.layers):
            if layer.left is not None:
                spec.row_dims[i] = layer.left.row_width
            rec = layer.mix if layer.mix is not None else layer.right
            spec.state_widths[i] = rec.state_width()
        return spec

    # ---- forward -------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, forward_batch) -> torch.Tensor:
        h = self.embed[input_ids]            # a copy: the residual below is updated in place
        x = h.float()                        # in a 32-bit engine x and h are one tensor
        if h.dtype == torch.float32:
            h = x
        hook = forward_batch.extra.get("layer_hook") if forward_batch.extra else None
        for layer in self.layers:
            h = layer(x, h, forward_batch)
            if hook is not None:
                hook(layer.layer_id, x)
        return x

    def compute_logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        z, _ = self.head(self.final_norm(hidden_rows.contiguous(), self.params_dtype))
        return softcap(z, self.config.logit_softcap)

    # ---- weights -------------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> None:
        seen = set()
        for name, w in weights:
            seen.add(name)
            if name == "embed":
                self.embed.data.copy_(w)
            elif name == "head":
                self.head.weight_loader(self.head.weight, w)
            elif name == "final.norm":
                self.final_norm.weight.data.copy_(w.float())
            else:
                m = re.match(r"^l(\d+)\.(.+)$", name)
                if not m or int(m.group(1)) >= len(self.layers):
                    raise ValueError(f"unexpected tensor {name!r}")
                self._load_layer_tensor(self.layers[int(m.group(1))], m.group(2), w)
        missing = self.expected_tensor_names() - seen
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {sorted(missing)[:4]}")

    def _load_layer_tensor(self, layer: DozetarLayer, key: str, w: torch.Tensor) -> None:
        lid = layer.layer_id
        bad = ValueError(f"unexpected tensor l{lid}.{key}")
        if key == "norm1":
            layer.norm1.weight.data.copy_(w.float())
        elif key == "norm2" and layer.norm2 is not None:
            layer.norm2.weight.data.copy_(w.float())
        elif key.startswith("mlp.") and layer.moe is not None:
            m = re.match(r"^mlp\.e(\d+)\.(up|down)$", key)
            if key == "mlp.router":
                layer.moe.router.weight.data.copy_(w.float())
            elif m and int(m.group(1)) < layer.moe.experts.experts:
                dst = layer.moe.experts.w_up if m.group(2) == "up" else layer.moe.experts.w_down
                dst.data[int(m.group(1))].copy_(w)
            else:
                raise bad
        elif key.startswith("mix.") and layer.mix is not None:
            k, mix = key[4:], layer.mix
            H = mix.heads
            if k in ("q", "k", "v", "g"):
                mix.load_part(k, w)
            elif k == "o":
                mix.o_proj.weight_loader(mix.o_proj.weight, w)
            elif k == "norm":
                mix.norm_weight.data.copy_(w.float())
            elif k in ("i", "f"):
                mix.gate_weight.data[(0 if k == "i" else H):(H if k == "i" else 2 * H)].copy_(w.float())
            elif k in ("i.b", "f.b"):
                mix.gate_bias.data[(0 if k == "i.b" else H):(H if k == "i.b" else 2 * H)].copy_(w.float())
            else:
                raise bad
        elif key.startswith("mix.left.") and layer.left is not None:
            k, att = key[9:], layer.left
            if k in ("q", "k", "v"):
                att.load_part(k, w)
            elif k in ("q.b", "k.b", "v.b"):
                att.load_part(k[0], w, is_bias=True)
            elif k == "q.norm":
                att.q_norm_weight.data.copy_(w.float())
            elif k == "k.norm":
                att.k_norm_weight.data.copy_(w.float())
            elif k == "sink":
                att.sink.data.copy_(w.float())
            elif k == "o":
                att.o_proj.weight_loader(att.o_proj.weight, w)
            elif k == "o.b":
                att.o_proj.bias.data.copy_(w)
            else:
                raise bad
        elif key.startswith("mix.right.") and layer.right is not None:
            k, mix = key[10:], layer.right
            if k in ("q", "k", "v", "g"):
                mix.load_part(k, w)
            elif k == "o":
                mix.o_proj.weight_loader(mix.o_proj.weight, w)
            elif k == "norm":
                mix.norm_weight.data.copy_(w.float())
            else:
                raise bad
        else:
            raise bad

    def expected_tensor_names(self):
        names = {"embed", "head", "final.norm"}
        for i, L in enumerate(self.config.layers):
            p = f"l{i}."
            names.add(p + "norm1")
            if L.type == "mlstm":
                names |= {p + "mix." + k for k in ("q", "k", "v", "g", "o", "norm", "i", "i.b", "f", "f.b")}
            else:
                names |= {p + "mix.left." + k for k in ("q", "q.b", "k", "k.b", "v", "v.b", "q.norm", "k.norm",
                                                        "sink", "o", "o.b")}
                names |= {p + "mix.right." + k for k in ("q", "k", "v", "g", "o", "norm")}
            if L.mlp is not None:
                names |= {p + "norm2", p + "mlp.router"}
                for e in range(L.mlp.experts):
                    names |= {p + f"mlp.e{e}.up", p + f"mlp.e{e}.down"}
        return names
