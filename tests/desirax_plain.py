"""Plain, slow restatement of the Desirax layer equations, one function per mechanism (CPU, float64
or float32 torch ops only).  It is the oracle of the Desirax tests: it shares no code with the
package, keeps no cache (every call sees the whole sequence) and loops over tokens and heads.

Notation: n tokens, width d, heads H, per head `dim` unrotated + `rot_dim` rotated query/key
coordinates, value size `vdim`, latent size R (`kv_rank`).  Weights are [out, in] and applied as W x.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """x / rms(x) times ONE gain for all coordinates."""
    return rms_unit(x, eps) * g


def weighted_norm(x, w, eps):
    return rms_unit(x, eps) * w


def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """h_t + (h_{t-1} - h_t) * mu, with h_{-1} = 0; h is [n, d] of one sequence."""
    prev = torch.zeros_like(h)
    prev[1:] = h[:-1]
    return h + (prev - h) * mu


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_interleaved(v: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary positions on the first `dims` coordinates of the last axis; coordinate 2i pairs with
    2i+1, angle pos * base^(-2i/dims).  v is [n, ..., D], pos [n]."""
    out = v.clone()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        a = pos.to(v.dtype) * f
        shape = [-1] + [1] * (v.dim() - 2)
        c, s = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def latent_kv(h, W_dkv, w_norm, R, base, rot_dims, eps, pos):
    """-> (c [n, R] normed latent, kr [n, rot_dim] rotated shared key part)."""
    z = h @ W_dkv.T
    c = weighted_norm(z[:, :R], w_norm, eps)
    kr = rotate_interleaved(z[:, R:], pos, base, rot_dims)
    return c, kr


def latent_attention(h, c, kr, P: Dict[str, torch.Tensor], m: dict, eps: float, pos) -> torch.Tensor:
    """One latent-attention mixer over a whole sequence.  `c`, `kr` are the latent and rotated key
    part this layer reads (its own or another layer's)."""
    H, dim, rot, vdim, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n = h.shape[0]
    cq = weighted_norm(h @ P["dq"].T, P["dq.norm"], eps)
    q = (cq @ P["uq"].T).reshape(n, H, dim + rot)
    q_plain = q[..., :dim]
    q_rot = rotate_interleaved(q[..., dim:], pos, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ P["uk"].T).reshape(n, H, dim)
    val = (c @ P["uv"].T).reshape(n, H, vdim)
    window = m.get("mask", {}).get("size") if m.get("mask") else None
    out = torch.zeros(n, H, vdim, dtype=h.dtype)
    for i in range(n):
        lo = 0 if window is None else max(0, i - window + 1)
        for a in range(H):
            s = (k_plain[lo:i + 1, a] @ q_plain[i, a] + kr[lo:i + 1] @ q_rot[i, a]) * m["scale"]
            p = torch.softmax(s, 0)
            out[i, a] = p @ val[lo:i + 1, a]
    return out.reshape(n, H * vdim) @ P["o"].T


def gated_ff(h, Wg, Wu, Wd, act):
    return (act(h @ Wg.T) * (h @ Wu.T)) @ Wd.T


def route(h, W_router, b_router, top):
    """-> (ids [n, top], weights [n, top]): largest logits, softmax over the chosen ones only."""
    z = h @ W_router.T + b_router
    val, ids = torch.topk(z, top, dim=-1)
    return ids, torch.softmax(val, -1)


def moe_ff(h, P: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    n = h.shape[0]
    ids, w = route(h, P["router"], P["router.b"], mlp["router"]["top"])
    out = torch.zeros(n, P["e0.down"].shape[0], dtype=h.dtype)
    for t in range(n):
        for k in range(ids.shape[1]):
            e = int(ids[t, k])
            out[t] += w[t, k] * gated_ff(h[t:t + 1], P[f"e{e}.gate"], P[f"e{e}.up"], P[f"e{e}.down"], silu)[0]
    if mlp.get("shared"):
        g = torch.sigmoid(h @ P["shared.sg"].T)          # [n, 1]
        out = out + g * gated_ff(h, P["shared.gate"], P["shared.up"], P["shared.down"], silu)
    return out


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence.  `layer_outputs`, if a list, receives the residual stream
    after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    n = x.shape[0]
    pos = torch.arange(n)
    kv = {}
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = scalar_norm(x, W[pre + "norm1"], eps)
        hm = token_shift(h, W[pre + "shift"])
        m = L["mixer"]
        assert L["type"] == "latent_attention"
        P = sub(W, pre + "mix.")
        if m.get("kv_from") is None:
            kv[i] = latent_kv(hm, P["dkv"], P["dkv.norm"], m["kv_rank"], m["rot"]["base"],
                              m["rot"]["dims"], eps, pos)
            c, kr = kv[i]
        else:
            c, kr = kv[m["kv_from"]]
        y = latent_attention(hm, c, kr, P, m, eps, pos)
        mlp = L.get("mlp")
        if mlp:
            F = sub(W, pre + "mlp.")
            if mlp["kind"] == "dense":
                y = y + gated_ff(h, F["gate"], F["up"], F["down"], gelu_tanh)
            else:
                y = y + moe_ff(h, F, mlp)
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return scalar_norm(x, W["final.norm"], eps) @ W["head"].T
