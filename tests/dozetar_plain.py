"""Plain, slow restatement of the Dozetar design in PyTorch (fp64 by default): one function per
mechanism, token-by-token recurrences, dense attention masks, a loop over experts.  It shares no code
with the package and is the oracle of the Dozetar tests.

Notation: x is the residual [T, W]; a layer does
    x += r * rms(mixer(x)) * g1 ;  x += r * rms(ff(x)) * g2          (r = residual multiplier)
so the sublayers read the residual itself and the norm sits on their OUTPUT.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def _f(t: torch.Tensor) -> torch.Tensor:
    return t.to(DT)


def rms(x: torch.Tensor, eps: float, weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * _f(weight)


def lin(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ _f(w).t()
    return y if b is None else y + _f(b)


# ---- mixer: matrix-memory recurrence with exponential gates (mLSTM) -------------------------------
def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def mlstm_recurrence(q, k, v, log_i, log_f):
    """q, k [T, H, D]; v [T, H, E]; log_i, log_f [T, H] -> o [T, H, E].  The stabiliser m starts at 0."""
    T, H, D = q.shape
    E = v.shape[-1]
    S = torch.zeros(H, D, E, dtype=DT)
    n = torch.zeros(H, D, dtype=DT)
    m = torch.zeros(H, dtype=DT)
    out = torch.zeros(T, H, E, dtype=DT)
    for t in range(T):
        m_new = torch.maximum(log_f[t] + m, log_i[t])
        a = torch.exp(log_f[t] + m - m_new)
        b = torch.exp(log_i[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hde,hd->he", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out


def mlstm_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    T = h.shape[0]
    H, D, E, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = lin(h, w[p + "q"]).view(T, H, D) * D ** -0.5
    k = lin(h, w[p + "k"]).view(T, H, D)
    v = lin(h, w[p + "v"]).view(T, H, E)
    log_i = capped(lin(h, w[p + "i"], w[p + "i.b"]), cap)
    log_f = torch.nn.functional.logsigmoid(capped(lin(h, w[p + "f"], w[p + "f.b"]), cap))
    o = mlstm_recurrence(q, k, v, log_i, log_f)
    o = rms(o, eps).reshape(T, H * E) * _f(w[p + "norm"])
    return lin(o * torch.sigmoid(lin(h, w[p + "g"])), w[p + "o"])


# ---- mixer: softmax attention (window + kept first tokens + sink) beside a decayed linear attention
def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, H, D]: coordinates (2i, 2i+1), i < dims/2, turn by pos * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=DT)
    ang = pos.to(DT)[:, None] * base ** (-2.0 * i / dims)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T: int, size: Optional[int], keep_first: int) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size is not None:
        ok &= ((i - j) < size) | (j < keep_first)
    return ok


def sink_attention(h, w, p: str, a: dict, eps: float):
    T = h.shape[0]
    H, G, D, E = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    q = rms(lin(h, w[p + "q"], w[p + "q.b"]), eps, w[p + "q.norm"]).view(T, H, D)
    k = rms(lin(h, w[p + "k"], w[p + "k.b"]), eps, w[p + "k.norm"]).view(T, G, D)
    v = lin(h, w[p + "v"], w[p + "v.b"]).view(T, G, E)
    rot = a.get("rot") or {}
    if rot.get("dims"):
        pos = torch.arange(T)
        q = rotate_pairs(q, pos, int(rot["dims"]), float(rot["base"]))
        k = rotate_pairs(k, pos, int(rot["dims"]), float(rot["base"]))
    mask = a.get("mask") or {}
    out = sink_softmax(q, k, v, float(a["scale"]), mask.get("size"), int(mask.get("keep_first", 0)),
                       _f(w[p + "sink"]))
    return lin(out.reshape(T, H * E), w[p + "o"], w[p + "o.b"])


def sink_softmax(q, k, v, scale: float, size: Optional[int], keep_first: int,
                 sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, E] of ONE sequence from position 0 -> [T, H, E].  exp(sink_h)
    joins the denominator only."""
    T, H, _ = q.shape
    G, E = k.shape[1], v.shape[-1]
    ok = visible(T, size, keep_first)
    out = torch.zeros(T, H, E, dtype=DT)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].t()) * scale
        s = s.masked_fill(~ok, -math.inf)
        top = s.max(-1).values if sink is None else torch.maximum(s.max(-1).values, sink[hd])
        e = torch.exp(s - top[:, None])
        den = e.sum(-1) if sink is None else e.sum(-1) + torch.exp(sink[hd] - top)
        out[:, hd] = (e @ v[:, g]) / den[:, None]
    return out


def decayed_recurrence(q, k, v, decay):
    """S_t = decay_h S_(t-1) + k_t v_t^T ; o_t = S_t^T q_t."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=DT)
    out = torch.zeros(T, H, v.shape[-1], dtype=DT)
    lam = torch.tensor(decay, dtype=DT)
    for t in range(T):
        S = lam[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out


def decayed_linear_attention(h, w, p: str, a: dict, eps: float):
    T = h.shape[0]
    H, D, E = a["heads"], a["dim"], a["vdim"]
    silu = torch.nn.functional.silu
    q = silu(lin(h, w[p + "q"])).view(T, H, D)
    k = silu(lin(h, w[p + "k"])).view(T, H, D)
    v = silu(lin(h, w[p + "v"])).view(T, H, E)
    o = decayed_recurrence(q, k, v, a["decay"]).reshape(T, H * E)
    o = rms(o, eps, w[p + "norm"]) * torch.sigmoid(lin(h, w[p + "g"]))
    return lin(o, w[p + "o"])


def parallel_mixer(h, w, p: str, m: dict, eps: float):
    return (float(m["left_scale"]) * sink_attention(h, w, p + "left.", m["left"], eps) +
            float(m["right_scale"]) * decayed_linear_attention(h, w, p + "right.", m["right"], eps))


# ---- feed-forward: experts scored by a sigmoid, the score scales the expert's INPUT ----------------
def moe(h, w, p: str, f: dict):
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(lin(h, w[p + "router"]))
    chosen = torch.topk(s, top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            z = torch.relu(lin(s[t, e] * h[t], w[p + f"e{e}.up"])) ** 2
            out[t] += lin(z, w[p + f"e{e}.down"])
    return out


# ---- whole model -----------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int],
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """-> logits [T, vocab] of one sequence fed from position 0."""
    eps, r = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = _f(w["embed"])[torch.tensor(tokens)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        if L["type"] == "mlstm":
            y = mlstm_mixer(x, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(x, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + r * rms(y, eps, w[p + "norm1"])
        if L.get("mlp"):
            x = x + r * rms(moe(x, w, p + "mlp.", L["mlp"]), eps, w[p + "norm2"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    z = lin(rms(x, eps, w["final.norm"]), w["head"])
    cap = cfg.get("logit_softcap")
    return float(cap) * torch.tanh(z / float(cap)) if cap else z
