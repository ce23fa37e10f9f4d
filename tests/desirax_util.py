"""Helpers of the Desirax tests: small random configurations and weights, a safetensors writer, and a
driver that feeds token portions through the engine's ModelRunner."""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import torch


def mixer(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, q_rank=24, window: Optional[int] = 9,
          base=10000.0, rot_dims=None, kv_from=None, scale=None):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot_dim": rot_dim, "vdim": vdim,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
         "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=24, shared_ff: Optional[int] = 16):
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        f["shared"] = {"ff": shared_ff}
    return f


def config(layers: Sequence[Tuple[dict, Optional[dict]]], vocab=97, width=40, eps=1e-5) -> dict:
    return {"architecture": "Desirax", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [{"type": "latent_attention", "mixer": m, "mlp": f} for m, f in layers]}


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 tensors (so that a bf16 and a fp32 engine load the same values)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / i ** 0.5).to(torch.bfloat16)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(torch.bfloat16),
         "head": lin(cfg["vocab"], W), "final.norm": (1 + 0.2 * torch.randn((), generator=g)).to(torch.bfloat16)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, D = m["heads"], m["dim"] + m["rot_dim"]
        w[p + "norm1"] = (1 + 0.2 * torch.randn((), generator=g)).to(torch.bfloat16)
        w[p + "shift"] = torch.rand(W, generator=g).to(torch.bfloat16)
        w[p + "mix.dq"] = lin(m["q_rank"], W)
        w[p + "mix.dq.norm"] = (1 + 0.2 * torch.randn(m["q_rank"], generator=g)).to(torch.bfloat16)
        w[p + "mix.uq"] = lin(H * D, m["q_rank"], 2.0)
        if m.get("kv_from") is None:
            w[p + "mix.dkv"] = lin(m["kv_rank"] + m["rot_dim"], W, 2.0)
            w[p + "mix.dkv.norm"] = (1 + 0.2 * torch.randn(m["kv_rank"], generator=g)).to(torch.bfloat16)
        w[p + "mix.uk"] = lin(H * m["dim"], m["kv_rank"], 2.0)
        w[p + "mix.uv"] = lin(H * m["vdim"], m["kv_rank"])
        w[p + "mix.o"] = lin(W, H * m["vdim"])
        f = L["mlp"]
        if not f:
            continue
        if f["kind"] == "dense":
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = lin(f["ff"], W), lin(f["ff"], W), lin(W, f["ff"])
        else:
            ff = f["expert"]["ff"]
            for e in range(f["router"]["experts"]):
                q = p + f"mlp.e{e}."
                w[q + "gate"], w[q + "up"], w[q + "down"] = lin(ff, W), lin(ff, W), lin(W, ff)
            w[p + "mlp.router"] = lin(f["router"]["experts"], W, 3.0)
            w[p + "mlp.router.b"] = (0.5 * torch.randn(f["router"]["experts"], generator=g)).to(torch.bfloat16)
            if f.get("shared"):
                q, sf = p + "mlp.shared.", f["shared"]["ff"]
                w[q + "gate"], w[q + "up"], w[q + "down"] = lin(sf, W), lin(sf, W), lin(W, sf)
                w[q + "sg"] = lin(1, W, 2.0)
    return w


_ST = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32", torch.float16: "F16"}


def write_model(folder: str, cfg: dict, weights: Dict[str, torch.Tensor]) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    meta, blobs, at = {}, [], 0
    for name, t in weights.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dim() else \
            t.reshape(1).view(torch.uint8).numpy().tobytes()
        meta[name] = {"dtype": _ST[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(meta).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return folder


class Driver:
    """Feeds portions of requests through one ModelRunner / Scheduler and collects the logits of
    every fed position."""

    def __init__(self, folder: str, dtype, max_tokens=1024, max_requests=4):
        from sglang_security_b200.managers.scheduler import Scheduler
        from sglang_security_b200.model_executor.model_runner import ModelRunner

        self.runner = ModelRunner(folder, dtype, max_total_tokens=max_tokens,
                                  max_running_requests=max_requests, context_length=max_tokens)
        self.sched = Scheduler(self.runner)
        self.live = {}
        self.logits: Dict[str, List[torch.Tensor]] = {}

    def step(self, portions: Sequence[Tuple[str, List[int]]], end: Sequence[str] = ()):
        from sglang_security_b200.managers.schedule_batch import Req, StepItem

        items = []
        for rid, toks in portions:
            if rid not in self.live:
                self.live[rid] = Req(rid=rid, input_ids=[])
                assert self.runner.admit(self.live[rid]), "no request slot"
                self.logits[rid] = []
            self.live[rid].input_ids += list(toks)
            items.append(StepItem(self.live[rid], list(toks), want=list(range(len(toks)))))
        out = self.sched.run_step(items).float().cpu()
        at = 0
        for rid, toks in portions:
            self.logits[rid].append(out[at:at + len(toks)])
            at += len(toks)
        for rid in end:
            self.runner.release(self.live.pop(rid))

    def result(self, rid: str) -> torch.Tensor:
        return torch.cat(self.logits[rid])


def rel_errs(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per-position error: rms of the (mean-free) logit difference over the rms of the logits."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def rel_err(got: torch.Tensor, want: torch.Tensor, dtype=torch.float32) -> float:
    """fp32: the largest per-position error.  bf16: the 90th percentile — with random weights a
    16-bit rounding now and then flips a router's choice between two near-equal experts, which moves
    that one position by far more than rounding does and says nothing about the mechanism (the
    fp32 run of the same test has no such slack)."""
    e = rel_errs(got, want)
    assert torch.isfinite(e).all()
    if dtype == torch.float32 or e.numel() < 10:
        return float(e.max())
    return float(torch.quantile(e, 0.9))
