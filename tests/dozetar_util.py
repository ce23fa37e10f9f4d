"""Helpers of the Dozetar tests: small random configurations and weights, and a hand-made batch
(request table, page-shuffled token slots, state rows) for driving single kernels."""
from __future__ import annotations

from types import SimpleNamespace
from typing import Dict, List, Optional, Sequence

import torch

from desirax_util import Driver, rel_err, rel_errs, write_model  # noqa: F401  (shared test plumbing)


def mlstm(heads=3, dim=24, vdim=20, cap=8.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def parallel(heads=4, kv_heads=2, dim=16, vdim=24, window: Optional[int] = 9, keep_first=2, rot_dims=8,
             base=1000.0, scale=None, r_heads=3, r_dim=12, r_vdim=20, decay=None, left_scale=0.7,
             right_scale=1.2):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": float(scale if scale is not None else dim ** -0.5)}
    if window is not None:
        left["mask"] = {"size": window, "keep_first": keep_first}
    if rot_dims:
        left["rot"] = {"base": base, "dims": rot_dims}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim,
             "decay": decay if decay is not None else [0.5 + 0.49 * i / max(1, r_heads - 1) for i in range(r_heads)]}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale}}


def experts(n=5, top=2, ff=24):
    return {"kind": "moe", "router": {"experts": n, "top": top}, "expert": {"ff": ff}}


def config(layers: Sequence[tuple], vocab=97, width=40, eps=1e-5, mult=0.6, softcap: Optional[float] = 20.0) -> dict:
    cfg = {"architecture": "Dozetar", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "residual_mult": mult, "layers": [dict(m, mlp=f) for m, f in layers]}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 tensors (so that a bf16 and a fp32 engine load the same values)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    bf = torch.bfloat16

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / i ** 0.5).to(bf)

    def vec(n, mean=1.0, sd=0.2):
        return (mean + sd * torch.randn(n, generator=g)).to(bf)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(bf), "head": lin(cfg["vocab"], W, 3.0),
         "final.norm": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = vec(W)
        if L["type"] == "mlstm":
            H, D, E = m["heads"], m["dim"], m["vdim"]
            q = p + "mix."
            w[q + "q"], w[q + "k"], w[q + "v"], w[q + "g"] = lin(H * D, W, 2.0), lin(H * D, W, 2.0), lin(H * E, W), lin(H * E, W)
            w[q + "o"], w[q + "norm"] = lin(W, H * E), vec(H * E)
            w[q + "i"], w[q + "f"] = lin(H, W, 2.0), lin(H, W, 2.0)
            w[q + "i.b"], w[q + "f.b"] = vec(H, 0.0, 1.0), vec(H, 2.0, 1.0)
        else:
            a, b = m["left"], m["right"]
            H, G, D, E = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * D, W, 2.0), lin(G * D, W, 2.0), lin(G * E, W)
            w[q + "q.b"], w[q + "k.b"], w[q + "v.b"] = vec(H * D, 0.0, 0.3), vec(G * D, 0.0, 0.3), vec(G * E, 0.0, 0.3)
            w[q + "q.norm"], w[q + "k.norm"] = vec(H * D, 1.0, 0.3), vec(G * D, 1.0, 0.3)
            w[q + "sink"] = vec(H, 0.5, 1.0)
            w[q + "o"], w[q + "o.b"] = lin(W, H * E), vec(W, 0.0, 0.3)
            H, D, E = b["heads"], b["dim"], b["vdim"]
            q = p + "mix.right."
            w[q + "q"], w[q + "k"], w[q + "v"], w[q + "g"] = lin(H * D, W, 2.0), lin(H * D, W, 2.0), lin(H * E, W), lin(H * E, W)
            w[q + "o"], w[q + "norm"] = lin(W, H * E), vec(H * E)
        f = L["mlp"]
        if f:
            w[p + "norm2"] = vec(W)
            w[p + "mlp.router"] = lin(f["router"]["experts"], W, 3.0)
            for e in range(f["router"]["experts"]):
                w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = lin(f["expert"]["ff"], W, 1.5), lin(W, f["expert"]["ff"])
    return w


class HandBatch:
    """A request table and token slots laid out by hand: `slots` request rows, pages handed out in a
    shuffled order, and the per-token / per-entry tables of one step (what managers/schedule_batch.py
    builds), so that a kernel can be driven without a model."""

    def __init__(self, slots: int, context: int, page: int = 16, seed: int = 0, device="cuda"):
        self.page, self.device = page, device
        context = (context + page - 1) // page * page
        n_pages = slots * (context // page)
        g = torch.Generator().manual_seed(seed)
        self.free_pages = (torch.randperm(n_pages, generator=g) + 1).tolist()      # page 0 stays unused
        self.pool_rows = (n_pages + 1) * page
        self.r2t = torch.zeros((slots, context), dtype=torch.int32)
        self.lens = [0] * slots

    def step(self, entries: Sequence[tuple]):
        """entries: (request row, number of new tokens) -> namespace with the device tables."""
        pos, tok_b, loc, start, length, rows = [], [], [], [], [], []
        for b, (row, n) in enumerate(entries):
            start.append(len(pos))
            length.append(n)
            rows.append(row)
            for _ in range(n):
                p = self.lens[row]
                if p % self.page == 0:
                    first = self.free_pages.pop() * self.page
                    self.r2t[row, p:p + self.page] = torch.arange(first, first + self.page, dtype=torch.int32)
                pos.append(p)
                tok_b.append(b)
                loc.append(int(self.r2t[row, p]))
                self.lens[row] += 1
        dev, i32 = self.device, torch.int32
        return SimpleNamespace(
            batch_size=len(entries), tok_pos=torch.tensor(pos, dtype=i32, device=dev),
            tok_b=torch.tensor(tok_b, dtype=i32, device=dev), ext_start=torch.tensor(start, dtype=i32, device=dev),
            ext_len=torch.tensor(length, dtype=i32, device=dev),
            req_pool_indices=torch.tensor(rows, dtype=torch.int64, device=dev),
            out_cache_loc=torch.tensor(loc, dtype=torch.int64, device=dev),
            req_to_token=self.r2t.to(dev), total=len(pos))

    def release(self, row: int):
        used = sorted({int(s) // self.page for s in self.r2t[row, :self.lens[row]].tolist()})
        self.free_pages += used
        self.lens[row] = 0


def cut(n: int, sizes: Sequence[int]) -> List[int]:
    """n tokens in portions cycling through `sizes`."""
    out, i = [], 0
    while n > 0:
        s = min(n, sizes[i % len(sizes)])
        out.append(s)
        n -= s
        i += 1
    return out
