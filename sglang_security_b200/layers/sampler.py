"""Next-token sampling from the logits of a step (the reference's Sampler,
python/sglang/srt/layers/sampler.py): greedy through the in-tree row-argmax kernel; temperature /
top-k / top-p through a sorted-probability filter and one multinomial draw per row."""
from __future__ import annotations

from typing import List

import torch

from .dense_kernel import argmax_rows


class Sampler:
    def __init__(self, device: str):
        self.device = device
        self._gens = {}

    def _generator(self, rid: str, seed):
        if seed is None:
            return None
        if rid not in self._gens:
            self._gens[rid] = torch.Generator(device=self.device).manual_seed(int(seed))
        return self._gens[rid]

    def forget(self, rid: str) -> None:
        self._gens.pop(rid, None)

    def __call__(self, logits: torch.Tensor, reqs: List) -> List[int]:
        """logits [n, vocab] (one row per request) -> n token ids."""
        if all(r.sampling_params.temperature <= 0 for r in reqs):
            rows = logits
            if rows.dtype in (torch.bfloat16, torch.float16):
                return argmax_rows(rows.contiguous()).tolist()
            return torch.argmax(rows, dim=-1).tolist()      # fp32 logits: keep their full precision
        out = []
        for i, r in enumerate(reqs):
            sp = r.sampling_params
            row = logits[i].float()
            if sp.temperature <= 0:
                out.append(int(torch.argmax(row)))
                continue
            probs = torch.softmax(row / sp.temperature, -1)
            sorted_p, order = torch.sort(probs, descending=True)
            keep = torch.ones_like(sorted_p, dtype=torch.bool)
            if sp.top_k and sp.top_k > 0:
                keep[sp.top_k:] = False
            if sp.top_p < 1.0:
                keep &= (torch.cumsum(sorted_p, 0) - sorted_p) < sp.top_p
            sorted_p = torch.where(keep, sorted_p, torch.zeros_like(sorted_p))
            pick = torch.multinomial(sorted_p / sorted_p.sum(), 1, generator=self._generator(r.rid, sp.seed))
            out.append(int(order[pick]))
        return out
