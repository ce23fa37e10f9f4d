"""Norm layers over a 32-bit residual stream (csrc/norm_shift.cu).

`ScalarRMSNorm`: x / sqrt(mean(x^2) + eps) times ONE learned gain shared by all coordinates.  The input
is the fp32 residual; the output is produced directly in the dtype of the following matrix products.
`TokenShift`: the learned per-coordinate mix of a token's normed activation with the previous
token's, h + (h_prev - h) * mu, whose carry between steps is a row of a `SeqStatePool`.  The two are
one kernel launch (`ScalarRMSNorm.forward_shifted`)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import _lib


def _launch(x, gain, weight, eps, mu, state, meta, slot, out_h, out_hm):
    if not x.is_cuda:
        raise _lib.B200Error("ScalarRMSNorm: tensor must live on a CUDA device (no CPU path)")
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise _lib.B200Error("ScalarRMSNorm: the residual must be a 2-D fp32 tensor with contiguous rows")
    t, w = x.shape
    ref = out_h if out_h is not None else out_hm
    rc = _lib.load().b200_scalar_rmsnorm_shift(
        x.data_ptr(), x.stride(0), _lib.ptr(gain), _lib.ptr(weight), float(eps), _lib.ptr(mu),
        _lib.ptr(state), state.stride(0) if state is not None else 0,
        _lib.ptr(meta.tok_pos) if meta is not None else None,
        _lib.ptr(meta.tok_b) if meta is not None else None,
        _lib.ptr(meta.ext_start) if meta is not None else None,
        _lib.ptr(meta.ext_len) if meta is not None else None, _lib.ptr(slot),
        _lib.ptr(out_h), out_h.stride(0) if out_h is not None else 0,
        _lib.ptr(out_hm), out_hm.stride(0) if out_hm is not None else 0, t, w,
        _lib.dtype_code(ref.dtype), _lib.current_stream())
    _lib.check(rc, "b200_scalar_rmsnorm_shift")


class TokenShift(nn.Module):
    """Owner of the mix vector mu [width] (fp32)."""

    def __init__(self, width: int):
        super().__init__()
        self.mu = nn.Parameter(torch.zeros(width, dtype=torch.float32), requires_grad=False)


class ScalarRMSNorm(nn.Module):
    def __init__(self, eps: float):
        super().__init__()
        self.gain = nn.Parameter(torch.ones((), dtype=torch.float32), requires_grad=False)
        self.variance_epsilon = eps

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        _launch(x, self.gain, None, self.variance_epsilon, None, None, None, None, out, None)
        return out

    def forward_shifted(self, x: torch.Tensor, out_dtype: torch.dtype, shift: TokenShift, meta,
                        state: Optional[torch.Tensor], slot: Optional[torch.Tensor],
                        need_plain: bool = True) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        """-> (h, hm): the normed rows and their token-shifted copy.  `meta` carries the batch's
        tok_pos / tok_b / ext_start / ext_len (int32, device); `state` [slots, width] fp32 holds each
        sequence's last normed row from the step before and receives the new one (`slot` [bs])."""
        h = torch.empty(x.shape, dtype=out_dtype, device=x.device) if need_plain else None
        hm = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        _launch(x, self.gain, None, self.variance_epsilon, shift.mu, state, meta, slot, h, hm)
        return h, hm


def residual_combine(x: torch.Tensor, a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None,
                     expert_rows: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None,
                     shared: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> None:
    """x (fp32, in place) += a + b + sum_k topk_weights[t, k] * expert_rows[t * top + k] + gate[t] *
    shared[t]; every term is optional and summed in fp32 before it meets the residual."""
    terms = [v for v in (a, b, expert_rows, shared) if v is not None]
    if not terms:
        return
    dt = terms[0].dtype
    for v in terms:
        if v.dtype != dt or v.stride(-1) != 1:
            raise _lib.B200Error("residual_combine: terms must share a dtype and have contiguous rows")
    t, w = x.shape
    top = topk_weights.shape[1] if topk_weights is not None else 0
    ld = lambda v: v.stride(0) if v is not None else 0
    rc = _lib.load().b200_residual_combine(
        x.data_ptr(), x.stride(0), _lib.ptr(a), ld(a), _lib.ptr(b), ld(b), _lib.ptr(expert_rows),
        ld(expert_rows), _lib.ptr(topk_weights), top, _lib.ptr(shared), ld(shared), _lib.ptr(gate),
        t, w, _lib.dtype_code(dt), _lib.current_stream())
    _lib.check(rc, "b200_residual_combine")
