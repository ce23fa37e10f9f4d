"""Latent attention layer (queries and keys/values through low-rank latents, one rotated key part
shared by all heads, optional causal sliding window, optional reuse of another layer's latent) over
LatentTokenToKVPool, on the kernels of csrc/latent_attn.cu.

Per token with mixer input h (dims: H heads, `dim` unrotated + `rot_dim` rotated query/key
coordinates, value size `vdim`, latent size R):
    [cq_raw | ckv_raw] = W_down h                    (one fused GEMM; layers that borrow a latent: W_dq only)
    cq = RMSnorm(cq_raw) * w_q ;  c = RMSnorm(ckv_raw[:R]) * w_kv ;  kr = rotary(ckv_raw[R:])  -> pool
    q  = W_uq cq                                      [H, dim + rot_dim]
    q_lat[h] = W_uk[h]^T q[h, :dim]                   (absorbed key up-projection, fp32 result)
    p  = softmax_j((q_lat[h] . c_j + rotary(q[h, dim:]) . kr_j) * scale)   over the visible keys
    out = W_o concat_h(W_uv[h] sum_j p_j c_j)
Only c and kr are cached, and the same kernel runs prompt portions and decoded tokens, so a
position's result does not depend on how the sequence was cut into steps."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import _lib
from ..linear import ColumnParallelLinear, RowParallelLinear
from ..rotary_embedding import InterleavedRotary


_SM_COUNT = 148      # B200


def _bmm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched product with a fp32 result (16-bit operands keep their tensor-core path)."""
    if a.dtype == torch.float32:
        return torch.bmm(a, b)
    try:
        return torch.bmm(a, b, out_dtype=torch.float32)
    except (TypeError, RuntimeError):
        return torch.bmm(a.float(), b.float())


class LatentAttention(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 q_rank: int, scale: float, layer_id: int, eps: float, window: Optional[int] = None,
                 rope_base: float = 10000.0, rope_dims: Optional[int] = None,
                 kv_layer_id: Optional[int] = None, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.width, self.heads, self.dim, self.rot_dim, self.vdim = width, heads, dim, rot_dim, vdim
        self.kv_rank, self.q_rank, self.scale, self.eps = kv_rank, q_rank, float(scale), eps
        self.layer_id = layer_id
        self.kv_layer_id = layer_id if kv_layer_id is None else kv_layer_id
        self.owns_kv = self.kv_layer_id == layer_id
        self.window = int(window) if window else 0
        kw = dict(bias=False, params_dtype=params_dtype, tp_rank=0, tp_size=1)
        down_out = q_rank + (kv_rank + rot_dim if self.owns_kv else 0)
        self.down_proj = ColumnParallelLinear(width, down_out, **kw)     # [W_dq ; W_dkv]
        self.q_up_proj = ColumnParallelLinear(q_rank, heads * (dim + rot_dim), **kw)
        self.o_proj = RowParallelLinear(heads * vdim, width, **kw)
        self.w_uk = nn.Parameter(torch.empty(heads, dim, kv_rank, dtype=params_dtype), requires_grad=False)
        self.w_uv_t = nn.Parameter(torch.empty(heads, kv_rank, vdim, dtype=params_dtype), requires_grad=False)
        self.q_norm_weight = nn.Parameter(torch.ones(q_rank, dtype=torch.float32), requires_grad=False)
        self.kv_norm_weight = nn.Parameter(torch.ones(kv_rank, dtype=torch.float32), requires_grad=False)
        self.rotary = InterleavedRotary(rot_dim if rope_dims is None else rope_dims, rope_base)
        if self.rotary.dims > rot_dim:
            raise ValueError("rotary dims exceed the rotated part of a head")

    # ---- checkpoint tensors ([out, in]) -> the layouts above ------------------------------------
    def load_down(self, w_dq: torch.Tensor, w_dkv: Optional[torch.Tensor]) -> None:
        w = w_dq if w_dkv is None else torch.cat([w_dq, w_dkv], 0)
        self.down_proj.weight.data.copy_(w)

    def load_uk(self, w: torch.Tensor) -> None:      # [H * dim, R]
        self.w_uk.data.copy_(w.view(self.heads, self.dim, self.kv_rank))

    def load_uv(self, w: torch.Tensor) -> None:      # [H * vdim, R] -> [H, R, vdim]
        self.w_uv_t.data.copy_(w.view(self.heads, self.vdim, self.kv_rank).transpose(1, 2))

    def forward(self, h: torch.Tensor, forward_batch) -> torch.Tensor:
        fb = forward_batch
        t = h.shape[0]
        lib = _lib.load()
        code = _lib.dtype_code(h.dtype)
        pool = fb.token_to_kv_pool
        cache = pool.get_kv_buffer(self.layer_id)
        raw, _ = self.down_proj(h)
        cq = torch.empty((t, self.q_rank), dtype=h.dtype, device=h.device)
        kv_raw = raw[:, self.q_rank:] if self.owns_kv else None
        inv_freq = self.rotary.inv_freq
        rc = lib.b200_latent_prep(
            raw.data_ptr(), raw.stride(0), self.q_rank, self.q_norm_weight.data_ptr(), cq.data_ptr(),
            cq.stride(0), _lib.ptr(kv_raw), raw.stride(0), self.kv_rank, self.rot_dim, self.rotary.dims,
            self.kv_norm_weight.data_ptr(), _lib.ptr(inv_freq), fb.tok_pos.data_ptr(),
            fb.out_cache_loc.data_ptr(), cache.data_ptr(), cache.stride(0), float(self.eps), t, code,
            _lib.current_stream())
        _lib.check(rc, "b200_latent_prep")
        q, _ = self.q_up_proj(cq)
        q3 = q.view(t, self.heads, self.dim + self.rot_dim)
        q_lat = _bmm_f32(q3[:, :, :self.dim].transpose(0, 1), self.w_uk)           # [H, T, R] fp32
        o_lat = torch.empty((self.heads, t, self.kv_rank), dtype=h.dtype, device=h.device)
        # few tokens with many keys each (decoding): spread every token's keys over several CTAs
        keys = min(self.window, int(fb.max_seq_len)) if self.window else int(fb.max_seq_len)
        ctas = t * ((self.heads + 63) // 64)
        splits = 1
        if h.dtype != torch.float32 and ctas < _SM_COUNT and keys > 128:
            splits = max(1, min((keys + 63) // 64, (2 * _SM_COUNT) // ctas, 64))
        ws = (torch.empty(splits * t * self.heads * (self.kv_rank + 2), dtype=torch.float32, device=h.device)
              if splits > 1 else None)
        rc = lib.b200_latent_attn(
            q_lat.data_ptr(), q_lat.stride(1), q_lat.stride(0), q.data_ptr(), q3.stride(0), q3.stride(1),
            self.dim, cache.data_ptr(), cache.stride(0), fb.req_to_token_pool.req_to_token.data_ptr(),
            fb.req_to_token_pool.req_to_token.stride(0), fb.req_pool_indices.data_ptr(),
            fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), fb.ext_start.data_ptr(), fb.ext_len.data_ptr(),
            fb.batch_size, _lib.ptr(inv_freq), self.rotary.dims, t,
            self.heads, self.kv_rank, self.rot_dim, self.window, int(fb.max_seq_len), self.scale,
            o_lat.data_ptr(), o_lat.stride(1), o_lat.stride(0), splits, _lib.ptr(ws),
            ws.numel() if ws is not None else 0, code, _lib.current_stream())
        _lib.check(rc, "b200_latent_attn")
        v = torch.bmm(o_lat, self.w_uv_t)                                          # [H, T, vdim]
        out, _ = self.o_proj(v.transpose(0, 1).reshape(t, self.heads * self.vdim))
        return out
