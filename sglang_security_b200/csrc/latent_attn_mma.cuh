// Tensor-core instance of the latent attention (16-bit storage types): the same interface as
// latent_attn_kernel, tiled like a flash attention over the shared latent rows.
//   CTA  = TQ consecutive tokens of one request x HG heads (<= 64 rows, row = tq * HG + hh), 8 warps:
//          warp w owns rows 16 * (w & 3) .. +15 and the output columns of half (w >> 2) (CW each), so
//          the fp32 output accumulators of a 512-wide latent fit the register file; both halves
//          compute the (identical) scores of their rows.
//   keys = the union of the tokens' windows, in tiles of 32 gathered by slot with 16-byte cp.async
//          into a double buffer; the c part of a key row is both the key and the value operand.
//   math = mma.sync m16n8k16, fp32 accumulation; scores, running max / sum and the rescaling in
//          fp32; the weights are rounded to the storage type only as the operand of P.V.
#pragma once
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kLaRows = 64, kLaKeys = 32, kLaThreads = 256;

// CW: output columns per warp half (multiple of 16); the latent is padded to 2 * CW >= R16.
template <typename T, int CW>
__global__ void __launch_bounds__(kLaThreads, 1)
latent_attn_mma_kernel(const float* __restrict__ q_lat, int64_t ldql_t, int64_t ldql_h,
                       const T* __restrict__ q_raw, int64_t ldqr_t, int64_t ldqr_h, int q_rot_off,
                       const T* __restrict__ cache, int64_t ldc, const int* __restrict__ r2t,
                       int64_t ld_r2t, const int64_t* __restrict__ req_pool,
                       const int* __restrict__ tok_pos, const int* __restrict__ ext_start,
                       const int* __restrict__ ext_len, int bs, const float* __restrict__ inv_freq,
                       int rot_dims, int H, int HG, int TQ, int R, int rot, int window, float scale,
                       T* __restrict__ out, int64_t ldo_t, int64_t ldo_h, int nsplit,
                       float* __restrict__ ws, int T_total) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int R16 = (R + 15) & ~15, rot16 = (rot + 15) & ~15;
  const int Dp = R16 + rot16, ldS = Dp + 8;          // row stride in elements: odd multiple of 16 bytes
  T* q_s = reinterpret_cast<T*>(smem_raw);            // [64][ldS]
  T* k_s = q_s + kLaRows * ldS;                       // [2][32][ldS]
  // ---- which tokens ---------------------------------------------------------------------------
  int b = 0, tile = blockIdx.x;
  for (; b < bs; ++b) {
    const int nt = (ext_len[b] + TQ - 1) / TQ;
    if (tile < nt) break;
    tile -= nt;
  }
  if (b >= bs) return;
  const int t0 = ext_start[b] + tile * TQ;
  const int ntok = min(TQ, ext_len[b] - tile * TQ);
  const int p0 = tok_pos[t0];
  const int h0 = blockIdx.y * HG;
  const int nh = min(HG, H - h0);
  const int64_t rp = req_pool[b];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // ---- zero the tiles (pads and rows that are never loaded must be finite), then stage Q --------
  {
    uint4 z = make_uint4(0, 0, 0, 0);
    uint4* p = reinterpret_cast<uint4*>(smem_raw);
    const int n16 = (kLaRows + 2 * kLaKeys) * ldS * static_cast<int>(sizeof(T)) / 16;
    for (int i = tid; i < n16; i += kLaThreads) p[i] = z;
  }
  __syncthreads();
  for (int e = tid; e < ntok * nh * R; e += kLaThreads) {
    const int r = e / R, d = e - r * R;
    const int tq = r / nh, hh = r - tq * nh;
    q_s[(tq * HG + hh) * ldS + d] = from_float<T>(q_lat[(t0 + tq) * ldql_t + (h0 + hh) * ldql_h + d]);
  }
  const int half_rot = (rot + 1) / 2;
  for (int e = tid; e < ntok * nh * half_rot; e += kLaThreads) {
    const int r = e / half_rot, i = e - r * half_rot;
    const int tq = r / nh, hh = r - tq * nh;
    const T* qr = q_raw + (t0 + tq) * ldqr_t + (h0 + hh) * ldqr_h + q_rot_off;
    float u = to_float<T>(qr[2 * i]), v = (2 * i + 1 < rot) ? to_float<T>(qr[2 * i + 1]) : 0.f;
    if (2 * i + 1 < rot_dims) {
      float s, c;
      sincosf(static_cast<float>(p0 + tq) * inv_freq[i], &s, &c);
      const float u2 = u * c - v * s, v2 = v * c + u * s;
      u = u2;
      v = v2;
    }
    T* dst = q_s + (tq * HG + hh) * ldS + R16 + 2 * i;
    dst[0] = from_float<T>(u);
    if (2 * i + 1 < rot) dst[1] = from_float<T>(v);
  }
  // ---- key range ------------------------------------------------------------------------------
  const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
  const int hi = p0 + ntok - 1;
  const int ntiles = (hi - lo + kLaKeys) / kLaKeys;
  // split-KV: this CTA takes tiles [tl0, tl1) and leaves (m, l, unnormalised acc) for the merge kernel
  const int per_split = (ntiles + nsplit - 1) / nsplit;
  const int tl0 = blockIdx.z * per_split, tl1 = min(ntiles, tl0 + per_split);
  const int cpk = (R + rot) / 8;                      // 16-byte chunks per key row (R, rot multiples of 8)
  const int cR = R / 8;
  // 8 threads copy one key row; a thread reads its key's slot id ONE tile ahead of the copy, so the
  // gather never waits on the request table
  const int lkey = tid >> 3, lsub = tid & 7;
  static_assert(kLaThreads == kLaKeys * 8, "8 loader threads per key");
  auto slot_of = [&](int tl) -> int64_t {
    const int j = lo + tl * kLaKeys + lkey;
    return (tl < tl1 && j <= hi) ? static_cast<int64_t>(r2t[rp * ld_r2t + j]) : -1;
  };
  auto load_tile = [&](int buf, int64_t slot) {
    if (slot >= 0) {
      const T* src = cache + slot * ldc;
      T* drow = k_s + (buf * kLaKeys + lkey) * ldS;
      for (int ch = lsub; ch < cpk; ch += 8)
        cp_async16(smem_u32(drow + (ch < cR ? ch * 8 : R16 + (ch - cR) * 8)), src + ch * 8);
    }
    cp_async_commit();
  };
  int64_t slot_next = slot_of(tl0);
  if (tl0 < tl1) {
    load_tile(0, slot_next);
    slot_next = slot_of(tl0 + 1);
  }
  // ---- per-warp state ---------------------------------------------------------------------------
  const int rw = (warp & 3) * 16, chalf = warp >> 2;
  const int g = lane >> 2, tq4 = lane & 3;
  const int row0 = rw + g, row1 = rw + g + 8;          // the two rows this thread holds
  int pos_r[2];
  bool ok_r[2];
  {
    const int rr[2] = {row0, row1};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int tq = rr[i] / HG, hh = rr[i] - tq * HG;
      ok_r[i] = tq < ntok && hh < nh;
      pos_r[i] = p0 + tq;
    }
  }
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  float acc[CW / 8][4];
#pragma unroll
  for (int n = 0; n < CW / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  const float sl2 = scale * 1.4426950408889634f;
  // a warp whose 16 rows are all padding (a decoded token fills HG of the 64 rows) only helps to
  // load the key tiles: it issues no ldmatrix / mma and writes nothing
  const bool warp_has_rows = rw < (ntok - 1) * HG + nh;
  const uint32_t q_base = smem_u32(q_s + (rw + (lane & 15)) * ldS + (lane >> 4) * 8);
  const int col0 = chalf * CW;

  for (int tl = tl0; tl < tl1; ++tl) {
    cp_async_wait<0>();
    __syncthreads();
    if (tl + 1 < tl1) {
      load_tile((tl + 1 - tl0) & 1, slot_next);
      slot_next = slot_of(tl + 2);
    }
    const T* kt = k_s + ((tl - tl0) & 1) * kLaKeys * ldS;
    if (!warp_has_rows) continue;
    // S = Q K^T : 16 rows x 32 keys
    float s[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    const uint32_t k_base = smem_u32(kt + ((lane & 7) + ((lane >> 4) << 3)) * ldS + ((lane >> 3) & 1) * 8);
    for (int ks = 0; ks < Dp; ks += 16) {
      uint32_t a[4];
      ldsm_x4(a[0], a[1], a[2], a[3], q_base + ks * static_cast<int>(sizeof(T)));
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, k_base + (np * 16 * ldS + ks) * static_cast<int>(sizeof(T)));
        mma16816<T>(s[2 * np], a, b0, b1);
        mma16816<T>(s[2 * np + 1], a, b2, b3);
      }
    }
    // mask, online softmax (rows row0: regs 0,1; row1: regs 2,3)
    const int jb = lo + tl * kLaKeys + 2 * tq4;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1, j = jb + n * 8 + (e & 1);
        const bool vis = ok_r[i] && j <= pos_r[i] && (window <= 0 || j > pos_r[i] - window);
        s[n][e] = vis ? s[n][e] * sl2 : -INFINITY;
        mx[i] = fmaxf(mx[i], s[n][e]);
      }
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float mn = fmaxf(m_r[i], mx[i]);
      corr[i] = (mn == -INFINITY) ? 1.f : exp2f(m_r[i] - mn);
      m_r[i] = mn;
    }
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const float p = (m_r[i] == -INFINITY) ? 0.f : exp2f(s[n][e] - m_r[i]);
        s[n][e] = p;
        ps[i] += p;
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 1);
      ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 2);
      l_r[i] = l_r[i] * corr[i] + ps[i];
    }
#pragma unroll
    for (int n = 0; n < CW / 8; ++n) {
      acc[n][0] *= corr[0];
      acc[n][1] *= corr[0];
      acc[n][2] *= corr[1];
      acc[n][3] *= corr[1];
    }
    // O += P V  (V = the c part of the key tile, columns col0 .. col0 + CW)
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      uint32_t a[4];
      a[0] = pack2<T>(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack2<T>(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      const uint32_t v_base = smem_u32(kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldS + col0 + (lane >> 4) * 8);
#pragma unroll
      for (int n = 0; n < CW / 16; ++n) {
        if (col0 + n * 16 < R16) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(b0, b1, b2, b3, v_base + n * 16 * static_cast<int>(sizeof(T)));
          mma16816<T>(acc[2 * n], a, b0, b1);
          mma16816<T>(acc[2 * n + 1], a, b2, b3);
        }
      }
    }
  }
  // ---- write out[t, h, col] -----------------------------------------------------------------------
  const int rr[2] = {row0, row1};
  if (nsplit > 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (!ok_r[i]) continue;
      const int tq = rr[i] / HG, hh = rr[i] - tq * HG;
      float* wrow = ws + ((static_cast<int64_t>(blockIdx.z) * T_total + (t0 + tq)) * H + (h0 + hh)) * (R + 2);
      if (chalf == 0 && tq4 == 0) {
        wrow[0] = m_r[i];
        wrow[1] = l_r[i];
      }
#pragma unroll
      for (int n = 0; n < CW / 8; ++n) {
        const int c = col0 + n * 8 + 2 * tq4;
        if (c < R) wrow[2 + c] = acc[n][2 * i];
        if (c + 1 < R) wrow[2 + c + 1] = acc[n][2 * i + 1];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!ok_r[i]) continue;
    const int tq = rr[i] / HG, hh = rr[i] - tq * HG;
    const float inv = 1.0f / l_r[i];
    T* orow = out + (t0 + tq) * ldo_t + (h0 + hh) * ldo_h;
#pragma unroll
    for (int n = 0; n < CW / 8; ++n) {
      const int c = col0 + n * 8 + 2 * tq4;
      if (c < R) orow[c] = from_float<T>(acc[n][2 * i] * inv);
      if (c + 1 < R) orow[c + 1] = from_float<T>(acc[n][2 * i + 1] * inv);
    }
  }
}

// out[t, h, :] = sum_z acc_z 2^(m_z - M) / sum_z l_z 2^(m_z - M) over the split-KV partials
template <typename T>
__global__ void __launch_bounds__(128)
latent_attn_merge_kernel(const float* __restrict__ ws, int nsplit, int T_total, int H, int R,
                         T* __restrict__ out, int64_t ldo_t, int64_t ldo_h) {
  const int t = blockIdx.x / H, h = blockIdx.x - t * H;
  float M = -INFINITY;
  for (int z = 0; z < nsplit; ++z)
    M = fmaxf(M, ws[((static_cast<int64_t>(z) * T_total + t) * H + h) * (R + 2)]);
  float L = 0.f;
  for (int z = 0; z < nsplit; ++z) {
    const float* p = ws + ((static_cast<int64_t>(z) * T_total + t) * H + h) * (R + 2);
    if (p[0] != -INFINITY) L = fmaf(p[1], exp2f(p[0] - M), L);
  }
  const float inv = 1.0f / L;
  for (int d = threadIdx.x; d < R; d += 128) {
    float o = 0.f;
    for (int z = 0; z < nsplit; ++z) {
      const float* p = ws + ((static_cast<int64_t>(z) * T_total + t) * H + h) * (R + 2);
      if (p[0] != -INFINITY) o = fmaf(p[2 + d], exp2f(p[0] - M), o);
    }
    out[t * ldo_t + h * ldo_h + d] = from_float<T>(o * inv);
  }
}

}  // namespace b200
