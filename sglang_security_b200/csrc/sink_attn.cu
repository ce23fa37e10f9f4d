// Grouped-query softmax attention over a paged token pool whose row holds [keys | values] of all
// key/value heads, with the options of the designs that use it:
//   * RMS norm of the query and key projections over a group of coordinates (the whole projection, or
//     one head) with a learned weight, before rotation;
//   * rotary positions in the interleaved pairing on the first `rot_dims` coordinates of each head;
//   * a causal sliding window that also keeps the first `keep_first` tokens of the sequence visible
//     (at their true positions);
//   * a learned sink per query head: exp(sink) joins the softmax denominator, with no key or value;
//   * key size D and value size E that differ.
//
//   qk_norm_rope_write : per token, from the projection outputs: q -> norm -> rotation -> fp32 queries;
//                        k -> norm -> rotation -> pool row; v -> pool row.  Norms and angles in fp32;
//                        the angle is position x frequency with the frequency held as a sum of two
//                        floats, so it is as exact at position 100000 as at position 10.
//   sink_attn          : one CTA per (token, query head); its 4 warps take the visible keys in tiles of
//                        32 (a lane scores one key, then the warp accumulates the tile's values column
//                        by column), each with a running maximum and sum, merged in a fixed order at the
//                        end.  Scores, weights and sums are fp32.  Every token walks its own list of
//                        visible keys through req_to_token, so prompts portions and decoded tokens
//                        of different requests mix freely in one launch.
#include "common.cuh"

namespace b200 {

constexpr int kPrepThreads = 256;

__device__ __forceinline__ float prep_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < kPrepThreads / 32) ? red[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// One projection row [heads * D] -> normed (groups of `group`, 0 = no norm) and rotated values.
// `inv` holds 1 / rms per group in shared memory.
template <typename T>
__device__ __forceinline__ float normed(const T* row, int idx, const float* w, const float* inv,
                                        int group) {
  float x = to_float<T>(row[idx]);
  if (group > 0) x *= inv[idx / group] * (w ? w[idx] : 1.f);
  return x;
}

template <typename T>
__device__ void group_inv_rms(const T* row, int n, int group, float eps, float* inv, float* red) {
  // few groups (the whole projection, or one per head): one block-wide sum per group
  for (int g = 0; g * group < n; ++g) {
    float s = 0.f;
    for (int d = threadIdx.x; d < group; d += kPrepThreads) {
      const float x = to_float<T>(row[g * group + d]);
      s = fmaf(x, x, s);
    }
    s = prep_block_sum(s, red);
    if (threadIdx.x == 0) inv[g] = 1.0f / sqrtf(s / static_cast<float>(group) + eps);
  }
  __syncthreads();
}

template <typename T, typename TP>
__global__ void __launch_bounds__(kPrepThreads)
qk_norm_rope_write_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                          const T* __restrict__ v, int64_t ldv, const float* __restrict__ qw,
                          const float* __restrict__ kw, int q_group, int k_group, float eps,
                          const float* __restrict__ freq_hi, const float* __restrict__ freq_lo,
                          int rot_dims, const int* __restrict__ tok_pos,
                          const int64_t* __restrict__ loc, TP* __restrict__ pool, int64_t ld_pool,
                          int k_off, int v_off, float* __restrict__ q_out, int64_t ldqo,
                          T* __restrict__ q_out16, int64_t ldqo16, int H, int G, int D, int E) {
  extern __shared__ float prep_smem[];       // [rot_dims / 2] cos, [rot_dims / 2] sin, group scales
  __shared__ float red[kPrepThreads / 32];
  const int t = blockIdx.x, half = rot_dims / 2;
  float* cs = prep_smem;
  float* sn = cs + half;
  float* inv_q = sn + half;
  float* inv_k = inv_q + (q_group > 0 ? (H * D) / q_group : 0);
  const float pos = static_cast<float>(tok_pos[t]);
  for (int i = threadIdx.x; i < half; i += kPrepThreads) {
    const float hi = freq_hi[i], lo = freq_lo ? freq_lo[i] : 0.f;
    const float a = pos * hi;
    const float err = fmaf(pos, hi, -a) + pos * lo;     // what the rounded product dropped
    float s, c;
    sincosf(a, &s, &c);
    cs[i] = c - err * s;
    sn[i] = s + err * c;
  }
  const T* qr = q + t * ldq;
  const T* kr = k + t * ldk;
  if (q_group > 0) group_inv_rms(qr, H * D, q_group, eps, inv_q, red);
  if (k_group > 0) group_inv_rms(kr, G * D, k_group, eps, inv_k, red);
  __syncthreads();
  TP* prow = pool + loc[t] * ld_pool;
  for (int idx = threadIdx.x; idx < (H + G) * D; idx += kPrepThreads) {
    const bool is_q = idx < H * D;
    const int i = is_q ? idx : idx - H * D;
    const int d = i % D;
    const T* row = is_q ? qr : kr;
    const float* w = is_q ? qw : kw;
    const float* inv = is_q ? inv_q : inv_k;
    const int group = is_q ? q_group : k_group;
    float x = normed(row, i, w, inv, group);
    if (d < rot_dims) {
      const float y = normed(row, i - d + (d ^ 1), w, inv, group);   // rot_dims is even: the pair stays in the head
      const float c = cs[d >> 1], s = sn[d >> 1];
      x = (d & 1) ? fmaf(x, c, y * s) : fmaf(x, c, -y * s);
    }
    if (is_q) {
      if (q_out) q_out[t * ldqo + i] = x;
      if (q_out16) q_out16[t * ldqo16 + i] = from_float<T>(x);
    } else {
      prow[k_off + i] = from_float<TP>(x);
    }
  }
  const T* vr = v + t * ldv;
  for (int i = threadIdx.x; i < G * E; i += kPrepThreads)
    prow[v_off + i] = from_float<TP>(to_float<T>(vr[i]));
}

constexpr int kSinkMaxWarps = 16;  // warps per CTA: 4 to 16, by the longest key list (host)
constexpr int kSinkMaxCols = 8;    // value size <= 256

template <typename TP, typename TO>
__global__ void __launch_bounds__(kSinkMaxWarps * 32)
sink_attn_kernel(const float* __restrict__ q, int64_t ldq, const TP* __restrict__ pool,
                 int64_t ld_pool, int k_off, int v_off, const int* __restrict__ req_to_token,
                 int64_t ld_r2t, const int64_t* __restrict__ req_idx, const int* __restrict__ tok_pos,
                 const int* __restrict__ tok_b, const float* __restrict__ sink, float scale, int window,
                 int keep_first, TO* __restrict__ out, int64_t ldo, int H, int G, int D, int E,
                 const int* __restrict__ tok_list) {
  extern __shared__ float sink_smem[];       // q [D], then per warp: acc [E], m, l
  const int kSinkWarps = blockDim.x >> 5;
  float* qs = sink_smem;
  float* wacc = qs + D;
  float* wm = wacc + kSinkWarps * E;
  float* wl = wm + kSinkWarps;
  const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, h = blockIdx.y, g = h / (H / G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = tok_pos[t];
  const int* r2t = req_to_token + req_idx[tok_b[t]] * ld_r2t;
  for (int d = threadIdx.x; d < D; d += kSinkWarps * 32) qs[d] = q[t * ldq + h * D + d] * scale;
  __syncthreads();
  // visible keys: the first `kf` positions, then lo .. p
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int kf = min(keep_first, lo);
  const int nkeys = kf + (p - lo + 1);
  float m = -INFINITY, l = 0.f, acc[kSinkMaxCols];
#pragma unroll
  for (int c = 0; c < kSinkMaxCols; ++c) acc[c] = 0.f;
  const bool vec = (D % 8 == 0) && sizeof(TP) == 2 && (ld_pool % 8 == 0) && ((k_off + g * D) % 8 == 0) &&
                   ((reinterpret_cast<uintptr_t>(pool) & 15) == 0);
  // values: 4 consecutive columns per lane with vector loads when every piece is aligned
  const bool vblk = (E % 4 == 0) && (ld_pool % 4 == 0) && ((v_off + g * E) % 4 == 0) &&
                    ((reinterpret_cast<uintptr_t>(pool) & 15) == 0);
  for (int n0 = warp * 32; n0 < nkeys; n0 += kSinkWarps * 32) {
    const int n = n0 + lane;
    int64_t slot = 0;
    float s = -INFINITY;
    if (n < nkeys) {
      const int j = n < kf ? n : lo + (n - kf);
      slot = r2t[j];
      const TP* kr = pool + slot * ld_pool + k_off + g * D;
      float s0 = 0.f, s1 = 0.f;
      bool done = false;
      if constexpr (sizeof(TP) == 2) {
#pragma unroll 4
        for (int d = 0; vec && d < D; d += 8) {
          const uint4 u = *reinterpret_cast<const uint4*>(kr + d);
          const TP* e8 = reinterpret_cast<const TP*>(&u);
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            s0 = fmaf(qs[d + i], to_float<TP>(e8[i]), s0);
            s1 = fmaf(qs[d + i + 1], to_float<TP>(e8[i + 1]), s1);
          }
        }
        done = vec;
      }
      if (!done) {
        int d = 0;
        for (; d + 1 < D; d += 2) {
          s0 = fmaf(qs[d], to_float<TP>(kr[d]), s0);
          s1 = fmaf(qs[d + 1], to_float<TP>(kr[d + 1]), s1);
        }
        if (d < D) s0 = fmaf(qs[d], to_float<TP>(kr[d]), s0);
      }
      s = s0 + s1;
    }
    float tm = s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
    const float mn = fmaxf(m, tm);
    const float corr = expf(m - mn);          // m = -inf on the first tile: exp(-inf) = 0
    const float pj = n < nkeys ? expf(s - mn) : 0.f;
    float ps = pj;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = l * corr + ps;
    m = mn;
#pragma unroll
    for (int c = 0; c < kSinkMaxCols; ++c) acc[c] *= corr;
    const int cnt = min(32, nkeys - n0);
    // unrolled so that the value rows of several keys are in flight at once (a rolled loop waits a
    // full memory round trip per key)
#pragma unroll 8
    for (int jj = 0; jj < 32; ++jj) {
      if (jj >= cnt) break;
      const float pw = __shfl_sync(0xffffffffu, pj, jj);
      const int64_t sl = __shfl_sync(0xffffffffu, slot, jj);
      const TP* vr = pool + sl * ld_pool + v_off + g * E;
      if (vblk) {
        // a lane owns 4 consecutive columns per 128: one 8-byte (16-bit pool) or 16-byte load each
#pragma unroll
        for (int c = 0; c < kSinkMaxCols / 4; ++c) {
          const int e = 128 * c + 4 * lane;
          if (e < E) {
            float x[4];
            if constexpr (sizeof(TP) == 2) {
              const uint2 u = *reinterpret_cast<const uint2*>(vr + e);
              const TP* t4 = reinterpret_cast<const TP*>(&u);
#pragma unroll
              for (int i = 0; i < 4; ++i) x[i] = to_float<TP>(t4[i]);
            } else {
              const float4 u = *reinterpret_cast<const float4*>(vr + e);
              x[0] = u.x, x[1] = u.y, x[2] = u.z, x[3] = u.w;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[4 * c + i] = fmaf(pw, x[i], acc[4 * c + i]);
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < kSinkMaxCols; ++c) {
          const int e = lane + 32 * c;
          if (e < E) acc[c] = fmaf(pw, to_float<TP>(vr[e]), acc[c]);
        }
      }
    }
  }
  if (lane == 0) {
    wm[warp] = m;
    wl[warp] = l;
  }
#pragma unroll
  for (int c = 0; c < kSinkMaxCols; ++c) {
    const int e = vblk ? 128 * (c / 4) + 4 * lane + (c & 3) : lane + 32 * c;
    if (e < E) wacc[warp * E + e] = acc[c];
  }
  __syncthreads();
  float mt = sink ? sink[h] : -INFINITY;
  for (int w = 0; w < kSinkWarps; ++w) mt = fmaxf(mt, wm[w]);
  float lt = sink ? expf(sink[h] - mt) : 0.f;
  float f[kSinkMaxWarps];
#pragma unroll
  for (int w = 0; w < kSinkMaxWarps; ++w) {
    f[w] = (w < kSinkWarps && wm[w] != -INFINITY) ? expf(wm[w] - mt) : 0.f;
    if (w < kSinkWarps) lt = fmaf(wl[w], f[w], lt);
  }
  for (int e = threadIdx.x; e < E; e += kSinkWarps * 32) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kSinkMaxWarps; ++w)
      if (w < kSinkWarps) o = fmaf(wacc[w * E + e], f[w], o);
    out[t * ldo + h * E + e] = from_float<TO>(o / lt);
  }
}

}  // namespace b200

extern "C" int b200_qk_norm_rope_write(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                       const void* v, int64_t ldv, const float* qw, const float* kw,
                                       int q_group, int k_group, float eps, const float* freq_hi,
                                       const float* freq_lo, int rot_dims, const int* tok_pos,
                                       const int64_t* loc, void* pool, int64_t ld_pool, int k_off,
                                       int v_off, float* q_out, int64_t ldqo, void* q_out16,
                                       int64_t ldqo16, int T, int H, int G, int D, int E, int dtype,
                                       void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(q && k && v && tok_pos && loc && pool && (q_out || q_out16),
               "b200_qk_norm_rope_write: null pointer");
  B200_REQUIRE(T > 0 && H > 0 && G > 0 && D > 0 && E > 0 && rot_dims >= 0 && rot_dims <= D &&
                   rot_dims % 2 == 0 && (rot_dims == 0 || freq_hi),
               "b200_qk_norm_rope_write: head size %d, rotated %d", D, rot_dims);
  B200_REQUIRE((q_group == 0 || (H * D) % q_group == 0) && (k_group == 0 || (G * D) % k_group == 0) &&
                   q_group >= 0 && k_group >= 0,
               "b200_qk_norm_rope_write: norm groups %d / %d do not divide the projections", q_group,
               k_group);
  const size_t smem = sizeof(float) * (rot_dims + (q_group ? H * D / q_group : 0) +
                                       (k_group ? G * D / k_group : 0) + 1);
  B200_REQUIRE(smem <= 48 * 1024, "b200_qk_norm_rope_write: too many norm groups");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("qk_norm_rope_write", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(qk_norm_rope_write_kernel<TT, TT>, dim3(T), dim3(kPrepThreads), smem, st, 1, 0,      \
                static_cast<const TT*>(q), ldq, static_cast<const TT*>(k), ldk,                      \
                static_cast<const TT*>(v), ldv, qw, kw, q_group, k_group, eps, freq_hi, freq_lo,     \
                rot_dims, tok_pos, loc, static_cast<TT*>(pool), ld_pool, k_off, v_off, q_out, ldqo,  \
                static_cast<TT*>(q_out16), ldqo16, H, G, D, E)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_qk_norm_rope_write: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("qk_norm_rope_write_kernel");
  return 0;
}

extern "C" int b200_sink_attn(const float* q, int64_t ldq, const void* pool, int64_t ld_pool, int k_off,
                              int v_off, const int* req_to_token, int64_t ld_r2t,
                              const int64_t* req_idx, const int* tok_pos, const int* tok_b,
                              const float* sink, float scale, int window, int keep_first, void* out,
                              int64_t ldo, int T, int H, int G, int D, int E, const int* tok_list,
                              int max_keys, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(q && pool && req_to_token && req_idx && tok_pos && tok_b && out,
               "b200_sink_attn: null pointer");
  B200_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && E > 0 && E <= 32 * kSinkMaxCols &&
                   window >= 0 && keep_first >= 0,
               "b200_sink_attn: heads %d / %d, key size %d, value size %d (max %d)", H, G, D, E,
               32 * kSinkMaxCols);
  // one warp per 64 keys of the longest list (a hint; 0 = unknown): a warp's tiles are dependent round
  // trips to memory (slots, keys, values), so long lists want many warps and short ones few
  const int kSinkWarps = max_keys <= 0 ? 4 : min(kSinkMaxWarps, max(4, ceil_div(max_keys, 64)));
  const size_t smem = sizeof(float) * (D + kSinkWarps * (E + 2));
  B200_REQUIRE(smem <= 48 * 1024, "b200_sink_attn: key size %d too large", D);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("sink_attn", st);
  const dim3 grid(T, H);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(sink_attn_kernel<TT, TT>, grid, dim3(kSinkWarps * 32), smem, st, 1, 0, q, ldq,       \
                static_cast<const TT*>(pool), ld_pool, k_off, v_off, req_to_token, ld_r2t, req_idx,  \
                tok_pos, tok_b, sink, scale, window, keep_first, static_cast<TT*>(out), ldo, H, G, D, \
                E, tok_list)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_sink_attn: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("sink_attn_kernel");
  return 0;
}
