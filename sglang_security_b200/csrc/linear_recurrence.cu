// Matrix-state linear recurrences over a mixed batch, state in fp32 and carried per sequence:
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T        S [D, E] per head        o_t = S_t^T q_t  (/ den_t)
//
//   kDecay : a_t = decay[head] (constant), b_t = 1, no denominator        (decayed linear attention)
//   kExpGates : log-space input and forget gates with a running stabiliser m (m_0 = 0):
//             li = cap tanh(zi / cap), lf = logsigmoid(cap tanh(zf / cap))   (cap <= 0: no capping)
//             m_t = max(lf + m_(t-1), li), a_t = exp(lf + m_(t-1) - m_t), b_t = exp(li - m_t)
//             n_t = a_t n_(t-1) + b_t k_t ;  den_t = max(|n_t . q_t|, exp(-m_t)) + den_eps     (mLSTM)
//
// One CTA owns (batch entry, head, a slice of the E columns) and walks the entry's new tokens in
// order, so a token's result is the same sum in the same order however the sequence was cut into
// steps.  A thread keeps S[d][e] for one column e and the rows d = p, p + P, ... in registers (P
// lanes of a warp share a column and add their partial dot products by shuffles).  The state row of a
// sequence is read when its portion does not start at position 0 (there it is zero) and written back
// at the end; a single decoded token is the same kernel with a portion of one.
//
//   gated_group_rmsnorm : out = o / sqrt(mean_group(o^2) + eps) * w * sigmoid(z), the mean taken over
//                         consecutive groups of `group` coordinates (one head, or the whole row).
#include "common.cuh"

namespace b200 {

constexpr int kRecThreads = 256;
constexpr int kRecRows = 32;     // rows of S per thread: D <= 32 * P, P <= 32
constexpr int kRecChunk = 16;    // tokens staged in shared memory at a time

__device__ __forceinline__ float rec_act(float z, int act) {
  return act == 1 ? z / (1.0f + expf(-z)) : z;
}
__device__ __forceinline__ float log_sigmoid(float z) {
  return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

template <typename T, bool GATES>
__global__ void __launch_bounds__(kRecThreads)
linear_recurrence_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                         const T* __restrict__ v, int64_t ldv, const float* __restrict__ gates,
                         int64_t ldg, const float* __restrict__ decay, float cap, float q_scale,
                         float den_eps, int act, float* __restrict__ state, int64_t ld_state,
                         const int64_t* __restrict__ slot, const int* __restrict__ tok_pos,
                         const int* __restrict__ ext_start, const int* __restrict__ ext_len,
                         float* __restrict__ out, int64_t ldo, int H, int D, int E, int P) {
  extern __shared__ float rec_smem[];
  const int ES = kRecThreads / P;
  float* qs = rec_smem;                       // [chunk][D]
  float* ks = qs + kRecChunk * D;             // [chunk][D]
  float* vs = ks + kRecChunk * D;             // [chunk][ES]
  float* gi = vs + kRecChunk * ES;            // [chunk]
  float* gf = gi + kRecChunk;                 // [chunk]
  const int b = blockIdx.z, h = blockIdx.y, e0 = blockIdx.x * ES;
  const int tid = threadIdx.x, p = tid % P, col = tid / P, e = e0 + col;
  const int start = ext_start[b], len = ext_len[b];
  if (len <= 0) return;
  const bool fresh = tok_pos[start] == 0;
  // per head: S [D][E], then (gated form) one copy of (n [D], m) per column slice, so that no CTA
  // reads what another CTA of the same launch writes
  const int64_t head_state = static_cast<int64_t>(D) * E + (GATES ? gridDim.x * (D + 1) : 0);
  float* st = state + slot[b] * ld_state + h * head_state;
  float* sn = st + static_cast<int64_t>(D) * E + blockIdx.x * (D + 1);
  float s[kRecRows], nr[GATES ? kRecRows : 1];
  float m = 0.f;
#pragma unroll
  for (int r = 0; r < kRecRows; ++r) {
    const int d = p + r * P;
    s[r] = (!fresh && d < D && e < E) ? st[static_cast<int64_t>(d) * E + e] : 0.f;
    if (GATES) nr[r] = (!fresh && d < D) ? sn[d] : 0.f;
  }
  if (GATES && !fresh) m = sn[D];
  const float lam = GATES ? 0.f : decay[h];
  for (int c0 = 0; c0 < len; c0 += kRecChunk) {
    const int n = min(kRecChunk, len - c0);
    __syncthreads();
    for (int idx = tid; idx < n * D; idx += kRecThreads) {
      const int j = idx / D, d = idx - j * D;
      const int64_t row = start + c0 + j;
      qs[j * D + d] = rec_act(to_float<T>(q[row * ldq + h * D + d]), act) * q_scale;
      ks[j * D + d] = rec_act(to_float<T>(k[row * ldk + h * D + d]), act);
    }
    for (int idx = tid; idx < n * ES; idx += kRecThreads) {
      const int j = idx / ES, c = idx - j * ES;
      const int64_t row = start + c0 + j;
      vs[j * ES + c] = (e0 + c < E) ? rec_act(to_float<T>(v[row * ldv + h * E + e0 + c]), act) : 0.f;
    }
    if (GATES && tid < n) {
      const int64_t row = start + c0 + tid;
      float zi = gates[row * ldg + h], zf = gates[row * ldg + H + h];
      if (cap > 0.f) {
        zi = cap * tanhf(zi / cap);
        zf = cap * tanhf(zf / cap);
      }
      gi[tid] = zi;
      gf[tid] = log_sigmoid(zf);
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      float a = lam, bb = 1.f;
      if (GATES) {
        const float li = gi[j], lf = gf[j];
        const float mn = fmaxf(lf + m, li);
        a = expf(lf + m - mn);
        bb = expf(li - mn);
        m = mn;
      }
      const float ve = vs[j * ES + col] * bb;
      const float* kj = ks + j * D;
      const float* qj = qs + j * D;
      float acc = 0.f, accn = 0.f;
#pragma unroll
      for (int r = 0; r < kRecRows; ++r) {
        const int d = p + r * P;
        if (d < D) {
          const float kd = kj[d], qd = qj[d];
          s[r] = fmaf(a, s[r], kd * ve);
          acc = fmaf(s[r], qd, acc);
          if (GATES) {
            nr[r] = fmaf(a, nr[r], bb * kd);
            accn = fmaf(nr[r], qd, accn);
          }
        }
      }
      for (int o = P >> 1; o > 0; o >>= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (GATES) accn += __shfl_xor_sync(0xffffffffu, accn, o);
      }
      if (p == 0 && e < E) {
        float y = acc;
        if (GATES) y = acc / (fmaxf(fabsf(accn), expf(-m)) + den_eps);
        out[(start + c0 + j) * ldo + h * E + e] = y;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRecRows; ++r) {
    const int d = p + r * P;
    if (d < D && e < E) st[static_cast<int64_t>(d) * E + e] = s[r];
    if (GATES && d < D && col == 0) sn[d] = nr[r];
  }
  if (GATES && tid == 0) sn[D] = m;
}

template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_kernel(const float* __restrict__ o, int64_t ldo, const float* __restrict__ w,
                           const TZ* __restrict__ z, int64_t ldz, TO* __restrict__ out, int64_t ldout,
                           int N, int group, float eps) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* row = o + t * ldo;
  for (int g0 = warp * group; g0 < N; g0 += 8 * group) {
    float ss = 0.f;
    for (int d = lane; d < group; d += 32) {
      const float x = row[g0 + d];
      ss = fmaf(x, x, ss);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float r = 1.0f / sqrtf(ss / static_cast<float>(group) + eps);
    for (int d = lane; d < group; d += 32) {
      float y = row[g0 + d] * r;
      if (w) y *= w[g0 + d];
      if (z) y *= 1.0f / (1.0f + expf(-to_float<TZ>(z[t * ldz + g0 + d])));
      out[t * ldout + g0 + d] = from_float<TO>(y);
    }
  }
}

}  // namespace b200

static int rec_parts(int D) {
  int P = 1;
  while (b200::kRecRows * P < D) P <<= 1;
  return P;
}

// fp32 values one sequence keeps per layer (see the layout in the kernel)
extern "C" int64_t b200_linear_recurrence_state_width(int H, int D, int E, int gated) {
  if (H <= 0 || D <= 0 || E <= 0 || D > b200::kRecRows * 32) return -1;
  const int slices = b200::ceil_div(E, b200::kRecThreads / rec_parts(D));
  return static_cast<int64_t>(H) * (static_cast<int64_t>(D) * E + (gated ? slices * (D + 1) : 0));
}

extern "C" int b200_linear_recurrence(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                      const void* v, int64_t ldv, const float* gates, int64_t ldg,
                                      const float* decay, float cap, float q_scale, float den_eps,
                                      int act, float* state, int64_t ld_state, const int64_t* slot,
                                      const int* tok_pos, const int* ext_start, const int* ext_len,
                                      float* out, int64_t ldo, int batch, int H, int D, int E,
                                      int dtype, void* stream) {
  using namespace b200;
  if (batch == 0) return 0;
  B200_REQUIRE(q && k && v && state && slot && tok_pos && ext_start && ext_len && out,
               "b200_linear_recurrence: null pointer");
  B200_REQUIRE((gates != nullptr) != (decay != nullptr),
               "b200_linear_recurrence: give either gate pre-activations or a decay per head");
  B200_REQUIRE(batch > 0 && H > 0 && D > 0 && E > 0 && D <= kRecRows * 32 && (act == 0 || act == 1),
               "b200_linear_recurrence: heads %d, key size %d (max %d), value size %d", H, D,
               kRecRows * 32, E);
  const int P = rec_parts(D);
  const int ES = kRecThreads / P;
  const size_t smem = static_cast<size_t>(kRecChunk) * (2 * D + ES + 2) * sizeof(float);
  B200_REQUIRE(smem <= 200 * 1024, "b200_linear_recurrence: key size %d too large", D);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("linear_recurrence", st);
  const dim3 grid(ceil_div(E, ES), H, batch);
#define LAUNCH(TT, G)                                                                                \
  do {                                                                                               \
    auto kern = linear_recurrence_kernel<TT, G>;                                                     \
    if (smem > 48 * 1024)                                                                            \
      B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                        static_cast<int>(smem)));                                    \
    launch_kernel(kern, grid, dim3(kRecThreads), smem, st, 1, 0, static_cast<const TT*>(q), ldq,     \
                  static_cast<const TT*>(k), ldk, static_cast<const TT*>(v), ldv, gates, ldg, decay, \
                  cap, q_scale, den_eps, act, state, ld_state, slot, tok_pos, ext_start, ext_len,    \
                  out, ldo, H, D, E, P);                                                             \
  } while (0)
#define BY_G(TT)                  \
  do {                            \
    if (gates) LAUNCH(TT, true);  \
    else LAUNCH(TT, false);       \
  } while (0)
  if (dtype == B200_BF16) BY_G(__nv_bfloat16);
  else if (dtype == B200_F16) BY_G(__half);
  else if (dtype == B200_F32) BY_G(float);
  else B200_REQUIRE(false, "b200_linear_recurrence: dtype %d", dtype);
#undef BY_G
#undef LAUNCH
  B200_CHECK_LAUNCH("linear_recurrence_kernel");
  return 0;
}

extern "C" int b200_gated_group_rmsnorm(const float* o, int64_t ldo, const float* w, const void* z,
                                        int64_t ldz, void* out, int64_t ldout, int T, int N,
                                        int group, float eps, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(o && out && T > 0 && N > 0 && group > 0 && N % group == 0,
               "b200_gated_group_rmsnorm: %d coordinates in groups of %d", N, group);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("gated_group_rmsnorm", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(gated_group_rmsnorm_kernel<TT, TT>, dim3(T), dim3(256), 0, st, 1, 0, o, ldo, w,      \
                static_cast<const TT*>(z), ldz, static_cast<TT*>(out), ldout, N, group, eps)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_gated_group_rmsnorm: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("gated_group_rmsnorm_kernel");
  return 0;
}
