// Recurrences with a matrix state per head and a decay per key channel, walked token by token in float32:
//
//   gated linear attention        S_t = diag(alpha_t) S_(t-1) + k_t v_t^T                      o_t = S_t^T q_t
//                                 alpha = sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau),  q times dim^(-1/2)
//   the generalized delta rule    S_t = diag(w_t) S_(t-1) - (a_t u_t)(u_t^T S_(t-1)) + k_t v_t^T  o_t = S_t^T r_t
//                                 w = exp(-coef * sigmoid(z)),  a = sigmoid(a_in + bias),  u = k / sqrt(sum k^2 + eps)
//
// and the second half of a two-step product of low rank that makes the decays' z:
//   low_rank_out    out[t, c] = bias[c] + sum_r act(lr[t, r]) * W2[c, r]     (float32 sums, act none or tanh)
//
// A block owns up to 64 value columns of one (sequence, head); four neighbouring lanes share a column, each with a
// quarter of its rows of S in registers (the 16-byte parts s, s + 4, ... of a key row, so that the four lanes'
// shared-memory reads lie side by side) through all of the sequence's tokens of the step; what a token needs of all
// rows (u^T S, S^T q) the four add up by two shuffles.  q, k, the decays (and the unit key and a * u) of a stage of
// tokens are made once in shared memory by all threads together, rows padded with zeros to a multiple of 16.  A
// token's arithmetic does not depend on where a stage or a step begins, so a sequence's outputs are the same bits
// however it is cut into steps.  A sequence that starts at position 0 starts from zeros whatever its state rows
// hold; padding sequences (slot -1) are skipped.
#include "common.cuh"

namespace {

constexpr int kColumns = 64;       // value columns a block, at most
constexpr int kSub = 4;            // lanes that share a column
constexpr int kStageBytes = 40 * 1024;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float sum_of_four(float v) {     // over the four lanes of a column
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

enum : int { kRuleGla = 0, kRuleDelta = 1 };

// R: rows of S a lane keeps (the padded key size is at most 4 R); register r = 4 g + e is row 4 (sub + 4 g) + e
template <typename T, int RULE, int R>
__global__ void __launch_bounds__(kColumns * kSub)
recurrence_kernel(const T* __restrict__ proj, long long stride, int q_col, int k_col, int v_col, int a_col,
                  const float* __restrict__ a_bias, const float* __restrict__ z, float coef, float unit_eps,
                  float* __restrict__ state, float* __restrict__ out, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int D, int V, int Dp,
                  int stage) {
  extern __shared__ __align__(16) float sm[];
  const int n_arrays = RULE == kRuleDelta ? 5 : 3;
  float* qs = sm;                    // [stage][Dp]
  float* ks = qs + stage * Dp;
  float* ds = ks + stage * Dp;       // the decay of every key channel
  float* us = ds + stage * Dp;       // the unit key (delta rule)
  float* as = us + stage * Dp;       // rate, then rate * unit key
  float* vs = sm + n_arrays * stage * Dp;   // [stage][columns of the block]
  const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, n_threads = blockDim.x;
  const int BV = n_threads / kSub, local = tid / kSub, sub = tid % kSub;
  const int j = blockIdx.z * BV + local;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  if (n <= 0) return;
  const bool col = j < V;
  const size_t out_width = (size_t)heads * V;
  const int slot = seq_slot[s];
  if (slot < 0) {
    if (col && sub == 0)
      for (int i = 0; i < n; ++i) out[(size_t)(t0 + i) * out_width + (size_t)h * V + j] = 0.f;
    return;
  }
  const int groups = Dp / 16;        // 16-byte parts of a key row that a lane takes
  float S[R];
  float* st = state + (((size_t)slot * heads + h) * D) * V + j;
  const bool carried = seq_start[s] > 0;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = 4 * (sub + kSub * (r / 4)) + r % 4;
    S[r] = (d < D && col && carried) ? st[(size_t)d * V] : 0.f;
  }
  const float q_scale = RULE == kRuleGla ? rsqrtf((float)D) : 1.f;
  const int warp = tid >> 5, lane = tid & 31, n_warps = n_threads >> 5;

  for (int i0 = 0; i0 < n; i0 += stage) {
    const int ns = min(stage, n - i0);
    __syncthreads();      // the stage before has been walked by everyone
    for (int idx = tid; idx < ns * Dp; idx += n_threads) {
      const int i = idx / Dp, d = idx % Dp;
      float qv = 0.f, kv = 0.f, dv = 0.f, av = 0.f;
      if (d < D) {
        const size_t t = (size_t)(t0 + i0 + i);
        const T* row = proj + t * stride;
        const float zz = z[t * heads * D + (size_t)h * D + d];
        qv = to_float(row[q_col + h * D + d]) * q_scale;
        kv = to_float(row[k_col + h * D + d]);
        if (RULE == kRuleGla) {
          dv = expf(-softplus_f(-zz) * coef);
        } else {
          dv = expf(-coef * sigmoid_f(zz));
          av = sigmoid_f(to_float(row[a_col + h * D + d]) + a_bias[h * D + d]);
        }
      }
      qs[idx] = qv;
      ks[idx] = kv;
      ds[idx] = dv;
      if (RULE == kRuleDelta) as[idx] = av;
    }
    for (int idx = tid; idx < ns * BV; idx += n_threads) {
      const int i = idx / BV, c = blockIdx.z * BV + idx % BV;
      vs[idx] = c < V ? to_float(proj[(size_t)(t0 + i0 + i) * stride + v_col + h * V + c]) : 0.f;
    }
    __syncthreads();
    if (RULE == kRuleDelta) {     // unit keys: a warp a token
      for (int i = warp; i < ns; i += n_warps) {
        float ss = 0.f;
        for (int d = lane; d < Dp; d += 32) ss = fmaf(ks[i * Dp + d], ks[i * Dp + d], ss);
        const float inv = 1.0f / sqrtf(warp_sum(ss) + unit_eps);
        for (int d = lane; d < Dp; d += 32) {
          const float u = ks[i * Dp + d] * inv;
          us[i * Dp + d] = u;
          as[i * Dp + d] *= u;
        }
      }
      __syncthreads();
    }
    for (int i = 0; i < ns; ++i) {
      const float v = vs[i * BV + local];
      const float4* q4 = reinterpret_cast<const float4*>(qs + i * Dp) + sub;
      const float4* k4 = reinterpret_cast<const float4*>(ks + i * Dp) + sub;
      const float4* d4 = reinterpret_cast<const float4*>(ds + i * Dp) + sub;
      float o0 = 0.f, o1 = 0.f;
      if (RULE == kRuleGla) {
#pragma unroll
        for (int g = 0; g < R / 4; ++g)
          if (g < groups) {
            const float4 qq = q4[kSub * g], kk = k4[kSub * g], dd = d4[kSub * g];
            S[4 * g + 0] = fmaf(dd.x, S[4 * g + 0], kk.x * v);
            S[4 * g + 1] = fmaf(dd.y, S[4 * g + 1], kk.y * v);
            S[4 * g + 2] = fmaf(dd.z, S[4 * g + 2], kk.z * v);
            S[4 * g + 3] = fmaf(dd.w, S[4 * g + 3], kk.w * v);
            o0 = fmaf(S[4 * g + 0], qq.x, o0);
            o1 = fmaf(S[4 * g + 1], qq.y, o1);
            o0 = fmaf(S[4 * g + 2], qq.z, o0);
            o1 = fmaf(S[4 * g + 3], qq.w, o1);
          }
      } else {
        const float4* u4 = reinterpret_cast<const float4*>(us + i * Dp) + sub;
        const float4* a4 = reinterpret_cast<const float4*>(as + i * Dp) + sub;
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int g = 0; g < R / 4; ++g)
          if (g < groups) {
            const float4 uu = u4[kSub * g];
            p0 = fmaf(uu.x, S[4 * g + 0], p0);
            p1 = fmaf(uu.y, S[4 * g + 1], p1);
            p0 = fmaf(uu.z, S[4 * g + 2], p0);
            p1 = fmaf(uu.w, S[4 * g + 3], p1);
          }
        const float uS = sum_of_four(p0 + p1);
#pragma unroll
        for (int g = 0; g < R / 4; ++g)
          if (g < groups) {
            const float4 qq = q4[kSub * g], kk = k4[kSub * g], dd = d4[kSub * g], aa = a4[kSub * g];
            S[4 * g + 0] = fmaf(dd.x, S[4 * g + 0], fmaf(-aa.x, uS, kk.x * v));
            S[4 * g + 1] = fmaf(dd.y, S[4 * g + 1], fmaf(-aa.y, uS, kk.y * v));
            S[4 * g + 2] = fmaf(dd.z, S[4 * g + 2], fmaf(-aa.z, uS, kk.z * v));
            S[4 * g + 3] = fmaf(dd.w, S[4 * g + 3], fmaf(-aa.w, uS, kk.w * v));
            o0 = fmaf(S[4 * g + 0], qq.x, o0);
            o1 = fmaf(S[4 * g + 1], qq.y, o1);
            o0 = fmaf(S[4 * g + 2], qq.z, o0);
            o1 = fmaf(S[4 * g + 3], qq.w, o1);
          }
      }
      const float o = sum_of_four(o0 + o1);
      if (col && sub == 0) out[(size_t)(t0 + i0 + i) * out_width + (size_t)h * V + j] = o;
    }
  }
  if (col) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = 4 * (sub + kSub * (r / 4)) + r % 4;
      if (d < D) st[(size_t)d * V] = S[r];
    }
  }
}

template <typename T, int RULE>
int launch_recurrence(const void* proj, long long stride, int q_col, int k_col, int v_col, int a_col, const float* a_bias,
                      const float* z, float coef, float unit_eps, float* state, float* out, const int* seq_slot,
                      const int* seq_start, const int* cu_new, int n_seqs, int heads, int D, int V, cudaStream_t stream,
                      const char* name) {
  const int BV = V <= 8 ? 8 : V <= 16 ? 16 : V <= 32 ? 32 : kColumns;      // (a block is whole warps: 8 columns x 4 lanes)
  const int Dp = (D + 15) / 16 * 16;
  const int n_arrays = RULE == kRuleDelta ? 5 : 3;
  const int per_token = (n_arrays * Dp + BV) * (int)sizeof(float);
  const int stage = max(1, min(16, kStageBytes / per_token));
  const size_t smem = (size_t)stage * per_token;
  const dim3 grid(n_seqs, heads, (V + BV - 1) / BV);
  cudaError_t e;
#define EMBER_RECURRENCE(R)                                                                                                  \
  e = launch_plain(recurrence_kernel<T, RULE, R>, grid, dim3(BV * kSub), smem, stream, (const T*)proj, stride, q_col, k_col, \
                   v_col, a_col, a_bias, z, coef, unit_eps, state, out, seq_slot, seq_start, cu_new, heads, D, V, Dp, stage)
  if (Dp <= 16) EMBER_RECURRENCE(4);
  else if (Dp <= 32) EMBER_RECURRENCE(8);
  else if (Dp <= 64) EMBER_RECURRENCE(16);
  else if (Dp <= 128) EMBER_RECURRENCE(32);
  else EMBER_RECURRENCE(64);
#undef EMBER_RECURRENCE
  if (e != cudaSuccess) return ember_fail("%s: %s", name, cudaGetErrorString(e));
  return 0;
}

// grid (T): lr = `rank` columns from `col` of a row of `in`
template <typename T>
__global__ void __launch_bounds__(128)
low_rank_out_kernel(const T* __restrict__ in, long long stride, int col, int rank, const float* __restrict__ w2,
                    const float* __restrict__ bias, float* __restrict__ out, int n_out, int act) {
  __shared__ float lr[256];
  const int t = blockIdx.x;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    const float v = to_float(in[(size_t)t * stride + col + r]);
    lr[r] = act ? tanhf(v) : v;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < n_out; c += blockDim.x) {
    const float* w = w2 + (size_t)c * rank;
    float acc = 0.f;
    for (int r = 0; r < rank; ++r) acc = fmaf(lr[r], w[r], acc);
    out[(size_t)t * n_out + c] = acc + bias[c];
  }
}

}  // namespace

// in [T, *] (dtype, row stride in elements), w2 float32 [n_out, rank], bias float32 [n_out], out float32 [T, n_out];
// act: 0 none, 1 tanh on the low-rank values.
EMBER_API int ember_low_rank_out(const void* in, long long stride, int col, int rank, const float* w2, const float* bias,
                                 float* out, int T, int n_out, int act, int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_out > 0 && rank >= 1 && rank <= 256, "low_rank_out: %d rows, %d outputs, rank %d (at most 256)", T, n_out, rank);
  EMBER_CHECK(act == 0 || act == 1, "low_rank_out: activation %d", act);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(low_rank_out_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)in, stride, col, rank, w2, bias, out, n_out, act);
  else if (dtype == EMBER_BF16)
    e = launch_plain(low_rank_out_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)in, stride, col, rank, w2,
                     bias, out, n_out, act);
  else
    return ember_fail("low_rank_out: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("low_rank_out: %s", cudaGetErrorString(e));
  return 0;
}

// proj [T, *] (dtype): q, k of heads x dim from q_col, k_col, v of heads x vdim from v_col; z float32 [T, heads * dim];
// state float32 [slots, heads, dim, vdim]; out float32 [T, heads * vdim].
EMBER_API int ember_gla_scan(const void* proj, long long stride, int q_col, int k_col, int v_col, const float* z, float tau,
                             float* state, float* out, const int* seq_slot, const int* seq_start, const int* cu_new,
                             int n_seqs, int heads, int dim, int vdim, int dtype, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && heads <= 65535 && dim >= 1 && dim <= 256 && vdim >= 1,
              "gla_scan: %d sequences, %d heads of %d x %d (key size at most 256)", n_seqs, heads, dim, vdim);
  EMBER_CHECK(tau > 0.f, "gla_scan: tau %g", (double)tau);
  if (dtype == EMBER_F32)
    return launch_recurrence<float, kRuleGla>(proj, stride, q_col, k_col, v_col, 0, nullptr, z, 1.0f / tau, 0.f, state, out,
                                              seq_slot, seq_start, cu_new, n_seqs, heads, dim, vdim, stream, "gla_scan");
  if (dtype == EMBER_BF16)
    return launch_recurrence<__nv_bfloat16, kRuleGla>(proj, stride, q_col, k_col, v_col, 0, nullptr, z, 1.0f / tau, 0.f, state,
                                                      out, seq_slot, seq_start, cu_new, n_seqs, heads, dim, vdim, stream,
                                                      "gla_scan");
  return ember_fail("gla_scan: element type %d", dtype);
}

// proj [T, *] (dtype): r, k, v, a_in of heads x dim from their columns; a_bias float32 [heads * dim]; z float32
// [T, heads * dim] (the decay's logits); state float32 [slots, heads, dim, dim]; out float32 [T, heads * dim].
EMBER_API int ember_generalized_delta_rule(const void* proj, long long stride, int r_col, int k_col, int v_col, int a_col,
                                           const float* a_bias, const float* z, float decay_coef, float unit_eps,
                                           float* state, float* out, const int* seq_slot, const int* seq_start,
                                           const int* cu_new, int n_seqs, int heads, int dim, int dtype,
                                           cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && heads <= 65535 && dim >= 1 && dim <= 256,
              "generalized_delta_rule: %d sequences, %d heads of %d (at most 256)", n_seqs, heads, dim);
  if (dtype == EMBER_F32)
    return launch_recurrence<float, kRuleDelta>(proj, stride, r_col, k_col, v_col, a_col, a_bias, z, decay_coef, unit_eps,
                                                state, out, seq_slot, seq_start, cu_new, n_seqs, heads, dim, dim, stream,
                                                "generalized_delta_rule");
  if (dtype == EMBER_BF16)
    return launch_recurrence<__nv_bfloat16, kRuleDelta>(proj, stride, r_col, k_col, v_col, a_col, a_bias, z, decay_coef,
                                                        unit_eps, state, out, seq_slot, seq_start, cu_new, n_seqs, heads,
                                                        dim, dim, stream, "generalized_delta_rule");
  return ember_fail("generalized_delta_rule: element type %d", dtype);
}
