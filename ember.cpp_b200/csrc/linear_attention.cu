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
// A block owns up to 64 value columns of one (sequence, head); a thread keeps its column of S in registers
// through all of the sequence's tokens of the step.  q, k, the decays (and the unit key and a * u) of a stage
// of tokens are made once in shared memory by all threads together, then every thread walks the stage's
// tokens reading them as broadcasts.  A token's arithmetic does not depend on where a stage or a step begins,
// so a sequence's outputs are the same bits however it is cut into steps.  A sequence that starts at position
// 0 starts from zeros whatever its state rows hold; padding sequences (slot -1) are skipped.
#include "common.cuh"

namespace {

constexpr int kColumns = 64;       // value columns (threads) a block, at most
constexpr int kStageBytes = 40 * 1024;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

enum : int { kRuleGla = 0, kRuleDelta = 1 };

template <typename T, int RULE, int DMAX>
__global__ void __launch_bounds__(kColumns)
recurrence_kernel(const T* __restrict__ proj, long long stride, int q_col, int k_col, int v_col, int a_col,
                  const float* __restrict__ a_bias, const float* __restrict__ z, float coef, float unit_eps,
                  float* __restrict__ state, float* __restrict__ out, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int D, int V, int stage) {
  extern __shared__ float sm[];
  const int n_arrays = RULE == kRuleDelta ? 5 : 3;
  float* qs = sm;                    // [stage][D]
  float* ks = qs + stage * D;
  float* ds = ks + stage * D;        // the decay of every key channel
  float* us = ds + stage * D;        // the unit key (delta rule)
  float* as = us + stage * D;        // rate, then rate * unit key
  float* vs = sm + n_arrays * stage * D;   // [stage][blockDim.x]
  const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, BV = blockDim.x;
  const int j = blockIdx.z * BV + tid;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  if (n <= 0) return;
  const bool col = j < V;
  const size_t out_width = (size_t)heads * V;
  const int slot = seq_slot[s];
  if (slot < 0) {
    if (col)
      for (int i = 0; i < n; ++i) out[(size_t)(t0 + i) * out_width + (size_t)h * V + j] = 0.f;
    return;
  }
  float S[DMAX];
  float* st = state + (((size_t)slot * heads + h) * D) * V + j;
  const bool carried = seq_start[s] > 0;
#pragma unroll
  for (int d = 0; d < DMAX; ++d) S[d] = (d < D && col && carried) ? st[(size_t)d * V] : 0.f;
  const float q_scale = RULE == kRuleGla ? rsqrtf((float)D) : 1.f;
  const int warp = tid >> 5, lane = tid & 31, n_warps = BV >> 5;

  for (int i0 = 0; i0 < n; i0 += stage) {
    const int ns = min(stage, n - i0);
    __syncthreads();      // the stage before has been walked by everyone
    for (int idx = tid; idx < ns * D; idx += BV) {
      const int i = idx / D, d = idx % D;
      const size_t t = (size_t)(t0 + i0 + i);
      const T* row = proj + t * stride;
      const float zz = z[t * heads * D + (size_t)h * D + d];
      qs[idx] = to_float(row[q_col + h * D + d]) * q_scale;
      ks[idx] = to_float(row[k_col + h * D + d]);
      if (RULE == kRuleGla) {
        ds[idx] = expf(-softplus_f(-zz) * coef);
      } else {
        ds[idx] = expf(-coef * sigmoid_f(zz));
        as[idx] = sigmoid_f(to_float(row[a_col + h * D + d]) + a_bias[h * D + d]);
      }
    }
    for (int idx = tid; idx < ns * BV; idx += BV) {
      const int i = idx / BV, c = blockIdx.z * BV + idx % BV;
      vs[idx] = c < V ? to_float(proj[(size_t)(t0 + i0 + i) * stride + v_col + h * V + c]) : 0.f;
    }
    __syncthreads();
    if (RULE == kRuleDelta) {     // unit keys: a warp a token
      for (int i = warp; i < ns; i += n_warps) {
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(ks[i * D + d], ks[i * D + d], ss);
        const float inv = 1.0f / sqrtf(warp_sum(ss) + unit_eps);
        for (int d = lane; d < D; d += 32) {
          const float u = ks[i * D + d] * inv;
          us[i * D + d] = u;
          as[i * D + d] *= u;
        }
      }
      __syncthreads();
    }
    for (int i = 0; i < ns; ++i) {
      const float v = vs[i * BV + tid];
      const float* q_ = qs + i * D;
      const float* k_ = ks + i * D;
      const float* d_ = ds + i * D;
      float o = 0.f;
      if (RULE == kRuleGla) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
          if (d < D) {
            S[d] = fmaf(d_[d], S[d], k_[d] * v);
            o = fmaf(S[d], q_[d], o);
          }
      } else {
        const float* u_ = us + i * D;
        const float* a_ = as + i * D;
        float uS = 0.f;
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
          if (d < D) uS = fmaf(u_[d], S[d], uS);
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
          if (d < D) {
            S[d] = fmaf(d_[d], S[d], fmaf(-a_[d], uS, k_[d] * v));
            o = fmaf(S[d], q_[d], o);
          }
      }
      if (col) out[(size_t)(t0 + i0 + i) * out_width + (size_t)h * V + j] = o;
    }
  }
  if (col) {
#pragma unroll
    for (int d = 0; d < DMAX; ++d)
      if (d < D) st[(size_t)d * V] = S[d];
  }
}

template <typename T, int RULE>
int launch_recurrence(const void* proj, long long stride, int q_col, int k_col, int v_col, int a_col, const float* a_bias,
                      const float* z, float coef, float unit_eps, float* state, float* out, const int* seq_slot,
                      const int* seq_start, const int* cu_new, int n_seqs, int heads, int D, int V, cudaStream_t stream,
                      const char* name) {
  const int BV = V <= 32 ? 32 : kColumns;
  const int n_arrays = RULE == kRuleDelta ? 5 : 3;
  const int per_token = (n_arrays * D + BV) * (int)sizeof(float);
  const int stage = max(1, min(16, kStageBytes / per_token));
  const size_t smem = (size_t)stage * per_token;
  const dim3 grid(n_seqs, heads, (V + BV - 1) / BV);
  cudaError_t e;
#define EMBER_RECURRENCE(DMAX)                                                                                           \
  e = launch_plain(recurrence_kernel<T, RULE, DMAX>, grid, dim3(BV), smem, stream, (const T*)proj, stride, q_col, k_col, \
                   v_col, a_col, a_bias, z, coef, unit_eps, state, out, seq_slot, seq_start, cu_new, heads, D, V, stage)
  if (D <= 32) EMBER_RECURRENCE(32);
  else if (D <= 64) EMBER_RECURRENCE(64);
  else if (D <= 128) EMBER_RECURRENCE(128);
  else EMBER_RECURRENCE(256);
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
