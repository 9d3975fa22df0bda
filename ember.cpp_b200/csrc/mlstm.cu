// The matrix memory of the xLSTM (mLSTM) over a step's packed tokens.
//
// Per head, with a memory S of dim x vdim float32 values, a normaliser n of dim values and a running
// maximum m (all three start at zero) and, per token, a log input gate i_t and a log forget gate f_t:
//     m_t = max(f_t + m_(t-1), i_t)
//     S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        n_t likewise with k_t alone
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + floor)
// Everything here is float32 whatever the step's element type; q, k and v come in that type.
//
// `mlstm_gates` makes the two log gates of every token and head from the mixer's input: the products
// with the gates' own rows (float32 sums), the bias, the soft cap cap * tanh(. / cap), and for the forget
// gate the logarithm of the sigmoid.  `mlstm_scan` walks each sequence's tokens in order: a block = a run
// of value columns j of one (sequence, head), a thread a column with S[:, j] in registers, and one more
// warp that keeps n (a lane a few of its values) and makes the denominators; k, q and v of a few tokens
// are staged in shared memory at a time, and one thread walks the maxima of those tokens.  Every column
// is independent of the others, so a token's result depends on its sequence alone, never on the batch
// or the step's cut.  A sequence that starts at position 0 starts from zeros whatever its slot's state
// holds; sequences of slot -1 are padding: their rows are zero and no state is touched.
#include "common.cuh"

namespace {

__device__ __forceinline__ float log_sigmoid(float v) { return fminf(v, 0.f) - log1pf(expf(-fabsf(v))); }

// grid (T), 128 threads: a warp takes one gate row (2 * heads of them: input gates, then forget gates) at a time.
template <typename T>
__global__ void mlstm_gates_kernel(const T* __restrict__ h, const T* __restrict__ w, const float* __restrict__ bias,
                                   float* __restrict__ gates, int heads, int width, float cap) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const T* row = h + (size_t)t * width;
  for (int r = warp; r < 2 * heads; r += warps) {
    const T* wr = w + (size_t)r * width;
    float acc = 0.f;
    for (int d = lane; d < width; d += 32) acc = fmaf(to_float(row[d]), to_float(wr[d]), acc);
    acc = warp_sum(acc) + bias[r];
    const float capped = cap > 0.f ? cap * tanhf(acc / cap) : acc;
    if (lane == 0) gates[(size_t)t * 2 * heads + r] = r < heads ? capped : log_sigmoid(capped);
  }
}

constexpr int kStage = 16;   // tokens staged in shared memory at a time

// grid (sequences, heads, column tiles); blockDim.x = cols + 32: `cols` column threads and the normaliser's warp.
// DMAX >= dim, a multiple of 32: the column's registers.
template <typename T, int DMAX>
__global__ void mlstm_scan_kernel(const T* __restrict__ qkv, long long stride, int q_col, int k_col, int v_col,
                                  const float* __restrict__ gates, float* __restrict__ S_state, float* __restrict__ n_state,
                                  float* __restrict__ m_state, float* __restrict__ out, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int dim,
                                  int vdim, float floor_) {
  extern __shared__ float smem[];
  const int cols = blockDim.x - 32;
  float* ks = smem;                         // [kStage][DMAX]
  float* qs = ks + kStage * DMAX;           // [kStage][DMAX]
  float* vs = qs + kStage * DMAX;           // [kStage][cols]; the numerators afterwards
  float* keep = vs + kStage * cols;         // [kStage] exp(f + m_before - m)
  float* take = keep + kStage;              // [kStage] exp(i - m)
  float* den = take + kStage;               // [kStage] exp(-m), then the denominator
  const int s = blockIdx.x, h = blockIdx.y;
  const bool column = (int)threadIdx.x < cols;
  const int j = blockIdx.z * cols + threadIdx.x;
  const bool live = column && j < vdim;
  const int lane = threadIdx.x & 31;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const int slot = seq_slot[s];
  const int inner = heads * vdim;
  if (slot < 0) {
    if (live)
      for (int i = 0; i < n; ++i) out[(size_t)(t0 + i) * inner + (size_t)h * vdim + j] = 0.f;
    return;
  }
  const bool carried = seq_start[s] > 0;
  const float q_scale = rsqrtf((float)dim);
  float* col = S_state + ((size_t)slot * heads + h) * dim * vdim + j;
  float* nrow = n_state + ((size_t)slot * heads + h) * dim;
  float S[DMAX];              // a column thread: S[:, j]; a lane of the normaliser's warp: n[lane + 32 r] in S[r]
  if (column) {
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = (live && carried && d < dim) ? col[(size_t)d * vdim] : 0.f;
  } else {
#pragma unroll
    for (int r = 0; r < DMAX / 32; ++r) {
      const int d = lane + 32 * r;
      S[r] = (carried && d < dim) ? nrow[d] : 0.f;
    }
  }
  float m = carried ? m_state[(size_t)slot * heads + h] : 0.f;   // walked by the normaliser's first lane

  for (int c0 = 0; c0 < n; c0 += kStage) {
    const int cn = min(kStage, n - c0);
    __syncthreads();
    for (int e = threadIdx.x; e < cn * DMAX; e += blockDim.x) {
      const int i = e / DMAX, d = e % DMAX;
      const T* src = qkv + (size_t)(t0 + c0 + i) * stride + (size_t)h * dim + d;
      qs[e] = d < dim ? to_float(src[q_col]) * q_scale : 0.f;
      ks[e] = d < dim ? to_float(src[k_col]) : 0.f;
    }
    if (column)
      for (int i = 0; i < cn; ++i)
        vs[i * cols + threadIdx.x] = live ? to_float(qkv[(size_t)(t0 + c0 + i) * stride + v_col + (size_t)h * vdim + j]) : 0.f;
    if ((int)threadIdx.x == cols) {
      for (int i = 0; i < cn; ++i) {
        const float* g = gates + (size_t)(t0 + c0 + i) * 2 * heads;
        const float li = g[h], lf = g[heads + h];
        const float m_new = fmaxf(lf + m, li);
        keep[i] = expf(lf + m - m_new);
        take[i] = expf(li - m_new);
        den[i] = expf(-m_new);
        m = m_new;
      }
    }
    __syncthreads();
    if (column) {
      for (int i = 0; i < cn; ++i) {
        const float* k = ks + i * DMAX;
        const float* q = qs + i * DMAX;
        const float a = keep[i], b = take[i] * vs[i * cols + threadIdx.x];
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int d = 0; d < DMAX; d += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(k + d);
          const float4 qv = *reinterpret_cast<const float4*>(q + d);
          S[d] = fmaf(a, S[d], b * kv.x);
          S[d + 1] = fmaf(a, S[d + 1], b * kv.y);
          S[d + 2] = fmaf(a, S[d + 2], b * kv.z);
          S[d + 3] = fmaf(a, S[d + 3], b * kv.w);
          o0 = fmaf(S[d], qv.x, o0);
          o1 = fmaf(S[d + 1], qv.y, o1);
          o2 = fmaf(S[d + 2], qv.z, o2);
          o3 = fmaf(S[d + 3], qv.w, o3);
        }
        vs[i * cols + threadIdx.x] = (o0 + o1) + (o2 + o3);     // the numerator, in the place of the value it came from
      }
    } else {
      for (int i = 0; i < cn; ++i) {
        const float a = keep[i], b = take[i];
        float dot = 0.f;
#pragma unroll
        for (int r = 0; r < DMAX / 32; ++r) {
          const int d = lane + 32 * r;
          S[r] = fmaf(a, S[r], b * ks[i * DMAX + d]);
          dot = fmaf(S[r], qs[i * DMAX + d], dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) den[i] = fmaxf(fabsf(dot), den[i]) + floor_;
      }
    }
    __syncthreads();
    if (live)
      for (int i = 0; i < cn; ++i)
        out[(size_t)(t0 + c0 + i) * inner + (size_t)h * vdim + j] = vs[i * cols + threadIdx.x] / den[i];
  }
  if (live) {
#pragma unroll
    for (int d = 0; d < DMAX; ++d)
      if (d < dim) col[(size_t)d * vdim] = S[d];
  }
  if (!column && blockIdx.z == 0) {
#pragma unroll
    for (int r = 0; r < DMAX / 32; ++r) {
      const int d = lane + 32 * r;
      if (d < dim) nrow[d] = S[r];
    }
    if (lane == 0) m_state[(size_t)slot * heads + h] = m;
  }
}

template <typename T, int DMAX>
cudaError_t launch_scan(const void* qkv, long long stride, int q_col, int k_col, int v_col, const float* gates, float* S, float* n,
                        float* m, float* out, const int* seq_slot, const int* seq_start, const int* cu_new, int n_seqs, int heads,
                        int dim, int vdim, float floor_, cudaStream_t stream) {
  // columns a block: all of a head's where they are few, so that the normaliser is walked once
  const int cols = vdim <= 128 ? (vdim + 31) / 32 * 32 : 64;
  const int tiles = (vdim + cols - 1) / cols;
  const size_t smem = (size_t)(2 * kStage * DMAX + kStage * cols + 3 * kStage) * sizeof(float);
  auto kernel = mlstm_scan_kernel<T, DMAX>;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  return launch_plain(kernel, dim3(n_seqs, heads, tiles), dim3(cols + 32), smem, stream, (const T*)qkv, stride, q_col, k_col,
                      v_col, gates, S, n, m, out, seq_slot, seq_start, cu_new, heads, dim, vdim, floor_);
}

template <typename T>
cudaError_t launch_scan_any(int dim, const void* qkv, long long stride, int q_col, int k_col, int v_col, const float* gates, float* S,
                            float* n, float* m, float* out, const int* seq_slot, const int* seq_start, const int* cu_new,
                            int n_seqs, int heads, int vdim, float floor_, cudaStream_t stream) {
#define EMBER_SCAN(D) \
  launch_scan<T, D>(qkv, stride, q_col, k_col, v_col, gates, S, n, m, out, seq_slot, seq_start, cu_new, n_seqs, heads, dim, vdim, floor_, stream)
  if (dim <= 32) return EMBER_SCAN(32);
  if (dim <= 64) return EMBER_SCAN(64);
  if (dim <= 128) return EMBER_SCAN(128);
  return EMBER_SCAN(256);
#undef EMBER_SCAN
}

}  // namespace

// h [T, width] and w [2 * heads, width] in the step's element type, bias float32 [2 * heads]; gates float32 [T, 2 * heads]:
// the log input gates of the heads, then their log forget gates.  cap 0: no soft cap.
EMBER_API int ember_mlstm_gates(const void* h, const void* w, const float* bias, float* gates, int T, int heads, int width,
                                float cap, int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && heads > 0 && width > 0 && cap >= 0.f, "mlstm_gates: bad sizes");
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(mlstm_gates_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)h, (const float*)w, bias, gates, heads,
                     width, cap);
  else if (dtype == EMBER_BF16)
    e = launch_plain(mlstm_gates_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)h,
                     (const __nv_bfloat16*)w, bias, gates, heads, width, cap);
  else
    return ember_fail("mlstm_gates: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("mlstm_gates: %s", cudaGetErrorString(e));
  return 0;
}

// qkv: rows of `stride` values holding q (heads x dim) from q_col, k from k_col, v (heads x vdim) from v_col; gates as
// ember_mlstm_gates leaves them; S [slots, heads, dim, vdim], n [slots, heads, dim], m [slots, heads] float32 (advanced);
// out float32 [T, heads * vdim].
EMBER_API int ember_mlstm_scan(const void* qkv, long long stride, int q_col, int k_col, int v_col, const float* gates, float* S,
                               float* n, float* m, float* out, const int* seq_slot, const int* seq_start, const int* cu_new,
                               int n_seqs, int heads, int dim, int vdim, float floor_, int dtype, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && vdim > 0, "mlstm_scan: bad sizes");
  EMBER_CHECK(dim >= 1 && dim <= 256, "mlstm_scan: a key size of %d is not in [1, 256]", dim);
  EMBER_CHECK(heads <= 65535, "mlstm_scan: %d heads exceed one launch", heads);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_scan_any<float>(dim, qkv, stride, q_col, k_col, v_col, gates, S, n, m, out, seq_slot, seq_start, cu_new, n_seqs,
                               heads, vdim, floor_, stream);
  else if (dtype == EMBER_BF16)
    e = launch_scan_any<__nv_bfloat16>(dim, qkv, stride, q_col, k_col, v_col, gates, S, n, m, out, seq_slot, seq_start, cu_new,
                                       n_seqs, heads, vdim, floor_, stream);
  else
    return ember_fail("mlstm_scan: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("mlstm_scan: %s", cudaGetErrorString(e));
  return 0;
}
