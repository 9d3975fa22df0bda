// Two small things a layer does with rows of neighbouring tokens and with the token ids:
//
//   token_shift   out[t] = h[t] + (h[t-1] - h[t]) * mu, the row before a sequence's first token of the step being
//                 the slot's carried row (zeros at position 0); the slot then carries the sequence's last row of
//                 the step.  The block of a sequence's first token does both: it reads the carried row and, having
//                 read it, writes the new one, so no other block touches the slot's row.
//   side_input    x[t] += unit_rms(W_proj (gelu_tanh(W_gate x[t]) * e[t])) * w, e[t] = `dim` columns from `col` of
//                 the token's row of a table; one block a token, float32 arithmetic, sums in a fixed order.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += red[w];
  return total;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
token_shift_kernel(const T* __restrict__ h, T* __restrict__ out, const float* __restrict__ mu, float* __restrict__ state,
                   const int* __restrict__ token_seq, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                   const int* __restrict__ cu_new, int width) {
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const int slot = seq_slot[s];
  const T* row = h + (size_t)t * width;
  T* o = out + (size_t)t * width;
  if (slot < 0) {
    for (int c = threadIdx.x; c < width; c += kThreads) o[c] = from_float<T>(0.f);
    return;
  }
  const int first = cu_new[s], last = cu_new[s + 1] - 1;
  if (t != first) {
    const T* before = row - width;
    for (int c = threadIdx.x; c < width; c += kThreads) {
      const float v = to_float(row[c]);
      o[c] = from_float<T>(fmaf(to_float(before[c]) - v, mu[c], v));
    }
    return;
  }
  const bool carried = seq_start[s] > 0;
  float* st = state + (size_t)slot * width;
  const T* newest = h + (size_t)last * width;
  for (int c = threadIdx.x; c < width; c += kThreads) {
    const float v = to_float(row[c]);
    const float before = carried ? st[c] : 0.f;
    o[c] = from_float<T>(fmaf(before - v, mu[c], v));
    st[c] = to_float(newest[c]);
  }
}

// dynamic shared memory: width + dim floats
template <typename T>
__global__ void __launch_bounds__(kThreads)
side_input_kernel(const float* __restrict__ x, float* __restrict__ out, const int* __restrict__ tokens,
                  const int* __restrict__ token_seq, const int* __restrict__ seq_slot, const T* __restrict__ table,
                  int vocab, int table_width, int col, int dim, const T* __restrict__ w_gate, const T* __restrict__ w_proj,
                  const float* __restrict__ w_norm, float eps, int width) {
  extern __shared__ float sm[];
  __shared__ float red[kThreads / 32];
  float* xs = sm;            // the token's row of the stream, then y
  float* g = sm + width;
  const int t = blockIdx.x;
  const float* row = x + (size_t)t * width;
  float* o = out + (size_t)t * width;
  if (seq_slot[token_seq[t]] < 0) {
    for (int c = threadIdx.x; c < width; c += kThreads) o[c] = row[c];
    return;
  }
  for (int c = threadIdx.x; c < width; c += kThreads) xs[c] = row[c];
  __syncthreads();
  const int tok = min(max(tokens[t], 0), vocab - 1);
  const T* e = table + (size_t)tok * table_width + col;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int d = warp; d < dim; d += kThreads / 32) {
    const T* w = w_gate + (size_t)d * width;
    float acc = 0.f;
    for (int c = lane; c < width; c += 32) acc = fmaf(to_float(w[c]), xs[c], acc);
    acc = warp_sum(acc);
    if (lane == 0) g[d] = gelu_tanh(acc) * to_float(e[d]);
  }
  __syncthreads();
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += kThreads) {
    const T* w = w_proj + (size_t)c * dim;
    float acc = 0.f;
    for (int d = 0; d < dim; ++d) acc = fmaf(to_float(w[d]), g[d], acc);
    xs[c] = acc;     // (a thread reads and writes its own columns only)
    ss = fmaf(acc, acc, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += kThreads) o[c] = row[c] + xs[c] * inv * w_norm[c];
}

}  // namespace

// h, out [T, width] (dtype); mu float32 [width]; state float32 [slots, width].
EMBER_API int ember_token_shift(const void* h, void* out, const float* mu, float* state, const int* token_seq,
                                const int* seq_slot, const int* seq_start, const int* cu_new, int T, int width, int dtype,
                                cudaStream_t stream) {
  EMBER_CHECK(T > 0 && width > 0 && state != nullptr, "token_shift: bad sizes");
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(token_shift_kernel<float>, dim3(T), dim3(kThreads), 0, stream, (const float*)h, (float*)out, mu, state,
                     token_seq, seq_slot, seq_start, cu_new, width);
  else if (dtype == EMBER_BF16)
    e = launch_plain(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(kThreads), 0, stream, (const __nv_bfloat16*)h,
                     (__nv_bfloat16*)out, mu, state, token_seq, seq_slot, seq_start, cu_new, width);
  else
    return ember_fail("token_shift: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("token_shift: %s", cudaGetErrorString(e));
  return 0;
}

// x, out float32 [T, width]; table [vocab, table_width], w_gate [dim, width], w_proj [width, dim] (dtype); w_norm float32 [width].
EMBER_API int ember_side_input(const float* x, float* out, const int* tokens, const int* token_seq, const int* seq_slot,
                               const void* table, int vocab, int table_width, int col, int dim, const void* w_gate,
                               const void* w_proj, const float* w_norm, float eps, int T, int width, int dtype,
                               cudaStream_t stream) {
  EMBER_CHECK(T > 0 && width > 0 && vocab > 0 && dim >= 1 && col >= 0 && col + dim <= table_width,
              "side_input: %d tokens, width %d, columns %d..%d of %d", T, width, col, col + dim, table_width);
  const size_t smem = (size_t)(width + dim) * sizeof(float);
  EMBER_CHECK(smem <= 48 * 1024, "side_input: width %d + %d values exceed a block's shared memory", width, dim);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(side_input_kernel<float>, dim3(T), dim3(kThreads), smem, stream, x, out, tokens, token_seq, seq_slot,
                     (const float*)table, vocab, table_width, col, dim, (const float*)w_gate, (const float*)w_proj, w_norm, eps, width);
  else if (dtype == EMBER_BF16)
    e = launch_plain(side_input_kernel<__nv_bfloat16>, dim3(T), dim3(kThreads), smem, stream, x, out, tokens, token_seq, seq_slot,
                     (const __nv_bfloat16*)table, vocab, table_width, col, dim, (const __nv_bfloat16*)w_gate,
                     (const __nv_bfloat16*)w_proj, w_norm, eps, width);
  else
    return ember_fail("side_input: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("side_input: %s", cudaGetErrorString(e));
  return 0;
}
