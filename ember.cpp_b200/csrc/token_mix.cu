// Two small things a layer does with rows of neighbouring tokens and with the token ids:
//
//   token_shift   out[t] = h[t] + (h[t-1] - h[t]) * mu, the row before a sequence's first token of the step being
//                 the slot's carried row (zeros at position 0); the slot then carries the sequence's last row of
//                 the step.  The block of a sequence's first token does both: it reads the carried row and, having
//                 read it, writes the new one, so no other block touches the slot's row.
//   cast_rows     rows of the float32 stream in the compute type (what a product reads)
//   table_gate    g[t, d] = z[t, d] * e[t, d], e[t] = `dim` columns from `col` of the token's row of a table: the
//                 per-layer input from the token ids, between its two products
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

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

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<T>(x[i]);
}

// grid (T)
template <typename T>
__global__ void table_gate_kernel(const T* __restrict__ z, T* __restrict__ out, const int* __restrict__ tokens,
                                  const T* __restrict__ table, int vocab, int table_width, int col, int dim) {
  const int t = blockIdx.x;
  const int tok = min(max(tokens[t], 0), vocab - 1);
  const T* e = table + (size_t)tok * table_width + col;
  for (int d = threadIdx.x; d < dim; d += blockDim.x)
    out[(size_t)t * dim + d] = from_float<T>(to_float(z[(size_t)t * dim + d]) * to_float(e[d]));
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

// x float32 [n], out [n] (dtype)
EMBER_API int ember_cast_rows(const float* x, void* out, size_t n, int dtype, cudaStream_t stream) {
  EMBER_CHECK(n > 0, "cast_rows: nothing to do");
  const unsigned grid = (unsigned)((n + 1023) / 1024 < 2048 ? (n + 1023) / 1024 : 2048);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(cast_rows_kernel<float>, dim3(grid), dim3(256), 0, stream, x, (float*)out, n);
  else if (dtype == EMBER_BF16)
    e = launch_plain(cast_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, x, (__nv_bfloat16*)out, n);
  else
    return ember_fail("cast_rows: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("cast_rows: %s", cudaGetErrorString(e));
  return 0;
}

// z, out [T, dim]; table [vocab, table_width] (all dtype); tokens int32 [T]
EMBER_API int ember_table_gate(const void* z, void* out, const int* tokens, const void* table, int vocab, int table_width,
                               int col, int dim, int T, int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && vocab > 0 && dim >= 1 && col >= 0 && col + dim <= table_width, "table_gate: %d tokens, columns %d..%d of %d",
              T, col, col + dim, table_width);
  const int threads = dim <= 32 ? 32 : dim <= 64 ? 64 : 128;
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(table_gate_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)z, (float*)out, tokens,
                     (const float*)table, vocab, table_width, col, dim);
  else if (dtype == EMBER_BF16)
    e = launch_plain(table_gate_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)z,
                     (__nv_bfloat16*)out, tokens, (const __nv_bfloat16*)table, vocab, table_width, col, dim);
  else
    return ember_fail("table_gate: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("table_gate: %s", cudaGetErrorString(e));
  return 0;
}
