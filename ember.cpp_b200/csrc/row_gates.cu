// Row kernels around mixers whose branches are normed one by one: the sum of branches with a gain per
// channel, the norms of q, k and v in front of an attention, and a gate on an attention's output.
//
// Everything is float32 arithmetic on rows whatever the element types that go in or come out.  A row is
// summed by one block (or one warp) in an order that depends on its length alone, so a row's result does
// not depend on the batch it is in.  Ordinary launches, as in norm_gate.cu.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxBranches = 8;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += red[i];
  return total;
}

__device__ __forceinline__ float sigmoidf(float v) { return 1.0f / (1.0f + expf(-v)); }

struct Branches {
  const float* rows[kMaxBranches];
  long long stride[kMaxBranches];
  float factor[kMaxBranches];
  const float* norm[kMaxBranches];   // the branch's own gain: it is divided by its root mean square first; null: taken as it is
  int n;
};

// x += gain * sum_k factor_k * b_k, where b_k = rows_k / rms(rows_k) * norm_k for a branch with a gain of its own
// and rows_k otherwise; gain null: 1.  One block a row; the branches' statistics first, then one pass over the row.
__global__ void __launch_bounds__(kThreads)
add_branches_kernel(float* __restrict__ x, const Branches b, const float* __restrict__ gain, int d, float eps) {
  __shared__ float red[kThreads / 32];
  const size_t row = blockIdx.x;
  float inv[kMaxBranches];
#pragma unroll
  for (int k = 0; k < kMaxBranches; ++k) {
    inv[k] = 1.f;
    if (k < b.n && b.norm[k]) {
      const float* r = b.rows[k] + row * b.stride[k];
      float ss = 0.f;
      for (int i = threadIdx.x; i < d; i += kThreads) ss = fmaf(r[i], r[i], ss);
      inv[k] = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    }
  }
  float* o = x + row * d;
  for (int i = threadIdx.x; i < d; i += kThreads) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxBranches; ++k)
      if (k < b.n) {
        const float v = b.rows[k][row * b.stride[k] + i];
        s = fmaf(b.factor[k], b.norm[k] ? v * inv[k] * b.norm[k][i] : v, s);
      }
    o[i] += gain ? gain[i] * s : s;
  }
}

// One block a token.  q | k | v are columns of a wider row (`in`, row stride in_stride, q at column 0).
//   q <- q / rms(q over all its heads) * q_gain (q_gain null: q as it is), then times the temperature
//        1 + coef * ln(floor((p + 1) / every) + 1) of the token's position p (coef 0: none)
//   k <- k / rms(k over all its heads) * k_gain (null: as it is)
//   v <- every head divided by its own root mean square (unit_v 0: as it is)
// out: q | k | v packed, in the output's element type.
template <typename TIN, typename TOUT>
__global__ void __launch_bounds__(kThreads)
qkv_norm_kernel(const TIN* __restrict__ in, long long in_stride, TOUT* __restrict__ out, const int* __restrict__ positions,
                const float* __restrict__ q_gain, const float* __restrict__ k_gain, int q_width, int k_width, int kv_heads,
                int vd, int unit_v, float eps, float coef, int every) {
  __shared__ float red[kThreads / 32];
  const size_t t = blockIdx.x;
  const TIN* row = in + t * in_stride;
  TOUT* o = out + t * (size_t)(q_width + k_width + kv_heads * vd);
  float q_mul = 1.f;
  if (coef != 0.f) q_mul = 1.0f + coef * logf((float)((positions[t] + 1) / every + 1));
  {
    float inv = 1.f;
    if (q_gain) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < q_width; i += kThreads) {
        const float v = to_float(row[i]);
        ss = fmaf(v, v, ss);
      }
      inv = 1.0f / sqrtf(block_sum(ss, red) / (float)q_width + eps);
    }
    for (int i = threadIdx.x; i < q_width; i += kThreads) {
      const float v = to_float(row[i]);
      o[i] = from_float<TOUT>((q_gain ? v * inv * q_gain[i] : v) * q_mul);
    }
  }
  {
    const TIN* k = row + q_width;
    float inv = 1.f;
    if (k_gain) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < k_width; i += kThreads) {
        const float v = to_float(k[i]);
        ss = fmaf(v, v, ss);
      }
      inv = 1.0f / sqrtf(block_sum(ss, red) / (float)k_width + eps);
    }
    for (int i = threadIdx.x; i < k_width; i += kThreads) {
      const float v = to_float(k[i]);
      o[q_width + i] = from_float<TOUT>(k_gain ? v * inv * k_gain[i] : v);
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int h = warp; h < kv_heads; h += kThreads / 32) {
    const TIN* v = row + q_width + k_width + (size_t)h * vd;
    float inv = 1.f;
    if (unit_v) {
      float ss = 0.f;
      for (int i = lane; i < vd; i += 32) {
        const float a = to_float(v[i]);
        ss = fmaf(a, a, ss);
      }
      inv = 1.0f / sqrtf(warp_sum(ss) / (float)vd + eps);
    }
    for (int i = lane; i < vd; i += 32) o[q_width + k_width + (size_t)h * vd + i] = from_float<TOUT>(to_float(v[i]) * inv);
  }
}

// out = a * gate(z): kind 0 silu, 1 sigmoid.  z: n columns of a wider matrix.
template <typename TA, typename TZ>
__global__ void gate_mul_kernel(const TA* __restrict__ a, const TZ* __restrict__ z, long long z_stride, TA* __restrict__ out,
                                size_t total, int n, int kind) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / n;
    const int c = (int)(i % n);
    const float g = to_float(z[row * z_stride + c]);
    out[i] = from_float<TA>(to_float(a[i]) * (kind == 1 ? sigmoidf(g) : g * sigmoidf(g)));
  }
}

}  // namespace

// rows[k], strides[k] (elements), factors[k], norms[k] (a float32 gain of d values, or null) for k < n_branches (host arrays)
EMBER_API int ember_add_branches(float* x, const void* const* rows, const long long* strides, const float* factors,
                                 const void* const* norms, int n_branches, const float* gain, int n_rows, int d, float eps,
                                 cudaStream_t stream) {
  EMBER_CHECK(n_rows > 0 && d > 0, "add_branches: %d rows of %d", n_rows, d);
  EMBER_CHECK(n_branches >= 1 && n_branches <= kMaxBranches, "add_branches: %d branches (1 to %d)", n_branches, kMaxBranches);
  Branches b;
  b.n = n_branches;
  for (int k = 0; k < kMaxBranches; ++k) {
    b.rows[k] = k < n_branches ? (const float*)rows[k] : nullptr;
    b.stride[k] = k < n_branches ? strides[k] : 0;
    b.factor[k] = k < n_branches ? factors[k] : 0.f;
    b.norm[k] = k < n_branches ? (const float*)norms[k] : nullptr;
  }
  const cudaError_t e = launch_plain(add_branches_kernel, dim3(n_rows), dim3(kThreads), 0, stream, x, b, gain, d, eps);
  if (e != cudaSuccess) return ember_fail("add_branches: %s", cudaGetErrorString(e));
  return 0;
}

EMBER_API int ember_qkv_norm(const void* in, long long in_stride, void* out, const int* positions, const float* q_gain,
                             const float* k_gain, int T, int q_width, int k_width, int kv_heads, int vd, int unit_v, float eps,
                             float coef, int every, int in_dtype, int out_dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && q_width > 0 && k_width > 0 && kv_heads > 0 && vd > 0, "qkv_norm: bad sizes");
  EMBER_CHECK(in_stride >= (long long)q_width + k_width + (long long)kv_heads * vd, "qkv_norm: rows of %lld values are too short",
              in_stride);
  EMBER_CHECK(coef == 0.f || every > 0, "qkv_norm: a temperature that grows every %d positions", every);
  cudaError_t e;
#define EMBER_QKV(TIN, TOUT)                                                                                                   \
  launch_plain(qkv_norm_kernel<TIN, TOUT>, dim3(T), dim3(kThreads), 0, stream, (const TIN*)in, in_stride, (TOUT*)out, positions, \
               q_gain, k_gain, q_width, k_width, kv_heads, vd, unit_v, eps, coef, every)
  if (in_dtype == EMBER_F32 && out_dtype == EMBER_F32) e = EMBER_QKV(float, float);
  else if (in_dtype == EMBER_F32 && out_dtype == EMBER_BF16) e = EMBER_QKV(float, __nv_bfloat16);
  else if (in_dtype == EMBER_BF16 && out_dtype == EMBER_BF16) e = EMBER_QKV(__nv_bfloat16, __nv_bfloat16);
  else return ember_fail("qkv_norm: element types %d -> %d", in_dtype, out_dtype);
#undef EMBER_QKV
  if (e != cudaSuccess) return ember_fail("qkv_norm: %s", cudaGetErrorString(e));
  return 0;
}

EMBER_API int ember_gate_mul(const void* a, const void* z, long long z_stride, void* out, int rows, int n, int kind, int a_dtype,
                             int z_dtype, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && n > 0 && (kind == 0 || kind == 1) && z_stride >= n, "gate_mul: %d rows of %d, kind %d", rows, n, kind);
  const size_t total = (size_t)rows * n;
  const int grid = (int)((total + 255) / 256 < 65535 * 16 ? (total + 255) / 256 : 65535 * 16);
  cudaError_t e;
#define EMBER_GM(TA, TZ) \
  launch_plain(gate_mul_kernel<TA, TZ>, dim3(grid), dim3(256), 0, stream, (const TA*)a, (const TZ*)z, z_stride, (TA*)out, total, n, kind)
  if (a_dtype == EMBER_F32 && z_dtype == EMBER_F32) e = EMBER_GM(float, float);
  else if (a_dtype == EMBER_BF16 && z_dtype == EMBER_F32) e = EMBER_GM(__nv_bfloat16, float);
  else if (a_dtype == EMBER_BF16 && z_dtype == EMBER_BF16) e = EMBER_GM(__nv_bfloat16, __nv_bfloat16);
  else return ember_fail("gate_mul: element types %d and %d", a_dtype, z_dtype);
#undef EMBER_GM
  if (e != cudaSuccess) return ember_fail("gate_mul: %s", cudaGetErrorString(e));
  return 0;
}
