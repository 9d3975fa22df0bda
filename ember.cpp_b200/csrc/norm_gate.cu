// RMS norm, the norm of a weighted sum added to the stream, and the gates of the gated layers.
//
// Everything here is float32 arithmetic on rows: statistics, sums and products are float32 whatever
// the element type of the rows that go in or come out.  A row is summed by one block in an order
// that depends on its length alone, so a row's result does not depend on the batch it is in.  The kernels are
// launched the ordinary way.  Programmatic dependent launch was tried for all the small kernels of this file, of
// ssm.cu, moe.cu and attention_decode_kept.cu and lost: a one-token step of four layers took 0.757 ms with ordinary
// launches, 0.865 ms with every kernel waiting for the one in front and releasing its follower at once, and 0.903 ms
// with the wait alone.  Several of these kernels run in more than one wave of blocks, and blocks that sit on the SMs
// waiting take the room of the waves that should run.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxBranches = 16;

// Sum over the block; every thread gets it, added in warp order.
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

// Four float32 values as T: one 16-byte (float) or 8-byte (bfloat16) store.
__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<const unsigned*>(&lo);
  v.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(dst) = v;
}
__device__ __forceinline__ float4 load4(const float* src) { return *reinterpret_cast<const float4*>(src); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* src) {
  const uint2 v = *reinterpret_cast<const uint2*>(src);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// out = x / sqrt(mean(x^2) + eps) * (offset + w).  VEC (d a multiple of 4): four values a thread and trip.
template <typename TOUT, bool VEC>
__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TOUT* __restrict__ out, int d, float eps,
               float offset) {
  __shared__ float red[kThreads / 32];
  const float* row = x + (size_t)blockIdx.x * d;
  TOUT* o = out + (size_t)blockIdx.x * d;
  float ss = 0.f;
  if constexpr (VEC) {
    for (int i = threadIdx.x * 4; i < d; i += kThreads * 4) {
      const float4 v = load4(row + i);
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    for (int i = threadIdx.x * 4; i < d; i += kThreads * 4) {
      const float4 v = load4(row + i), g = load4(w + i);
      store4(o + i, v.x * inv * (offset + g.x), v.y * inv * (offset + g.y), v.z * inv * (offset + g.z), v.w * inv * (offset + g.w));
    }
  } else {
    for (int i = threadIdx.x; i < d; i += kThreads) {
      const float v = row[i];
      ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += kThreads) o[i] = from_float<TOUT>(row[i] * inv * (offset + w[i]));
  }
}

struct Branches {
  const float* rows[kMaxBranches];
  long long stride[kMaxBranches];  // elements between two rows
  float factor[kMaxBranches];
  int n;
};

__device__ __forceinline__ float weighted(const Branches& b, size_t row, int i) {
  float s = 0.f;
  for (int k = 0; k < b.n; ++k) s = fmaf(b.factor[k], b.rows[k][row * (size_t)b.stride[k] + i], s);
  return s;
}
__device__ __forceinline__ float4 weighted4(const Branches& b, size_t row, int i) {
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < b.n; ++k) {
    const float4 v = load4(b.rows[k] + row * (size_t)b.stride[k] + i);
    const float f = b.factor[k];
    s.x = fmaf(f, v.x, s.x), s.y = fmaf(f, v.y, s.y), s.z = fmaf(f, v.z, s.z), s.w = fmaf(f, v.w, s.w);
  }
  return s;
}

// x += norm(sum_k factor_k * rows_k): the sum is made twice (once for the statistics, once for the
// result) in the same order, so nothing is kept between the passes.  VEC: the width and every branch's row
// stride are multiples of 4 and every pointer lies on 16 bytes: four values a thread and trip.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
add_normed_kernel(float* __restrict__ x, const Branches b, const float* __restrict__ w, int d, float eps, float offset) {
  __shared__ float red[kThreads / 32];
  const size_t row = blockIdx.x;
  float* o = x + row * d;
  float ss = 0.f;
  if constexpr (VEC) {
    for (int i = threadIdx.x * 4; i < d; i += kThreads * 4) {
      const float4 v = weighted4(b, row, i);
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    for (int i = threadIdx.x * 4; i < d; i += kThreads * 4) {
      const float4 v = weighted4(b, row, i), g = load4(w + i), r = load4(o + i);
      store4(o + i, r.x + v.x * inv * (offset + g.x), r.y + v.y * inv * (offset + g.y), r.z + v.z * inv * (offset + g.z),
             r.w + v.w * inv * (offset + g.w));
    }
  } else {
    for (int i = threadIdx.x; i < d; i += kThreads) {
      const float v = weighted(b, row, i);
      ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += kThreads) o[i] += weighted(b, row, i) * inv * (offset + w[i]);
  }
}

// rows of [gate | up] (n each) -> act(gate) * up
//   kind 0: g * sigmoid(g) * u
//   kind 1: g = min(g, limit), u = clamp(u, -limit, limit): g * sigmoid(alpha * g) * (u + shift)
__device__ __forceinline__ float gate_of(float g, float u, int kind, float limit, float alpha, float shift) {
  if (kind == 0) return g * sigmoidf(g) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoidf(alpha * g) * (u + shift);
}

// VEC (n a multiple of 4): four outputs a thread and trip.
template <typename T, bool VEC>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t total, int n, int kind,
                                 float limit, float alpha, float shift) {
  constexpr int W = VEC ? 4 : 1;
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += (size_t)gridDim.x * blockDim.x * W) {
    const size_t row = i / n;
    const int c = (int)(i % n);
    const T* src = gu + row * 2 * n + c;
    if constexpr (VEC) {
      const float4 g = load4(src), u = load4(src + n);
      store4(out + i, gate_of(g.x, u.x, kind, limit, alpha, shift), gate_of(g.y, u.y, kind, limit, alpha, shift),
             gate_of(g.z, u.z, kind, limit, alpha, shift), gate_of(g.w, u.w, kind, limit, alpha, shift));
    } else {
      out[i] = from_float<T>(gate_of(to_float(src[0]), to_float(src[n]), kind, limit, alpha, shift));
    }
  }
}

__device__ __forceinline__ float gatef(float z, int kind) { return kind == 1 ? sigmoidf(z) : z * sigmoidf(z); }

// out = unit(y * silu(z)) * w, the root mean square taken over each of `parts` equal pieces of a row.
// y float32 [T, n]; z: n columns of a wider matrix (row stride z_stride).  grid (T, parts).
// VEC: the part's width, the row widths and the gate's row stride are multiples of 4 (and the gate's first column too).
// GATE_FIRST false: out = unit(y) * w * silu(z), the root mean square being y's own (the gate comes after the norm).
// kind 1: the gate is sigmoid(z) in place of silu(z).
template <typename T, bool VEC, bool GATE_FIRST>
__global__ void __launch_bounds__(kThreads)
gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long z_stride,
                        const float* __restrict__ w, T* __restrict__ out, int n, int part, float eps, int kind) {
  __shared__ float red[kThreads / 32];
  const size_t t = blockIdx.x;
  const int c0 = blockIdx.y * part;
  const float* yr = y + t * n + c0;
  const T* zr = z + t * (size_t)z_stride + c0;
  T* o = out + t * n + c0;
  float ss = 0.f;
  if constexpr (VEC) {
    for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
      const float4 a = load4(yr + i), g = load4(zr + i);
      const float v0 = GATE_FIRST ? a.x * gatef(g.x, kind) : a.x, v1 = GATE_FIRST ? a.y * gatef(g.y, kind) : a.y,
                  v2 = GATE_FIRST ? a.z * gatef(g.z, kind) : a.z, v3 = GATE_FIRST ? a.w * gatef(g.w, kind) : a.w;
      ss = fmaf(v0, v0, fmaf(v1, v1, fmaf(v2, v2, fmaf(v3, v3, ss))));
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)part + eps);
    for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
      const float4 a = load4(yr + i), g = load4(zr + i), gain = load4(w + c0 + i);
      if constexpr (GATE_FIRST)
        store4(o + i, a.x * gatef(g.x, kind) * inv * gain.x, a.y * gatef(g.y, kind) * inv * gain.y,
               a.z * gatef(g.z, kind) * inv * gain.z, a.w * gatef(g.w, kind) * inv * gain.w);
      else
        store4(o + i, a.x * inv * gain.x * gatef(g.x, kind), a.y * inv * gain.y * gatef(g.y, kind),
               a.z * inv * gain.z * gatef(g.z, kind), a.w * inv * gain.w * gatef(g.w, kind));
    }
  } else {
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
      const float zv = to_float(zr[i]);
      const float v = GATE_FIRST ? yr[i] * gatef(zv, kind) : yr[i];
      ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
      const float zv = to_float(zr[i]);
      o[i] = from_float<T>(GATE_FIRST ? yr[i] * gatef(zv, kind) * inv * w[c0 + i] : yr[i] * inv * w[c0 + i] * gatef(zv, kind));
    }
  }
}

}  // namespace

EMBER_API int ember_rmsnorm(const float* x, const float* w, void* out, int rows, int d, float eps, float offset,
                            int out_dtype, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && d > 0, "rmsnorm: %d rows of %d", rows, d);
  cudaError_t e;
  if (out_dtype == EMBER_F32)
    e = d % 4 == 0 ? launch_plain(rmsnorm_kernel<float, true>, dim3(rows), dim3(kThreads), 0, stream, x, w, (float*)out, d, eps, offset)
                   : launch_plain(rmsnorm_kernel<float, false>, dim3(rows), dim3(kThreads), 0, stream, x, w, (float*)out, d, eps, offset);
  else if (out_dtype == EMBER_BF16)
    e = d % 4 == 0 ? launch_plain(rmsnorm_kernel<__nv_bfloat16, true>, dim3(rows), dim3(kThreads), 0, stream, x, w,
                                  (__nv_bfloat16*)out, d, eps, offset)
                   : launch_plain(rmsnorm_kernel<__nv_bfloat16, false>, dim3(rows), dim3(kThreads), 0, stream, x, w,
                                  (__nv_bfloat16*)out, d, eps, offset);
  else
    return ember_fail("rmsnorm: element type %d", out_dtype);
  if (e != cudaSuccess) return ember_fail("rmsnorm: %s", cudaGetErrorString(e));
  return 0;
}

// rows[k], strides[k] (elements), factors[k] for k < n_branches (host arrays)
EMBER_API int ember_add_normed(float* x, const void* const* rows, const long long* strides, const float* factors,
                               int n_branches, const float* w, int n_rows, int d, float eps, float offset,
                               cudaStream_t stream) {
  EMBER_CHECK(n_rows > 0 && d > 0, "add_normed: %d rows of %d", n_rows, d);
  EMBER_CHECK(n_branches >= 1 && n_branches <= kMaxBranches, "add_normed: %d branches (1 to %d)", n_branches, kMaxBranches);
  Branches b;
  b.n = n_branches;
  for (int k = 0; k < n_branches; ++k) {
    b.rows[k] = (const float*)rows[k];
    b.stride[k] = strides[k];
    b.factor[k] = factors[k];
  }
  bool vec = d % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0;
  for (int k = 0; k < n_branches; ++k) vec = vec && strides[k] % 4 == 0 && (uintptr_t)rows[k] % 16 == 0;
  const cudaError_t e = vec ? launch_plain(add_normed_kernel<true>, dim3(n_rows), dim3(kThreads), 0, stream, x, b, w, d, eps, offset)
                            : launch_plain(add_normed_kernel<false>, dim3(n_rows), dim3(kThreads), 0, stream, x, b, w, d, eps, offset);
  if (e != cudaSuccess) return ember_fail("add_normed: %s", cudaGetErrorString(e));
  return 0;
}

EMBER_API int ember_gated_act(const void* gu, void* out, int rows, int n, int kind, float limit, float alpha, float shift,
                              int dtype, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && n > 0 && (kind == 0 || kind == 1), "gated_act: %d rows of %d, kind %d", rows, n, kind);
  const size_t total = (size_t)rows * n;
  const bool vec = n % 4 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0;
  const size_t items = vec ? total / 4 : total;
  const int grid = (int)((items + 255) / 256 < 65535 * 16 ? (items + 255) / 256 : 65535 * 16);
  cudaError_t e;
#define EMBER_GATE(T, VEC) \
  launch_plain(gated_act_kernel<T, VEC>, dim3(grid), dim3(256), 0, stream, (const T*)gu, (T*)out, total, n, kind, limit, alpha, shift)
  if (dtype == EMBER_F32)
    e = vec ? EMBER_GATE(float, true) : EMBER_GATE(float, false);
  else if (dtype == EMBER_BF16)
    e = vec ? EMBER_GATE(__nv_bfloat16, true) : EMBER_GATE(__nv_bfloat16, false);
  else
    return ember_fail("gated_act: element type %d", dtype);
#undef EMBER_GATE
  if (e != cudaSuccess) return ember_fail("gated_act: %s", cudaGetErrorString(e));
  return 0;
}

EMBER_API int ember_gated_group_norm(const float* y, const void* z, long long z_stride, const float* w, void* out, int rows,
                                     int n, int parts, float eps, int gate_first, int dtype, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && n > 0 && parts > 0 && n % parts == 0, "gated_group_norm: %d rows of %d in %d parts", rows, n, parts);
  EMBER_CHECK(parts <= 65535, "gated_group_norm: %d parts exceed one launch", parts);
  const int kind = (gate_first >> 1) & 1;   // bit 0: the gate before the norm; bit 1: a sigmoid gate in place of silu
  const dim3 grid(rows, parts);
  const int elem = dtype == EMBER_F32 ? 4 : 2;
  // a part as short as a head takes a warp or two, not a block of eight that mostly idle
  const int per_pass = (n / parts + 3) / 4;
  const int threads = per_pass >= kThreads ? kThreads : (per_pass + 31) / 32 * 32;
  const bool vec = (n / parts) % 4 == 0 && n % 4 == 0 && z_stride % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                   (uintptr_t)z % (4 * elem) == 0 && (uintptr_t)out % (4 * elem) == 0;
  cudaError_t e;
#define EMBER_GGN1(T, VEC, FIRST)                                                                                  \
  launch_plain(gated_group_norm_kernel<T, VEC, FIRST>, grid, dim3(threads), 0, stream, y, (const T*)z, z_stride, w, (T*)out, \
               n, n / parts, eps, kind)
#define EMBER_GGN(T, VEC) ((gate_first & 1) ? EMBER_GGN1(T, VEC, true) : EMBER_GGN1(T, VEC, false))
  if (dtype == EMBER_F32)
    e = vec ? EMBER_GGN(float, true) : EMBER_GGN(float, false);
  else if (dtype == EMBER_BF16)
    e = vec ? EMBER_GGN(__nv_bfloat16, true) : EMBER_GGN(__nv_bfloat16, false);
  else
    return ember_fail("gated_group_norm: element type %d", dtype);
#undef EMBER_GGN
#undef EMBER_GGN1
  if (e != cudaSuccess) return ember_fail("gated_group_norm: %s", cudaGetErrorString(e));
  return 0;
}
