// Attention over cached low-rank rows, and the small operations around it.
//
// A layer of this kind caches, per position, a normed row c of `rank` values and a rotated key part
// k_r of `rot` values that all heads share (page p of the layer: [1][64][rank] and [1][64][rot]).  A
// query head arrives already carried into the row's space: `rank` values to be compared with c, then
// `rot` rotated values to be compared with k_r.  Its output is the softmax-weighted sum of the rows c.
//
//   rotate          pairs (i, i + dims/2) of a vector's first `dims` values turned by position * freq[i],
//                   cos and sin times a magnitude; the rest copied; float32 angles, sincosf
//   latent_rows     per token: the query row's RMS norm, the cached row's RMS norm, the shared key
//                   part's rotation, and the write of both into the cache, one launch
//   head_linear     out[t, h] = a[t, h] W[h]^T for every head h, heads side by side in a row
//   latent_attention_plain   one warp per (token, head), keys in groups of 32 from position 0, an online
//                   softmax whose order depends on key positions alone: the kernel of the 32-bit path
//                   and the twin that the faster kernels are tested against
#include "common.cuh"

namespace {

constexpr int kThreads = 128;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += red[w];
  return total;
}

// One pair of a rotation: (u, v) at `position` with frequency f.
__device__ __forceinline__ void turn(float u, float v, int position, float f, float magnitude, float& ou, float& ov) {
  float sn, cs;
  sincosf((float)position * f, &sn, &cs);
  sn *= magnitude;
  cs *= magnitude;
  ou = u * cs - v * sn;
  ov = v * cs + u * sn;
}

// grid (T, heads); src and dst may be the same tensor (a thread reads its pair before it writes it).
template <typename TS, typename TD>
__global__ void rotate_kernel(const TS* src, long long src_stride, int src_col, int src_head, TD* dst, long long dst_stride,
                              int dst_col, int dst_head, int width, const int* __restrict__ positions,
                              const float* __restrict__ freqs, float magnitude, int dims, int interleaved) {
  const int t = blockIdx.x, h = blockIdx.y, half = dims / 2;
  const TS* s = src + (size_t)t * src_stride + src_col + (size_t)h * src_head;
  TD* d = dst + (size_t)t * dst_stride + dst_col + (size_t)h * dst_head;
  const int p = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float ou, ov;
    const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;   // pair i: neighbours, or half apart
    turn(to_float(s[iu]), to_float(s[iv]), p, freqs[i], magnitude, ou, ov);
    d[iu] = from_float<TD>(ou);
    d[iv] = from_float<TD>(ov);
  }
  for (int i = dims + threadIdx.x; i < width; i += blockDim.x) d[i] = from_float<TD>(to_float(s[i]));
}

// grid (T): down float32 [T, q_rank (+ rank + rot)].
template <typename T>
__global__ void __launch_bounds__(kThreads)
latent_rows_kernel(const float* __restrict__ down, int down_width, int q_rank, const float* __restrict__ q_gain,
                   const float* __restrict__ c_gain, int rank, int rot, float eps, const float* __restrict__ freqs,
                   float magnitude, int dims, T* __restrict__ c_q, T* __restrict__ kc, T* __restrict__ vc,
                   const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                   const int* __restrict__ pages, int max_blocks) {
  __shared__ float red[kThreads / 32];
  const int t = blockIdx.x;
  const int s = token_seq[t];
  T* cq = c_q + (size_t)t * q_rank;
  if (seq_slot[s] < 0) {
    for (int i = threadIdx.x; i < q_rank; i += kThreads) cq[i] = from_float<T>(0.f);
    return;
  }
  const float* row = down + (size_t)t * down_width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += kThreads) ss = fmaf(row[i], row[i], ss);
  float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += kThreads) cq[i] = from_float<T>(row[i] * inv * q_gain[i]);
  if (kc == nullptr) return;
  const int p = positions[t];
  const int page = pages[(size_t)s * max_blocks + p / kPage];
  if (page < 0) return;
  const float* c = row + q_rank;
  ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += kThreads) ss = fmaf(c[i], c[i], ss);
  inv = 1.0f / sqrtf(block_sum(ss, red) / (float)rank + eps);
  T* kdst = kc + ((size_t)page * kPage + (p % kPage)) * rank;
  for (int i = threadIdx.x; i < rank; i += kThreads) kdst[i] = from_float<T>(c[i] * inv * c_gain[i]);
  const float* r = c + rank;
  T* vdst = vc + ((size_t)page * kPage + (p % kPage)) * rot;
  const int half = dims / 2;
  for (int i = threadIdx.x; i < half; i += kThreads) {
    float ou, ov;
    turn(r[i], r[i + half], p, freqs[i], magnitude, ou, ov);
    vdst[i] = from_float<T>(ou);
    vdst[i + half] = from_float<T>(ov);
  }
  for (int i = dims + threadIdx.x; i < rot; i += kThreads) vdst[i] = from_float<T>(r[i]);
}

// out[t, out_col + h * out_head + n] = sum_k a[t, a_col + h * a_head + k] * w[h][n][k], float32 sums in ascending k.
// grid (ceil(T / 32), ceil(N / 32), heads), block (32, 8): a tile of 32 tokens x 32 outputs of one head.
template <typename T>
__global__ void head_linear_kernel(const T* __restrict__ a, long long a_stride, int a_col, int a_head,
                                   const T* __restrict__ w, T* __restrict__ out, long long out_stride, int out_col,
                                   int out_head, int T_tokens, int N, int K) {
  __shared__ float as[32][33], ws[32][33];
  const int h = blockIdx.z, m0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const T* ah = a + a_col + (size_t)h * a_head;
  const T* wh = w + (size_t)h * N * K;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 8 * i, k = k0 + tx;
      as[r][tx] = (m0 + r < T_tokens && k < K) ? to_float(ah[(size_t)(m0 + r) * a_stride + k]) : 0.f;
      ws[r][tx] = (n0 + r < N && k < K) ? to_float(wh[(size_t)(n0 + r) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) {
      const float wv = ws[tx][kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(as[ty + 8 * i][kk], wv, acc[i]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 8 * i, n = n0 + tx;
    if (m < T_tokens && n < N) out[(size_t)m * out_stride + out_col + (size_t)h * out_head + n] = from_float<T>(acc[i]);
  }
}

constexpr int kMaxRank = 1024;

// q [T, heads * (rank + rot)]; out [T, heads * rank]; dynamic shared memory: 4 warps x (rank + rot) floats.
template <typename T>
__global__ void __launch_bounds__(128)
latent_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc, T* __restrict__ out,
                              const int* __restrict__ positions, const int* __restrict__ token_seq,
                              const int* __restrict__ seq_slot, const int* __restrict__ pages, int max_blocks, int T_tokens,
                              int heads, int rank, int rot, float scale) {
  extern __shared__ float q_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + warp;
  if (item >= T_tokens * heads) return;   // whole warps leave together
  const int t = item / heads, h = item % heads;
  const int row = rank + rot;
  float* q_s = q_all + (size_t)warp * row;
  T* o = out + (size_t)t * heads * rank + (size_t)h * rank;
  const int s = token_seq[t];
  if (seq_slot[s] < 0) {
    for (int d = lane; d < rank; d += 32) o[d] = from_float<T>(0.f);
    return;
  }
  const int p = positions[t];
  const int* my_pages = pages + (size_t)s * max_blocks;
  const T* qr = q + (size_t)t * heads * row + (size_t)h * row;
  for (int d = lane; d < row; d += 32) q_s[d] = to_float(qr[d]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[kMaxRank / 32];
#pragma unroll
  for (int i = 0; i < kMaxRank / 32; ++i) acc[i] = 0.f;
  const int n_keys = p + 1;
  for (int base = 0; base < n_keys; base += 32) {
    const int j = base + lane;
    const int page = j < n_keys ? my_pages[j / kPage] : -1;
    const bool valid = page >= 0;   // a page that is not held contributes nothing and is never read
    size_t r = 0;
    float sc = -INFINITY;
    if (valid) {
      r = (size_t)page * kPage + (j % kPage);
      const T* c = kc + r * rank;
      const T* kr = vc + r * rot;
      float dot = 0.f;
      for (int d = 0; d < rank; ++d) dot = fmaf(q_s[d], to_float(c[d]), dot);
      for (int d = 0; d < rot; ++d) dot = fmaf(q_s[rank + d], to_float(kr[d]), dot);
      sc = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float pj = valid ? expf(sc - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < kMaxRank / 32; ++i) acc[i] *= corr;
    const int n_valid = min(32, n_keys - base);
    for (int jj = 0; jj < n_valid; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const unsigned long long rr = __shfl_sync(0xffffffffu, (unsigned long long)r, jj);
      const T* c = kc + rr * rank;
#pragma unroll
      for (int i = 0; i < kMaxRank / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) acc[i] = fmaf(pv, to_float(c[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < kMaxRank / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < rank) o[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace

// src [T, *] of element type src_dtype, dst [T, *] of dst_dtype (row strides in elements); see rotate_kernel.
EMBER_API int ember_rotate_pairs(const void* src, long long src_stride, int src_col, int src_head, int src_dtype, void* dst,
                                 long long dst_stride, int dst_col, int dst_head, int dst_dtype, int T, int heads, int width,
                                 const int* positions, const float* freqs, float magnitude, int dims, int interleaved,
                                 cudaStream_t stream);

EMBER_API int ember_rotate(const void* src, long long src_stride, int src_col, int src_head, int src_dtype, void* dst,
                           long long dst_stride, int dst_col, int dst_head, int dst_dtype, int T, int heads, int width,
                           const int* positions, const float* freqs, float magnitude, int dims, cudaStream_t stream) {
  return ember_rotate_pairs(src, src_stride, src_col, src_head, src_dtype, dst, dst_stride, dst_col, dst_head, dst_dtype, T, heads,
                            width, positions, freqs, magnitude, dims, 0, stream);
}

// The same with the pairing as an argument: interleaved 0 pairs dimension i with i + dims / 2, 1 pairs 2i with 2i + 1.
EMBER_API int ember_rotate_pairs(const void* src, long long src_stride, int src_col, int src_head, int src_dtype, void* dst,
                                 long long dst_stride, int dst_col, int dst_head, int dst_dtype, int T, int heads, int width,
                                 const int* positions, const float* freqs, float magnitude, int dims, int interleaved,
                                 cudaStream_t stream) {
  EMBER_CHECK(T > 0 && heads > 0 && heads <= 65535 && width > 0, "rotate: bad sizes");
  EMBER_CHECK(dims > 0 && dims % 2 == 0 && dims <= width, "rotate: %d rotated dimensions of %d", dims, width);
  const dim3 grid(T, heads);
  const int threads = dims / 2 >= 64 || width - dims >= 64 ? 128 : 32;
#define EMBER_ROTATE(TS, TD)                                                                                          \
  rotate_kernel<TS, TD><<<grid, threads, 0, stream>>>((const TS*)src, src_stride, src_col, src_head, (TD*)dst, dst_stride, \
                                                      dst_col, dst_head, width, positions, freqs, magnitude, dims, interleaved)
  if (src_dtype == EMBER_F32 && dst_dtype == EMBER_F32)
    EMBER_ROTATE(float, float);
  else if (src_dtype == EMBER_BF16 && dst_dtype == EMBER_BF16)
    EMBER_ROTATE(__nv_bfloat16, __nv_bfloat16);
  else if (src_dtype == EMBER_F32 && dst_dtype == EMBER_BF16)
    EMBER_ROTATE(float, __nv_bfloat16);
  else
    return ember_fail("rotate: element types %d -> %d", src_dtype, dst_dtype);
#undef EMBER_ROTATE
  EMBER_LAUNCH_OK("rotate");
  return 0;
}

// kc, vc null: a layer that reads another's cached rows makes only its query row.
EMBER_API int ember_latent_rows(const float* down, int down_width, int q_rank, const float* q_gain, const float* c_gain,
                                int rank, int rot, float eps, const float* freqs, float magnitude, int dims, void* c_q,
                                void* kc, void* vc, const int* positions, const int* token_seq, const int* seq_slot,
                                const int* pages, int max_blocks, int T, int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && q_rank > 0 && down_width >= q_rank, "latent_rows: bad sizes");
  EMBER_CHECK((kc == nullptr) == (vc == nullptr), "latent_rows: both cache tensors or none");
  if (kc != nullptr) {
    EMBER_CHECK(rank > 0 && rot > 0 && down_width == q_rank + rank + rot, "latent_rows: rows of %d are not %d + %d + %d",
                down_width, q_rank, rank, rot);
    EMBER_CHECK(dims > 0 && dims % 2 == 0 && dims <= rot, "latent_rows: %d rotated dimensions of %d", dims, rot);
  }
  if (dtype == EMBER_F32)
    latent_rows_kernel<float><<<T, kThreads, 0, stream>>>(down, down_width, q_rank, q_gain, c_gain, rank, rot, eps, freqs,
                                                          magnitude, dims, (float*)c_q, (float*)kc, (float*)vc, positions,
                                                          token_seq, seq_slot, pages, max_blocks);
  else if (dtype == EMBER_BF16)
    latent_rows_kernel<__nv_bfloat16><<<T, kThreads, 0, stream>>>(
        down, down_width, q_rank, q_gain, c_gain, rank, rot, eps, freqs, magnitude, dims, (__nv_bfloat16*)c_q,
        (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, positions, token_seq, seq_slot, pages, max_blocks);
  else
    return ember_fail("latent_rows: element type %d", dtype);
  EMBER_LAUNCH_OK("latent_rows");
  return 0;
}

EMBER_API int ember_head_linear(const void* a, long long a_stride, int a_col, int a_head, const void* w, void* out,
                                long long out_stride, int out_col, int out_head, int T, int heads, int N, int K, int dtype,
                                cudaStream_t stream) {
  EMBER_CHECK(T > 0 && heads > 0 && heads <= 65535 && N > 0 && K > 0, "head_linear: bad sizes");
  EMBER_CHECK((N + 31) / 32 <= 65535, "head_linear: %d outputs exceed one launch", N);
  const dim3 grid((T + 31) / 32, (N + 31) / 32, heads), block(32, 8);
  if (dtype == EMBER_F32)
    head_linear_kernel<float><<<grid, block, 0, stream>>>((const float*)a, a_stride, a_col, a_head, (const float*)w,
                                                          (float*)out, out_stride, out_col, out_head, T, N, K);
  else if (dtype == EMBER_BF16)
    head_linear_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((const __nv_bfloat16*)a, a_stride, a_col, a_head,
                                                                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride,
                                                                  out_col, out_head, T, N, K);
  else
    return ember_fail("head_linear: element type %d", dtype);
  EMBER_LAUNCH_OK("head_linear");
  return 0;
}

EMBER_API int ember_latent_attention_plain(const void* q, const void* kc, const void* vc, void* out, const int* positions,
                                           const int* token_seq, const int* seq_slot, const int* pages, int max_blocks, int T,
                                           int heads, int rank, int rot, float scale, int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && heads > 0 && max_blocks > 0, "latent_attention: bad sizes");
  EMBER_CHECK(rank >= 1 && rank <= kMaxRank && rot >= 1, "latent_attention: rows of %d + %d values (at most %d + any)", rank,
              rot, kMaxRank);
  const long long items = (long long)T * heads;
  const int grid = (int)((items + 3) / 4);
  const size_t smem = 4 * (size_t)(rank + rot) * sizeof(float);
  EMBER_CHECK(smem <= 48 * 1024, "latent_attention: rows of %d values exceed the kernel's shared memory", rank + rot);
  if (dtype == EMBER_F32)
    latent_attention_plain_kernel<float><<<grid, 128, smem, stream>>>((const float*)q, (const float*)kc, (const float*)vc,
                                                                      (float*)out, positions, token_seq, seq_slot, pages,
                                                                      max_blocks, T, heads, rank, rot, scale);
  else if (dtype == EMBER_BF16)
    latent_attention_plain_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, (__nv_bfloat16*)out, positions, token_seq,
        seq_slot, pages, max_blocks, T, heads, rank, rot, scale);
  else
    return ember_fail("latent_attention: element type %d", dtype);
  EMBER_LAUNCH_OK("latent_attention_plain");
  return 0;
}
