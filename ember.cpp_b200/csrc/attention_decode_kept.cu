// Decode attention (one new token per sequence, bfloat16) for mixers whose visible keys are the first
// `keep_first` positions of the sequence plus a window of the last positions (or all of them): the visible
// keys, counted in order (kept positions that lie before the window, then the window), are cut into chunks
// of 128; a block takes one chunk of one key/value head of one token and serves all query heads of that
// head, so that a key or value row is fetched once for the group; a second small launch merges the chunks.
//
// In a block each of four warps takes 32 keys, a key a lane: the lane reads its key's row in 16-byte pieces
// and makes the dot products with every query head of the group (the queries lie in shared memory, read by
// all lanes at once); one maximum and one correction per head for the warp's 32 keys; then the 32 value rows
// are walked through together, every lane owning a run of the value dims.  Softmax, sums and accumulators are
// float32.  Partial results (m, l, acc[vd]) per (token, head, chunk) go to scratch that the caller gives.
// With `slopes` the score of key j loses slopes[head] * (p - j); with `sinks` the merge adds exp(sinks[head]) to the
// softmax's denominator (a term without a key or a value).
#include "common.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kChunkKeys = 32 * kWarps;

// PER: query heads a key/value head (rounded up); DPL: value dims a lane (vd <= 32 * DPL, vd % DPL == 0)
template <int PER, int DPL>
__global__ void __launch_bounds__(32 * kWarps)
decode_kept_partial_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ kc,
                           const __nv_bfloat16* __restrict__ vc, float* __restrict__ part,
                           const int* __restrict__ positions, const int* __restrict__ seq_slot,
                           const int* __restrict__ pages, int max_blocks, int n_heads, int kv_heads, int hd, int vd,
                           float scale, int window, int keep_first, int n_chunks, const float* __restrict__ slopes, int chunk,
                           const float* __restrict__ head_scales) {
  __shared__ float q_s[PER][256];
  __shared__ float m_s[kWarps][PER], l_s[kWarps][PER];
  __shared__ float acc_s[kWarps][PER][32 * DPL];
  const int c = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int per = n_heads / kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = seq_slot[t];
  const int p = positions[t];
  // the first visible key: the window's, or (chunk > 0) the first position of the query's own run of `chunk` positions
  const int lo = chunk > 0 ? p / chunk * chunk : (window > 0 ? max(0, p - window + 1) : 0);
  const int n_kept = window > 0 ? min(keep_first, lo) : 0;
  const int n_keys = n_kept + p - lo + 1;
  const int k0 = c * kChunkKeys;
  const size_t stride = (size_t)vd + 2;
  if (slot < 0 || k0 >= n_keys) {  // nothing here: a partial result that the merge passes over
    if ((int)threadIdx.x < per) {
      float* dst = part + (((size_t)t * n_heads + g * per + threadIdx.x) * n_chunks + c) * stride;
      dst[0] = -INFINITY;
      dst[1] = 0.f;
    }
    return;
  }
  const int k1 = min(n_keys, k0 + kChunkKeys);
  const int width = (n_heads + kv_heads) * hd + kv_heads * vd;
  const __nv_bfloat16* q = qkv + (size_t)t * width + (size_t)g * per * hd;
  for (int i = threadIdx.x; i < per * hd; i += 32 * kWarps) q_s[i / hd][i % hd] = __bfloat162float(__ldcg(q + i));
  __syncthreads();

  const int* my_pages = pages + (size_t)t * max_blocks;
  const int idx = k0 + warp * 32 + lane;
  const int j = idx < n_kept ? idx : lo + idx - n_kept;
  const int page = idx < k1 ? my_pages[j / kPage] : -1;
  const bool valid = page >= 0;
  const size_t row = valid ? ((size_t)page * kv_heads + g) * kPage + (j % kPage) : 0;

  float sc[PER];
#pragma unroll
  for (int h = 0; h < PER; ++h) sc[h] = 0.f;
  if (valid) {
    const __nv_bfloat16* k = kc + row * hd;
    for (int d = 0; d < hd; d += 8) {  // (head sizes are multiples of 8: rows of 16-byte pieces)
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      float kv[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h2[i]);
        kv[2 * i] = f.x;
        kv[2 * i + 1] = f.y;
      }
#pragma unroll
      for (int h = 0; h < PER; ++h) {
        if (h < per) {
#pragma unroll
          for (int i = 0; i < 8; ++i) sc[h] = fmaf(q_s[h][d + i], kv[i], sc[h]);
        }
      }
    }
  }
  float pj[PER];
#pragma unroll
  for (int h = 0; h < PER; ++h) {
    const float slope = slopes && h < per ? slopes[g * per + h] : 0.f;
    const float hs = head_scales && h < per ? scale * head_scales[g * per + h] : scale;
    const float s = valid ? sc[h] * hs - slope * (float)(p - j) : -INFINITY;
    const float m = warp_max(s);  // (the warp's first key is always there: m is finite)
    pj[h] = valid ? expf(s - m) : 0.f;
    const float l = warp_sum(pj[h]);
    if (lane == 0) {
      m_s[warp][h] = m;
      l_s[warp][h] = l;
    }
  }
  float acc[PER][DPL];
#pragma unroll
  for (int h = 0; h < PER; ++h)
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[h][i] = 0.f;
  const int n_valid = min(32, k1 - (k0 + warp * 32));  // <= 0: this warp has no keys
  const bool dims = lane * DPL < vd;
  for (int jj = 0; jj < n_valid; ++jj) {
    const unsigned long long r = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
    const int there = __shfl_sync(0xffffffffu, (int)valid, jj);
    float v[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) v[i] = 0.f;
    if (dims && there) {
      const __nv_bfloat16* vr = vc + r * vd + lane * DPL;
      if constexpr (DPL == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vr);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
        v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
      } else if constexpr (DPL == 2) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vr));
        v[0] = a.x, v[1] = a.y;
      } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) v[i] = __bfloat162float(vr[i]);
      }
    }
#pragma unroll
    for (int h = 0; h < PER; ++h) {
      const float pv = __shfl_sync(0xffffffffu, pj[h], jj);
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[h][i] = fmaf(pv, v[i], acc[h][i]);
    }
  }
  if (n_valid <= 0 && lane == 0) {
#pragma unroll
    for (int h = 0; h < PER; ++h) {
      m_s[warp][h] = -INFINITY;
      l_s[warp][h] = 0.f;
    }
  }
#pragma unroll
  for (int h = 0; h < PER; ++h)
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc_s[warp][h][lane * DPL + i] = acc[h][i];
  __syncthreads();
  // the four warps' results as one: thread per (head, value dim)
  for (int e = threadIdx.x; e < per * vd; e += 32 * kWarps) {
    const int h = e / vd, d = e % vd;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, m_s[w][h]);
    float l = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float f = m_s[w][h] == -INFINITY ? 0.f : expf(m_s[w][h] - m);
      l = fmaf(l_s[w][h], f, l);
      a = fmaf(acc_s[w][h][d], f, a);
    }
    float* dst = part + (((size_t)t * n_heads + g * per + h) * n_chunks + c) * stride;
    if (d == 0) {
      dst[0] = m;
      dst[1] = l;
    }
    dst[2 + d] = a;
  }
}

// grid (T * n_heads): out = sum_c e^(m_c - M) acc_c / sum_c e^(m_c - M) l_c, chunks in order
__global__ void decode_kept_merge_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out,
                                         const int* __restrict__ seq_slot, int n_heads, int vd, int n_chunks,
                                         const float* __restrict__ sinks) {
  const int item = blockIdx.x, t = item / n_heads;
  __nv_bfloat16* o = out + (size_t)item * vd;
  if (seq_slot[t] < 0) {
    for (int d = threadIdx.x; d < vd; d += blockDim.x) o[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const size_t stride = (size_t)vd + 2;
  const float* src = part + (size_t)item * n_chunks * stride;
  float m = sinks ? sinks[item % n_heads] : -INFINITY;
  for (int c = 0; c < n_chunks; ++c) m = fmaxf(m, src[c * stride]);
  float l = sinks ? expf(sinks[item % n_heads] - m) : 0.f;
  for (int c = 0; c < n_chunks; ++c) {
    const float mc = src[c * stride];
    if (mc != -INFINITY) l = fmaf(src[c * stride + 1], expf(mc - m), l);
  }
  const float inv = 1.0f / l;
  for (int d = threadIdx.x; d < vd; d += blockDim.x) {
    float a = 0.f;
    for (int c = 0; c < n_chunks; ++c) {
      const float mc = src[c * stride];
      if (mc != -INFINITY) a = fmaf(src[c * stride + 2 + d], expf(mc - m), a);
    }
    o[d] = __float2bfloat16_rn(a * inv);
  }
}

template <int PER, int DPL>
void launch_partial(dim3 grid, cudaStream_t stream, const void* qkv, const void* kc, const void* vc, float* part,
                    const int* positions, const int* seq_slot, const int* pages, int max_blocks, int n_heads,
                    int kv_heads, int hd, int vd, float scale, int window, int keep_first, int n_chunks, const float* slopes,
                    int chunk, const float* head_scales) {
  launch_plain(decode_kept_partial_kernel<PER, DPL>, grid, dim3(32 * kWarps), 0, stream, (const __nv_bfloat16*)qkv,
             (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, part, positions, seq_slot, pages, max_blocks, n_heads,
             kv_heads, hd, vd, scale, window, keep_first, n_chunks, slopes, chunk, head_scales);
}

}  // namespace

// Floats of scratch that a call needs.
EMBER_API size_t ember_attention_decode_kept_scratch(int T, int n_heads, int vd, int max_keys) {
  const size_t n_chunks = (size_t)((max_keys + kChunkKeys - 1) / kChunkKeys);
  return (size_t)T * n_heads * n_chunks * ((size_t)vd + 2);
}

// One token per sequence (token t is sequence t of the step), their keys and values already in the cache.
// max_keys: the most keys any token of the call can see (the grid is sized by it; a captured graph serves every
// length up to it).  Returns 2, having launched nothing, for sizes this kernel has no instantiation for
// (more than 8 query heads a key/value head, values of more than 128 or of an odd size above 32, head sizes that
// are no multiples of 8 or above 256): the caller then takes the plain kernel.
EMBER_API int ember_attention_decode_biased(const void* qkv, const void* kc, const void* vc, void* out, float* scratch,
                                            const int* positions, const int* seq_slot, const int* pages, int max_blocks,
                                            int T, int n_heads, int kv_heads, int hd, int vd, float scale, int window,
                                            int keep_first, int max_keys, const float* slopes, const float* sinks,
                                            cudaStream_t stream);

EMBER_API int ember_attention_decode_kept(const void* qkv, const void* kc, const void* vc, void* out, float* scratch,
                                          const int* positions, const int* seq_slot, const int* pages, int max_blocks,
                                          int T, int n_heads, int kv_heads, int hd, int vd, float scale, int window,
                                          int keep_first, int max_keys, cudaStream_t stream) {
  return ember_attention_decode_biased(qkv, kc, vc, out, scratch, positions, seq_slot, pages, max_blocks, T, n_heads, kv_heads,
                                       hd, vd, scale, window, keep_first, max_keys, nullptr, nullptr, stream);
}

// The same with a distance penalty (slopes: float32 per query head, or null) and a sink in the softmax's denominator
// (sinks: float32 per query head, or null).
EMBER_API int ember_attention_decode_chunked(const void* qkv, const void* kc, const void* vc, void* out, float* scratch,
                                             const int* positions, const int* seq_slot, const int* pages, int max_blocks,
                                             int T, int n_heads, int kv_heads, int hd, int vd, float scale, int window,
                                             int keep_first, int max_keys, const float* slopes, const float* sinks, int chunk,
                                             const float* head_scales, cudaStream_t stream);

EMBER_API int ember_attention_decode_biased(const void* qkv, const void* kc, const void* vc, void* out, float* scratch,
                                            const int* positions, const int* seq_slot, const int* pages, int max_blocks,
                                            int T, int n_heads, int kv_heads, int hd, int vd, float scale, int window,
                                            int keep_first, int max_keys, const float* slopes, const float* sinks,
                                            cudaStream_t stream) {
  return ember_attention_decode_chunked(qkv, kc, vc, out, scratch, positions, seq_slot, pages, max_blocks, T, n_heads, kv_heads,
                                        hd, vd, scale, window, keep_first, max_keys, slopes, sinks, 0, nullptr, stream);
}

// The same with sight limited to the query's own chunk (chunk > 0, in place of a window) and one more factor on the
// scores of every query head (head_scales: float32 per query head, or null).
EMBER_API int ember_attention_decode_chunked(const void* qkv, const void* kc, const void* vc, void* out, float* scratch,
                                             const int* positions, const int* seq_slot, const int* pages, int max_blocks,
                                             int T, int n_heads, int kv_heads, int hd, int vd, float scale, int window,
                                             int keep_first, int max_keys, const float* slopes, const float* sinks, int chunk,
                                             const float* head_scales, cudaStream_t stream) {
  EMBER_CHECK(chunk >= 0 && (chunk == 0 || (window == 0 && keep_first == 0)), "attention_decode_kept: chunk %d beside window %d",
              chunk, window);
  EMBER_CHECK(T > 0 && n_heads > 0 && kv_heads > 0 && max_blocks > 0 && max_keys > 0, "attention_decode_kept: bad sizes");
  EMBER_CHECK(n_heads % kv_heads == 0, "attention_decode_kept: %d heads are not a multiple of %d key/value heads", n_heads,
              kv_heads);
  EMBER_CHECK(window >= 0 && keep_first >= 0, "attention_decode_kept: window %d, kept first %d", window, keep_first);
  const int per = n_heads / kv_heads;
  int dpl = 0;
  for (int cand = 1; cand <= 4; cand *= 2)
    if (!dpl && vd <= 32 * cand && vd % cand == 0) dpl = cand;
  if (per > 8 || !dpl || hd % 8 || hd > 256) return 2;
  EMBER_CHECK(kv_heads <= 65535 && T <= 65535, "attention_decode_kept: %d tokens x %d heads exceed one launch", T, kv_heads);
  const int n_chunks = (max_keys + kChunkKeys - 1) / kChunkKeys;
  const dim3 grid(n_chunks, kv_heads, T);
  const int per_up = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : 8;
#define EMBER_KEPT(PER, DPL)                                                                                              \
  launch_partial<PER, DPL>(grid, stream, qkv, kc, vc, scratch, positions, seq_slot, pages, max_blocks, n_heads, kv_heads, \
                           hd, vd, scale, window, keep_first, n_chunks, slopes, chunk, head_scales)
#define EMBER_KEPT_PER(PER)          \
  do {                               \
    if (dpl == 1) EMBER_KEPT(PER, 1); \
    else if (dpl == 2) EMBER_KEPT(PER, 2); \
    else EMBER_KEPT(PER, 4);          \
  } while (0)
  if (per_up == 1) EMBER_KEPT_PER(1);
  else if (per_up == 2) EMBER_KEPT_PER(2);
  else if (per_up == 4) EMBER_KEPT_PER(4);
  else EMBER_KEPT_PER(8);
#undef EMBER_KEPT_PER
#undef EMBER_KEPT
  EMBER_LAUNCH_OK("attention_decode_kept");
  launch_plain(decode_kept_merge_kernel, dim3(T * n_heads), dim3(vd <= 32 ? 32 : (vd <= 64 ? 64 : 128)), 0, stream,
             (const float*)scratch, (__nv_bfloat16*)out, seq_slot, n_heads, vd, n_chunks, sinks);
  EMBER_LAUNCH_OK("attention_decode_kept (merge)");
  return 0;
}
