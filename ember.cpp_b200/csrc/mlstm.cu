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
// are staged in shared memory at a time, and that warp makes the maxima of those tokens with a scan, a lane
// a token.  Every column is independent of the others, so a token's result depends on its sequence alone,
// never on the batch or the step's cut beyond rounding.  A sequence that starts at position 0 starts from zeros whatever its slot's state
// holds; sequences of slot -1 are padding: their rows are zero and no state is touched.
//
// A long sequence is cut into pieces that are walked side by side.  The recurrence is linear in (S, n) once
// the gates are known, and the maximum is associative: a piece walked from nothing (S = 0, n = 0, m = -inf)
// ends in (S', n', m') and the sum F of its log forget gates, and a state (S, n, m) in front of it becomes
// m'' = max(F + m, m'), S'' = exp(F + m - m'') S + exp(m' - m'') S' (n likewise).  So: a first walk of every
// piece from nothing, a small kernel that makes every piece's start state from those in order, and a second
// walk of every piece from its start state, which writes the results.
#include "common.cuh"

namespace {

__device__ __forceinline__ float log_sigmoid(float v) { return fminf(v, 0.f) - log1pf(expf(-fabsf(v))); }

// 16 bytes of a row as float32 values.
__device__ __forceinline__ void load_row_part(const float* src, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(src);
  v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
}
__device__ __forceinline__ void load_row_part(const __nv_bfloat16* src, float (&v)[8]) {
  const uint4 x = *reinterpret_cast<const uint4*>(src);
  const unsigned w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    v[2 * u] = __uint_as_float(w[u] << 16);
    v[2 * u + 1] = __uint_as_float(w[u] & 0xffff0000u);
  }
}

// grid (T, row groups), 128 threads: a warp a gate row (2 * heads of them: input gates, then forget gates).  A row is
// summed by one warp in an order that its length alone fixes: 16-byte parts where every row starts on 16 bytes.
template <typename T>
__global__ void mlstm_gates_kernel(const T* __restrict__ h, const T* __restrict__ w, const float* __restrict__ bias,
                                   float* __restrict__ gates, int heads, int width, float cap) {
  constexpr int kVec = 16 / (int)sizeof(T);
  const int t = blockIdx.x, lane = threadIdx.x & 31;
  const int r = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= 2 * heads) return;
  const T* row = h + (size_t)t * width;
  const T* wr = w + (size_t)r * width;
  float acc = 0.f;
  if (width % kVec == 0 && ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(w)) & 15) == 0) {
    float acc2 = 0.f;
    for (int d = lane * kVec; d < width; d += 32 * kVec) {
      float a[kVec], b[kVec];
      load_row_part(row + d, a);
      load_row_part(wr + d, b);
#pragma unroll
      for (int u = 0; u < kVec; u += 2) {
        acc = fmaf(a[u], b[u], acc);
        acc2 = fmaf(a[u + 1], b[u + 1], acc2);
      }
    }
    acc += acc2;
  } else {
    for (int d = lane; d < width; d += 32) acc = fmaf(to_float(row[d]), to_float(wr[d]), acc);
  }
  acc = warp_sum(acc) + bias[r];
  const float capped = cap > 0.f ? cap * tanhf(acc / cap) : acc;
  if (lane == 0) gates[(size_t)t * 2 * heads + r] = r < heads ? capped : log_sigmoid(capped);
}

constexpr int kStage = 32;   // tokens staged in shared memory at a time: a lane of the normaliser's warp each

constexpr int kSplit = 4;    // lanes that share a column: each keeps a quarter of S[:, j]

// grid (sequences x pieces, heads, column tiles); blockDim.x = kSplit * cols + 32: kSplit neighbouring lanes a column
// (lane s of them keeps S[d, j] for d in the 16-byte parts s, s + kSplit, ... of a key row: DMAX / kSplit registers) and
// the normaliser's warp.  DMAX >= dim, a multiple of 32.  Two blocks an SM up to a key size of 128 (96 registers a thread:
// with three blocks and 72 the loads of k and q stand closer in front of their use, 400 against 373 microseconds for
// 2,048 tokens of 8 heads of 128 x 256), one above.
template <typename T, int DMAX>
__global__ void __launch_bounds__(kSplit * 64 + 32, DMAX <= 128 ? 2 : 1)
mlstm_scan_kernel(const T* __restrict__ qkv, long long stride, int q_col, int k_col, int v_col,
                                  const float* __restrict__ gates, float* __restrict__ S_state, float* __restrict__ n_state,
                                  float* __restrict__ m_state, float* __restrict__ out, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int dim,
                                  int vdim, float floor_, int piece, int pieces, int phase, float* __restrict__ scratch) {
  extern __shared__ float smem[];
  constexpr int kMine = DMAX / kSplit;      // values of S a column lane keeps
  const int workers = blockDim.x - 32;      // the column lanes
  const int cols = workers / kSplit;
  float* ks = smem;                         // [kStage][DMAX]
  float* qs = ks + kStage * DMAX;           // [kStage][DMAX]
  float* vs = qs + kStage * DMAX;           // [kStage][cols]; the numerators afterwards
  float* keep = vs + kStage * cols;         // [kStage] exp(f + m_before - m)
  float* take = keep + kStage;              // [kStage] exp(i - m)
  float* den = take + kStage;               // [kStage] exp(-m), then the denominator
  // phase 0: the whole walk (one piece).  phase 1: a piece from nothing, its end left in scratch.  phase 2: a piece from
  // the start state that the carry left in scratch.
  const int s = blockIdx.x / pieces, pc = blockIdx.x % pieces, h = blockIdx.y;
  const bool column = (int)threadIdx.x < workers;
  const int c = threadIdx.x / kSplit, part = threadIdx.x % kSplit;
  const int j = blockIdx.z * cols + c;
  const bool live = column && j < vdim;
  const int lane = threadIdx.x & 31;
  const int seq_n = cu_new[s + 1] - cu_new[s];
  const int lo = pc * piece, hi = min(seq_n, lo + piece);
  if (lo >= seq_n) return;
  const int t0 = cu_new[s] + lo, n = hi - lo;
  const int slot = seq_slot[s];
  const int inner = heads * vdim;
  const int j0 = blockIdx.z * cols, jn = min(cols, vdim - j0);       // the block's columns
  if (slot < 0) {
    if (phase != 1)
      for (int e = threadIdx.x; e < n * jn; e += blockDim.x)
        out[(size_t)(t0 + e / jn) * inner + (size_t)h * vdim + j0 + e % jn] = 0.f;
    return;
  }
  const bool carried = phase == 2 || (phase == 0 && seq_start[s] > 0);
  const float q_scale = rsqrtf((float)dim);
  // where this walk starts from and where it leaves its end: the slot's rows, or the piece's place in scratch
  float* mine = phase == 0 ? nullptr : scratch + ((size_t)blockIdx.x * heads + h) * ((size_t)dim * vdim + dim + 3);
  float* col = (phase == 0 ? S_state + ((size_t)slot * heads + h) * dim * vdim : mine) + j;
  float* nrow = phase == 0 ? n_state + ((size_t)slot * heads + h) * dim : mine + (size_t)dim * vdim;
  float* mval = phase == 0 ? m_state + (size_t)slot * heads + h : mine + (size_t)dim * vdim + dim + (phase == 2 ? 2 : 0);
  // a column lane: S[d, j] in S[4 r + u] for d = 4 (kSplit r + part) + u; a lane of the normaliser's warp: n[lane + 32 r] in S[r]
  float S[kMine];
  if (column) {
#pragma unroll
    for (int r = 0; r < kMine; ++r) {
      const int d = 4 * (kSplit * (r / 4) + part) + r % 4;
      S[r] = (live && carried && d < dim) ? col[(size_t)d * vdim] : 0.f;
    }
  } else {
#pragma unroll
    for (int r = 0; r < DMAX / 32; ++r) {
      const int d = lane + 32 * r;
      S[r] = (carried && d < dim) ? nrow[d] : 0.f;
    }
  }
  float m = carried ? *mval : (phase == 1 ? -INFINITY : 0.f);   // walked by the normaliser's warp (every lane holds it)
  constexpr int kVec = 16 / (int)sizeof(T);
  // rows of q and k in 16-byte parts where every part starts on 16 bytes
  const bool vectors = dim % kVec == 0 && stride % kVec == 0 && q_col % kVec == 0 && k_col % kVec == 0 &&
                       (reinterpret_cast<uintptr_t>(qkv) & 15) == 0;
  float F = 0.f;                                                 // (phase 1) the sum of the piece's log forget gates

  for (int c0 = 0; c0 < n; c0 += kStage) {
    const int cn = min(kStage, n - c0);
    const int cn4 = (cn + 3) & ~3;      // tokens are walked four at a time: the rows behind the last one are zeros
    __syncthreads();
    if (vectors) {
      for (int e = threadIdx.x; e < cn4 * (DMAX / kVec); e += blockDim.x) {
        const int i = e / (DMAX / kVec), d = (e % (DMAX / kVec)) * kVec;
        const T* src = qkv + (size_t)(t0 + c0 + i) * stride + (size_t)h * dim + d;
        float qv[kVec], kv[kVec];
        if (d < dim && i < cn) {
          load_row_part(src + q_col, qv);
          load_row_part(src + k_col, kv);
        } else {
#pragma unroll
          for (int u = 0; u < kVec; ++u) qv[u] = kv[u] = 0.f;
        }
#pragma unroll
        for (int u = 0; u < kVec; u += 4) {
          *reinterpret_cast<float4*>(qs + i * DMAX + d + u) =
              make_float4(qv[u] * q_scale, qv[u + 1] * q_scale, qv[u + 2] * q_scale, qv[u + 3] * q_scale);
          *reinterpret_cast<float4*>(ks + i * DMAX + d + u) = make_float4(kv[u], kv[u + 1], kv[u + 2], kv[u + 3]);
        }
      }
    } else {
      for (int e = threadIdx.x; e < cn4 * DMAX; e += blockDim.x) {
        const int i = e / DMAX, d = e % DMAX;
        const T* src = qkv + (size_t)(t0 + c0 + i) * stride + (size_t)h * dim + d;
        qs[e] = d < dim && i < cn ? to_float(src[q_col]) * q_scale : 0.f;
        ks[e] = d < dim && i < cn ? to_float(src[k_col]) : 0.f;
      }
    }
    for (int e = threadIdx.x; e < cn4 * cols; e += blockDim.x) {
      const int i = e / cols, cc = e % cols;
      vs[e] = cc < jn && i < cn ? to_float(qkv[(size_t)(t0 + c0 + i) * stride + v_col + (size_t)h * vdim + j0 + cc]) : 0.f;
    }
    if (!column) {
      // The maxima of the stage's tokens at once, a lane a token.  m -> max(a + m, b) is what a run of tokens does to
      // the maximum in front of it (one token: a = f, b = i; a run behind another: a = a1 + a2, b = max(a2 + b1, b2)),
      // so a scan over the lanes leaves every token's (a, b) from the stage's start, and m_t = max(a_t + m, b_t).
      // The maximum is a stabiliser: the memory, the normaliser and exp(-m) all carry the factor exp(-m_t), and the
      // result is the same for any m_t as long as each token's factors use the m of the token before it, as here.
      float a = 0.f, b = -INFINITY, li = 0.f, lf = 0.f;
      if (lane < cn) {
        const float* g = gates + (size_t)(t0 + c0 + lane) * 2 * heads;
        li = g[h];
        lf = g[heads + h];
        a = lf;
        b = li;
      }
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float a1 = __shfl_up_sync(0xffffffffu, a, off), b1 = __shfl_up_sync(0xffffffffu, b, off);
        if (lane >= off) {
          b = fmaxf(a + b1, b);
          a += a1;
        }
      }
      const float m_new = fmaxf(a + m, b);
      float m_before = __shfl_up_sync(0xffffffffu, m_new, 1);
      if (lane == 0) m_before = m;
      keep[lane] = lane < cn ? expf(lf + m_before - m_new) : 1.f;     // (behind the last token: nothing changes)
      take[lane] = lane < cn ? expf(li - m_new) : 0.f;
      den[lane] = expf(-m_new);
      m = __shfl_sync(0xffffffffu, m_new, cn - 1);
      F += __shfl_sync(0xffffffffu, a, cn - 1);
    }
    __syncthreads();
    // Four tokens at a time: their rows are read and their sums made side by side, and one lane of the column's four
    // writes each token's numerator afterwards, so that nothing is written between the reads of a group.
    if (column && phase == 1) {      // no results: the memory alone
      for (int i0 = 0; i0 < cn; i0 += 4) {
        float a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          a[u] = keep[i0 + u];
          b[u] = take[i0 + u] * vs[(i0 + u) * cols + c];
        }
#pragma unroll
        for (int r = 0; r < kMine; r += 4) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float4 kv = *reinterpret_cast<const float4*>(ks + (i0 + u) * DMAX + 4 * part + kSplit * r);
            S[r] = fmaf(a[u], S[r], b[u] * kv.x);
            S[r + 1] = fmaf(a[u], S[r + 1], b[u] * kv.y);
            S[r + 2] = fmaf(a[u], S[r + 2], b[u] * kv.z);
            S[r + 3] = fmaf(a[u], S[r + 3], b[u] * kv.w);
          }
        }
      }
    } else if (column) {
      for (int i0 = 0; i0 < cn; i0 += 4) {
        float a[4], b[4], o[4], p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          a[u] = keep[i0 + u];
          b[u] = take[i0 + u] * vs[(i0 + u) * cols + c];
          o[u] = p[u] = 0.f;
        }
#pragma unroll
        for (int r = 0; r < kMine; r += 4) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float4 kv = *reinterpret_cast<const float4*>(ks + (i0 + u) * DMAX + 4 * part + kSplit * r);
            const float4 qv = *reinterpret_cast<const float4*>(qs + (i0 + u) * DMAX + 4 * part + kSplit * r);
            S[r] = fmaf(a[u], S[r], b[u] * kv.x);
            S[r + 1] = fmaf(a[u], S[r + 1], b[u] * kv.y);
            S[r + 2] = fmaf(a[u], S[r + 2], b[u] * kv.z);
            S[r + 3] = fmaf(a[u], S[r + 3], b[u] * kv.w);
            o[u] = fmaf(S[r], qv.x, o[u]);
            p[u] = fmaf(S[r + 1], qv.y, p[u]);
            o[u] = fmaf(S[r + 2], qv.z, o[u]);
            p[u] = fmaf(S[r + 3], qv.w, p[u]);
          }
        }
        // the column's lanes are neighbours in one warp; every one of them has read the group's values before the exchange
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          o[u] += p[u];
          o[u] += __shfl_xor_sync(0xffffffffu, o[u], 1);
          o[u] += __shfl_xor_sync(0xffffffffu, o[u], 2);
        }
        const float own = part == 0 ? o[0] : part == 1 ? o[1] : part == 2 ? o[2] : o[3];
        if (i0 + part < cn) vs[(i0 + part) * cols + c] = own;     // the numerator, in the place of the value it came from
      }
    } else {
      for (int i0 = 0; i0 < cn; i0 += 4) {
        float a[4], b[4], dot[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          a[u] = keep[i0 + u];
          b[u] = take[i0 + u];
          dot[u] = 0.f;
        }
#pragma unroll
        for (int r = 0; r < DMAX / 32; ++r) {
          const int d = lane + 32 * r;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            S[r] = fmaf(a[u], S[r], b[u] * ks[(i0 + u) * DMAX + d]);
            dot[u] = fmaf(S[r], qs[(i0 + u) * DMAX + d], dot[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) dot[u] = warp_sum(dot[u]);
        const float own = lane == 0 ? dot[0] : lane == 1 ? dot[1] : lane == 2 ? dot[2] : dot[3];
        if (lane < 4 && i0 + lane < cn) den[i0 + lane] = fmaxf(fabsf(own), den[i0 + lane]) + floor_;
      }
    }
    __syncthreads();
    if (phase != 1)
      for (int e = threadIdx.x; e < cn * jn; e += blockDim.x) {
        const int i = e / jn, cc = e % jn;
        out[(size_t)(t0 + c0 + i) * inner + (size_t)h * vdim + j0 + cc] = vs[i * cols + cc] / den[i];
      }
  }
  // the end: into the piece's place (phase 1), or into the slot's rows by the walk that reaches the sequence's end
  if (phase == 2) {
    if (hi < seq_n) return;
    col = S_state + ((size_t)slot * heads + h) * dim * vdim + j;
    nrow = n_state + ((size_t)slot * heads + h) * dim;
    mval = m_state + (size_t)slot * heads + h;
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < kMine; ++r) {
      const int d = 4 * (kSplit * (r / 4) + part) + r % 4;
      if (d < dim) col[(size_t)d * vdim] = S[r];
    }
  }
  if (!column && blockIdx.z == 0) {
#pragma unroll
    for (int r = 0; r < DMAX / 32; ++r) {
      const int d = lane + 32 * r;
      if (d < dim) nrow[d] = S[r];
    }
    if (lane == 0) {
      *mval = m;
      if (phase == 1) mval[1] = F;
    }
  }
}

// grid (sequences, heads, blocks over the dim * vdim + dim values of S and n): every piece's place in scratch, which holds
// the piece's end from nothing (S', n', m', F, -), gets the state in front of the piece (S, n, -, -, m) instead.
__global__ void mlstm_carry_kernel(float* __restrict__ scratch, const float* __restrict__ S_state, const float* __restrict__ n_state,
                                   const float* __restrict__ m_state, const int* __restrict__ seq_slot,
                                   const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int dim, int vdim,
                                   int piece, int pieces) {
  const int s = blockIdx.x, h = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  const int values = dim * vdim + dim;
  const int slot = seq_slot[s];
  if (slot < 0 || e >= values) return;
  const int seq_n = cu_new[s + 1] - cu_new[s];
  const bool carried = seq_start[s] > 0;
  float cur = 0.f, m = 0.f;
  if (carried) {
    cur = e < dim * vdim ? S_state[((size_t)slot * heads + h) * dim * vdim + e] : n_state[((size_t)slot * heads + h) * dim + e - dim * vdim];
    m = m_state[(size_t)slot * heads + h];
  }
  for (int p = 0; p < pieces && p * piece < seq_n; ++p) {
    float* mine = scratch + (((size_t)s * pieces + p) * heads + h) * ((size_t)values + 3);
    const float m_loc = mine[values], F = mine[values + 1];
    const float m_new = fmaxf(F + m, m_loc);
    const float next = expf(F + m - m_new) * cur + expf(m_loc - m_new) * mine[e];
    mine[e] = cur;
    if (e == 0) mine[values + 2] = m;
    cur = next;
    m = m_new;
  }
}

template <typename T, int DMAX>
cudaError_t launch_scan(const void* qkv, long long stride, int q_col, int k_col, int v_col, const float* gates, float* S, float* n,
                        float* m, float* out, const int* seq_slot, const int* seq_start, const int* cu_new, int n_seqs, int heads,
                        int dim, int vdim, float floor_, int piece, int pieces, float* scratch, cudaStream_t stream) {
  // columns a block (a multiple of 8: whole warps of column lanes): all of a head's where they are few, so that the
  // normaliser is walked once
  const int cols = vdim <= 64 ? (vdim + 7) / 8 * 8 : 64;
  const int tiles = (vdim + cols - 1) / cols;
  const size_t smem = (size_t)(2 * kStage * DMAX + kStage * cols + 3 * kStage) * sizeof(float);
  auto kernel = mlstm_scan_kernel<T, DMAX>;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  cudaError_t e = cudaSuccess;
  for (int phase = pieces > 1 ? 1 : 0; phase <= (pieces > 1 ? 2 : 0) && e == cudaSuccess; ++phase) {
    e = launch_plain(kernel, dim3(n_seqs * pieces, heads, tiles), dim3(kSplit * cols + 32), smem, stream, (const T*)qkv, stride, q_col, k_col,
                     v_col, gates, S, n, m, out, seq_slot, seq_start, cu_new, heads, dim, vdim, floor_, piece, pieces, phase, scratch);
    if (phase == 1 && e == cudaSuccess) {
      const int values = dim * vdim + dim;
      e = launch_plain(mlstm_carry_kernel, dim3(n_seqs, heads, (values + 255) / 256), dim3(256), 0, stream, scratch,
                       (const float*)S, (const float*)n, (const float*)m, seq_slot, seq_start, cu_new, heads, dim, vdim, piece,
                       pieces);
    }
  }
  return e;
}

template <typename T>
cudaError_t launch_scan_any(int dim, const void* qkv, long long stride, int q_col, int k_col, int v_col, const float* gates, float* S,
                            float* n, float* m, float* out, const int* seq_slot, const int* seq_start, const int* cu_new,
                            int n_seqs, int heads, int vdim, float floor_, int piece, int pieces, float* scratch,
                            cudaStream_t stream) {
#define EMBER_SCAN(D)                                                                                                            \
  launch_scan<T, D>(qkv, stride, q_col, k_col, v_col, gates, S, n, m, out, seq_slot, seq_start, cu_new, n_seqs, heads, dim, vdim, \
                    floor_, piece, pieces, scratch, stream)
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
  const dim3 grid(T, (2 * heads + 3) / 4);      // four warps a block, a row each
  if (dtype == EMBER_F32)
    e = launch_plain(mlstm_gates_kernel<float>, grid, dim3(128), 0, stream, (const float*)h, (const float*)w, bias, gates, heads,
                     width, cap);
  else if (dtype == EMBER_BF16)
    e = launch_plain(mlstm_gates_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)h,
                     (const __nv_bfloat16*)w, bias, gates, heads, width, cap);
  else
    return ember_fail("mlstm_gates: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("mlstm_gates: %s", cudaGetErrorString(e));
  return 0;
}

// qkv: rows of `stride` values holding q (heads x dim) from q_col, k from k_col, v (heads x vdim) from v_col; gates as
// ember_mlstm_gates leaves them; S [slots, heads, dim, vdim], n [slots, heads, dim], m [slots, heads] float32 (advanced);
// out float32 [T, heads * vdim].  pieces 1: one walk of every sequence; more (with scratch of ember_mlstm_scan_scratch floats):
// pieces of `piece` tokens side by side.
EMBER_API size_t ember_mlstm_scan_scratch(int n_seqs, int pieces, int heads, int dim, int vdim) {
  return (size_t)n_seqs * pieces * heads * ((size_t)dim * vdim + dim + 3);
}

EMBER_API int ember_mlstm_scan(const void* qkv, long long stride, int q_col, int k_col, int v_col, const float* gates, float* S,
                               float* n, float* m, float* out, const int* seq_slot, const int* seq_start, const int* cu_new,
                               int n_seqs, int heads, int dim, int vdim, float floor_, int piece, int pieces, float* scratch,
                               int dtype, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && vdim > 0 && piece >= 1 && pieces >= 1, "mlstm_scan: bad sizes");
  EMBER_CHECK(pieces == 1 || scratch != nullptr, "mlstm_scan: pieces side by side need scratch");
  EMBER_CHECK((long long)n_seqs * pieces <= 2147483647LL, "mlstm_scan: %d sequences x %d pieces exceed one launch", n_seqs, pieces);
  EMBER_CHECK(dim >= 1 && dim <= 256, "mlstm_scan: a key size of %d is not in [1, 256]", dim);
  EMBER_CHECK(heads <= 65535, "mlstm_scan: %d heads exceed one launch", heads);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_scan_any<float>(dim, qkv, stride, q_col, k_col, v_col, gates, S, n, m, out, seq_slot, seq_start, cu_new, n_seqs,
                               heads, vdim, floor_, piece, pieces, scratch, stream);
  else if (dtype == EMBER_BF16)
    e = launch_scan_any<__nv_bfloat16>(dim, qkv, stride, q_col, k_col, v_col, gates, S, n, m, out, seq_slot, seq_start, cu_new,
                                       n_seqs, heads, vdim, floor_, piece, pieces, scratch, stream);
  else
    return ember_fail("mlstm_scan: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("mlstm_scan: %s", cudaGetErrorString(e));
  return 0;
}
