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
// A block owns up to 64 value columns of one (sequence, head); 4 to 16 neighbouring lanes share a column, each with
// its part of the column's rows of S in registers (the 16-byte parts s, s + SUB, ... of a key row, so that the lanes'
// shared-memory reads lie side by side) through all of the sequence's tokens of the step; what a token needs of all
// rows (u^T S, S^T q) the lanes add up by shuffles.  The walk is a chain of dependent steps, so what makes it fast is
// many warps an SM with few rows each (up to 1,024 threads a block, 4 to 16 rows a lane).  q, k, the decays (and the
// unit key and a * u) of a stage of tokens are made once in shared memory by all threads together, rows padded with
// zeros to 16, 32, 64, 128 or 256.  A
// token's arithmetic does not depend on where a stage or a step begins, so a sequence's outputs are the same bits
// however it is cut into steps.  A sequence that starts at position 0 starts from zeros whatever its state rows
// hold; padding sequences (slot -1) are skipped.
//
// A sequence that brings many tokens is cut into pieces of kPiece tokens that are walked side by side.  Both rules are
// linear in the state, S_end = M S_start + S_local, with M the product of the piece's transitions (diag(alpha_t), or
// diag(w_t) - (a_t u_t) u_t^T): the first walk starts every piece from zeros and leaves S_local, and walks beside the
// value columns a few more whose start is not zero and whose tokens write nothing, which leaves M (one column of ones
// for the diagonal rule, the unit matrix's columns for the delta rule); a carry kernel makes every piece's start state
// in order, and the slot's new state; the second walk starts every piece from its start state and makes the outputs.
// That re-orders the sums (linearly) for sequences of kPiecesFrom tokens and more; lanes per column are few there
// (four), since many blocks an SM hide the chain's latency.
#include "common.cuh"

namespace {

constexpr int kColumns = 64;       // value columns a block, at most
constexpr int kStageBytes = 40 * 1024;
constexpr int kPiece = 128;        // tokens of a piece
enum : int { kWhole = 0, kLocal = 1, kFromStart = 2 };   // what a walk begins with and leaves

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }
template <int SUB>
__device__ __forceinline__ float sum_of_column(float v) {     // over the SUB lanes of a column
#pragma unroll
  for (int off = 1; off < SUB; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

enum : int { kRuleGla = 0, kRuleDelta = 1 };

// SUB: lanes that share a column; R: rows of S a lane keeps (the padded key size is SUB * R); register r = 4 g + e is
// row 4 (sub + SUB g) + e
template <typename T, int RULE, int R, int SUB>
__global__ void __launch_bounds__(kColumns * SUB, (SUB == 4 && R <= 32) ? 2 : 1)     // (pieces: two blocks an SM at least)
recurrence_kernel(const T* __restrict__ proj, long long stride, int q_col, int k_col, int v_col, int a_col,
                  const float* __restrict__ a_bias, const float* __restrict__ z, float coef, float unit_eps,
                  float* __restrict__ state, float* __restrict__ out, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int D, int V, int Dp,
                  int stage, int mode, int pieces, int extra, float* __restrict__ local_states,
                  const float* __restrict__ start_states) {
  extern __shared__ __align__(16) float sm[];
  const int n_arrays = RULE == kRuleDelta ? 5 : 3;
  float* qs = sm;                    // [stage][Dp]
  float* ks = qs + stage * Dp;
  float* ds = ks + stage * Dp;       // the decay of every key channel
  float* us = ds + stage * Dp;       // the unit key (delta rule)
  float* as = us + stage * Dp;       // rate, then rate * unit key
  float* vs = sm + n_arrays * stage * Dp;   // [stage][columns of the block]
  // grid.x: sequences, or (sequence, piece) pairs; the walk's tokens are the sequence's new ones or the piece's
  const int s = blockIdx.x / pieces, piece = blockIdx.x % pieces, h = blockIdx.y, tid = threadIdx.x, n_threads = blockDim.x;
  constexpr int kSub = SUB;
  const int BV = n_threads / kSub, local = tid / kSub, sub = tid % kSub;
  const int j = blockIdx.z * BV + local;
  const int first = mode == kWhole ? 0 : piece * kPiece;
  const int n_all = cu_new[s + 1] - cu_new[s];
  const int t0 = cu_new[s] + first, n = mode == kWhole ? n_all : min(kPiece, n_all - first);
  if (n <= 0) return;
  const int Vx = V + extra;               // value columns and, in the first walk of pieces, the transition's
  const bool col = j < V, more = j >= V && j < Vx;
  const size_t out_width = (size_t)heads * V;
  const int slot = seq_slot[s];
  if (slot < 0) {
    if (col && sub == 0 && mode != kLocal)
      for (int i = 0; i < n; ++i) out[(size_t)(t0 + i) * out_width + (size_t)h * V + j] = 0.f;
    return;
  }
  float S[R];
  float* st = state + (((size_t)slot * heads + h) * D) * V + j;
  const bool carried = seq_start[s] > 0;
  const size_t piece_row = ((size_t)s * pieces + piece) * heads + h;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = 4 * (sub + kSub * (r / 4)) + r % 4;
    float v0 = 0.f;
    if (mode == kWhole) v0 = (d < D && col && carried) ? st[(size_t)d * V] : 0.f;
    else if (mode == kFromStart) v0 = (d < D && col) ? start_states[(piece_row * D + d) * V + j] : 0.f;
    else if (more && d < D) v0 = (RULE == kRuleGla || d == j - V) ? 1.f : 0.f;     // ones, or a column of the unit matrix
    S[r] = v0;
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
#pragma unroll 2
    for (int i = 0; i < ns; ++i) {
      const float v = vs[i * BV + local];
      const float4* q4 = reinterpret_cast<const float4*>(qs + i * Dp) + sub;
      const float4* k4 = reinterpret_cast<const float4*>(ks + i * Dp) + sub;
      const float4* d4 = reinterpret_cast<const float4*>(ds + i * Dp) + sub;
      float o0 = 0.f, o1 = 0.f;
      if (mode == kLocal) {      // the first walk of pieces wants the states alone: no read-out
        if (RULE == kRuleGla) {
#pragma unroll
          for (int g = 0; g < R / 4; ++g) {
            const float4 kk = k4[kSub * g], dd = d4[kSub * g];
            S[4 * g + 0] = fmaf(dd.x, S[4 * g + 0], kk.x * v);
            S[4 * g + 1] = fmaf(dd.y, S[4 * g + 1], kk.y * v);
            S[4 * g + 2] = fmaf(dd.z, S[4 * g + 2], kk.z * v);
            S[4 * g + 3] = fmaf(dd.w, S[4 * g + 3], kk.w * v);
          }
        } else {
          const float4* u4 = reinterpret_cast<const float4*>(us + i * Dp) + sub;
          const float4* a4 = reinterpret_cast<const float4*>(as + i * Dp) + sub;
          float p0 = 0.f, p1 = 0.f;
#pragma unroll
          for (int g = 0; g < R / 4; ++g) {
            const float4 uu = u4[kSub * g];
            p0 = fmaf(uu.x, S[4 * g + 0], p0);
            p1 = fmaf(uu.y, S[4 * g + 1], p1);
            p0 = fmaf(uu.z, S[4 * g + 2], p0);
            p1 = fmaf(uu.w, S[4 * g + 3], p1);
          }
          const float uS = sum_of_column<SUB>(p0 + p1);
#pragma unroll
          for (int g = 0; g < R / 4; ++g) {
            const float4 kk = k4[kSub * g], dd = d4[kSub * g], aa = a4[kSub * g];
            S[4 * g + 0] = fmaf(dd.x, S[4 * g + 0], fmaf(-aa.x, uS, kk.x * v));
            S[4 * g + 1] = fmaf(dd.y, S[4 * g + 1], fmaf(-aa.y, uS, kk.y * v));
            S[4 * g + 2] = fmaf(dd.z, S[4 * g + 2], fmaf(-aa.z, uS, kk.z * v));
            S[4 * g + 3] = fmaf(dd.w, S[4 * g + 3], fmaf(-aa.w, uS, kk.w * v));
          }
        }
        continue;
      }
      if (RULE == kRuleGla) {
#pragma unroll
        for (int g = 0; g < R / 4; ++g) {
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
        for (int g = 0; g < R / 4; ++g) {
            const float4 uu = u4[kSub * g];
            p0 = fmaf(uu.x, S[4 * g + 0], p0);
            p1 = fmaf(uu.y, S[4 * g + 1], p1);
            p0 = fmaf(uu.z, S[4 * g + 2], p0);
            p1 = fmaf(uu.w, S[4 * g + 3], p1);
          }
        const float uS = sum_of_column<SUB>(p0 + p1);
#pragma unroll
        for (int g = 0; g < R / 4; ++g) {
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
      const float o = sum_of_column<SUB>(o0 + o1);
      if (col && sub == 0 && mode != kLocal) out[(size_t)(t0 + i0 + i) * out_width + (size_t)h * V + j] = o;
    }
  }
  if (mode == kWhole && col) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = 4 * (sub + kSub * (r / 4)) + r % 4;
      if (d < D) st[(size_t)d * V] = S[r];
    }
  }
  if (mode == kLocal && (col || more)) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = 4 * (sub + kSub * (r / 4)) + r % 4;
      if (d < D) local_states[(piece_row * D + d) * Vx + j] = S[r];
    }
  }
}

// The pieces' start states in order: start_0 = the slot's state (zeros at position 0), start_(p+1) = M_p start_p +
// local_p; the last one is the slot's new state.  M_p lies behind local_p's value columns: one column (the diagonal
// rule's products of decays) or `D` columns.
//
// The diagonal rule: grid (sequences, heads, tiles of 256 state values), a thread a state value.
__global__ void __launch_bounds__(256)
carry_diagonal_kernel(const float* __restrict__ local_states, float* __restrict__ start_states, float* __restrict__ state,
                      const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ cu_new,
                      int heads, int D, int V, int pieces) {
  const int s = blockIdx.x, h = blockIdx.y, at = blockIdx.z * blockDim.x + threadIdx.x;
  const int slot = seq_slot[s];
  const int n = cu_new[s + 1] - cu_new[s];
  if (slot < 0 || n <= 0 || at >= D * V) return;
  const int d = at / V, j = at % V;
  const int n_pieces = (n + kPiece - 1) / kPiece, Vx = V + 1;
  float* st = state + (((size_t)slot * heads + h) * D + d) * V + j;
  float cur = seq_start[s] > 0 ? *st : 0.f;
  for (int p = 0; p < n_pieces; ++p) {
    const size_t row = (((size_t)s * pieces + p) * heads + h) * D + d;
    start_states[row * V + j] = cur;
    cur = fmaf(local_states[row * Vx + V], cur, local_states[row * Vx + j]);
  }
  *st = cur;
}

// The delta rule: grid (sequences, heads, tiles of kCarryColumns value columns), 256 threads: thread t keeps column
// t % kCarryColumns of the rows t / kCarryColumns + 16 k.  A piece's M comes through shared memory 32 of its columns at
// a time (rows padded against bank conflicts), the tile's current columns lie there transposed.
constexpr int kCarryColumns = 16;
constexpr int kCarryRows = 256 / kCarryColumns;     // rows that the threads cover at once

template <int NK>      // rows a thread: 16 NK covers the key size
__global__ void __launch_bounds__(256)
carry_matrix_kernel(const float* __restrict__ local_states, float* __restrict__ start_states, float* __restrict__ state,
                    const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ cu_new,
                    int heads, int D, int V, int pieces) {
  extern __shared__ __align__(16) float carry_sm[];
  float* cols = carry_sm;                          // [D][kCarryColumns]: the current columns, row e at cols[e * 16 ..]
  float* sM = carry_sm + D * kCarryColumns;        // [D][36]: 32 columns of M (rows start on 16 bytes, apart in the banks)
  const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int jj = tid % kCarryColumns, d0 = tid / kCarryColumns;
  const int j = blockIdx.z * kCarryColumns + jj;
  const int slot = seq_slot[s];
  const int n = cu_new[s + 1] - cu_new[s];
  if (slot < 0 || n <= 0) return;
  const int n_pieces = (n + kPiece - 1) / kPiece, Vx = V + D;
  float* st = state + (((size_t)slot * heads + h) * D) * V;
  const bool carried = seq_start[s] > 0;
  float cur[NK];                                   // rows d0 + 16 k
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int d = d0 + kCarryRows * k;
    cur[k] = (carried && d < D && j < V) ? st[(size_t)d * V + j] : 0.f;
  }
  for (int p = 0; p < n_pieces; ++p) {
    const size_t row0 = (((size_t)s * pieces + p) * heads + h) * D;
    __syncthreads();      // the piece before has read the columns
#pragma unroll
    for (int k = 0; k < NK; ++k) {
      const int d = d0 + kCarryRows * k;
      if (d < D) {
        cols[d * kCarryColumns + jj] = cur[k];
        if (j < V) start_states[(row0 + d) * V + j] = cur[k];
      }
    }
    float acc[NK];
#pragma unroll
    for (int k = 0; k < NK; ++k) acc[k] = 0.f;
    for (int e0 = 0; e0 < D; e0 += 32) {
      __syncthreads();    // the columns are written; the chunk before has been used
      for (int idx = tid; idx < D * 32; idx += 256) {
        const int d = idx / 32, e = idx % 32;
        sM[d * 36 + e] = e0 + e < D ? local_states[(row0 + d) * Vx + V + e0 + e] : 0.f;
      }
      __syncthreads();
      for (int e = 0; e < 32; e += 4) {          // (columns past D are zeros in sM; the current columns there are read as 0)
        float c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) c[i] = e0 + e + i < D ? cols[(e0 + e + i) * kCarryColumns + jj] : 0.f;
#pragma unroll
        for (int k = 0; k < NK; ++k) {
          const int d = d0 + kCarryRows * k;
          if (d < D) {
            const float4 m = *reinterpret_cast<const float4*>(sM + d * 36 + e);
            acc[k] = fmaf(m.x, c[0], acc[k]);
            acc[k] = fmaf(m.y, c[1], acc[k]);
            acc[k] = fmaf(m.z, c[2], acc[k]);
            acc[k] = fmaf(m.w, c[3], acc[k]);
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < NK; ++k) {
      const int d = d0 + kCarryRows * k;
      cur[k] = (d < D && j < V) ? acc[k] + local_states[(row0 + d) * Vx + j] : 0.f;
    }
  }
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int d = d0 + kCarryRows * k;
    if (d < D && j < V) st[(size_t)d * V + j] = cur[k];
  }
}

inline int padded_rows(int D) { return D <= 16 ? 16 : D <= 32 ? 32 : D <= 64 ? 64 : D <= 128 ? 128 : 256; }

template <typename T, int RULE>
int launch_walk(int mode, int pieces, const void* proj, long long stride, int q_col, int k_col, int v_col, int a_col,
                const float* a_bias, const float* z, float coef, float unit_eps, float* state, float* out, const int* seq_slot,
                const int* seq_start, const int* cu_new, int n_seqs, int heads, int D, int V, float* local_states,
                float* start_states, cudaStream_t stream, const char* name) {
  const int extra = mode == kLocal ? (RULE == kRuleGla ? 1 : D) : 0;
  const int Vx = V + extra;
  const int BV = Vx <= 8 ? 8 : Vx <= 16 ? 16 : Vx <= 32 ? 32 : kColumns;     // (a block is whole warps: 8 columns x 4 lanes at least)
  const int Dp = padded_rows(D);
  // pieces: many blocks an SM, so four lanes a column (the fewest shuffles and instructions in all; eight lanes with half
  // the rows each measured slower: 0.88 against 0.71 ms a layer of gated linear attention at keys of 128)
  const int lanes = mode != kWhole || Dp <= 16 ? 4 : Dp <= 32 ? 8 : 16;
  const int n_arrays = RULE == kRuleDelta ? 5 : 3;
  const int per_token = (n_arrays * Dp + BV) * (int)sizeof(float);
  const int stage = max(1, min(16, kStageBytes / per_token));
  const size_t smem = (size_t)stage * per_token;
  const dim3 grid(n_seqs * pieces, heads, (Vx + BV - 1) / BV);
  cudaError_t e;
#define EMBER_RECURRENCE(R, SUB)                                                                                              \
  e = launch_plain(recurrence_kernel<T, RULE, R, SUB>, grid, dim3(BV * lanes), smem, stream, (const T*)proj, stride, q_col, \
                   k_col, v_col, a_col, a_bias, z, coef, unit_eps, state, out, seq_slot, seq_start, cu_new, heads, D, V, Dp, \
                   stage, mode, pieces, extra, local_states, (const float*)start_states)
  if (lanes == 4) {
    if (Dp <= 16) EMBER_RECURRENCE(4, 4);
    else if (Dp <= 32) EMBER_RECURRENCE(8, 4);
    else if (Dp <= 64) EMBER_RECURRENCE(16, 4);
    else if (Dp <= 128) EMBER_RECURRENCE(32, 4);
    else EMBER_RECURRENCE(64, 4);
  } else if (Dp <= 32) EMBER_RECURRENCE(4, 8);
  else if (Dp <= 64) EMBER_RECURRENCE(4, 16);
  else if (Dp <= 128) EMBER_RECURRENCE(8, 16);
  else EMBER_RECURRENCE(16, 16);
#undef EMBER_RECURRENCE
  if (e != cudaSuccess) return ember_fail("%s: %s", name, cudaGetErrorString(e));
  return 0;
}

// Floats of scratch that a walk in pieces needs: every piece's local state with its transition, and its start state.
inline size_t pieces_scratch(int rule, int n_seqs, int pieces, int heads, int D, int V) {
  const size_t rows = (size_t)n_seqs * pieces * heads * D;
  return rows * (V + (rule == kRuleGla ? 1 : D)) + rows * V;
}

// pieces 0: one walk a sequence.  pieces > 0: ceil(most new tokens / kPiece); scratch of pieces_scratch floats.
template <typename T, int RULE>
int launch_recurrence(const void* proj, long long stride, int q_col, int k_col, int v_col, int a_col, const float* a_bias,
                      const float* z, float coef, float unit_eps, float* state, float* out, const int* seq_slot,
                      const int* seq_start, const int* cu_new, int n_seqs, int heads, int D, int V, int pieces, float* scratch,
                      cudaStream_t stream, const char* name) {
  if (pieces <= 0)
    return launch_walk<T, RULE>(kWhole, 1, proj, stride, q_col, k_col, v_col, a_col, a_bias, z, coef, unit_eps, state, out, seq_slot,
                                seq_start, cu_new, n_seqs, heads, D, V, nullptr, nullptr, stream, name);
  EMBER_CHECK(scratch != nullptr, "%s: a walk in pieces needs scratch", name);
  float* local_states = scratch;
  float* start_states = scratch + (size_t)n_seqs * pieces * heads * D * (V + (RULE == kRuleGla ? 1 : D));
  int rc = launch_walk<T, RULE>(kLocal, pieces, proj, stride, q_col, k_col, v_col, a_col, a_bias, z, coef, unit_eps, state, out,
                                seq_slot, seq_start, cu_new, n_seqs, heads, D, V, local_states, start_states, stream, name);
  if (rc) return rc;
  cudaError_t e;
  if (RULE == kRuleGla)
    e = launch_plain(carry_diagonal_kernel, dim3(n_seqs, heads, (D * V + 255) / 256), dim3(256), 0, stream,
                     (const float*)local_states, start_states, state, seq_slot, seq_start, cu_new, heads, D, V, pieces);
  else {
    const size_t smem = (size_t)D * (kCarryColumns + 36) * sizeof(float);
    const dim3 grid(n_seqs, heads, (V + kCarryColumns - 1) / kCarryColumns);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(carry_matrix_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return ember_fail("%s (carry): shared memory for a key size of %d", name, D);
    if (D <= 64)
      e = launch_plain(carry_matrix_kernel<4>, grid, dim3(256), smem, stream, (const float*)local_states, start_states, state,
                       seq_slot, seq_start, cu_new, heads, D, V, pieces);
    else if (D <= 128)
      e = launch_plain(carry_matrix_kernel<8>, grid, dim3(256), smem, stream, (const float*)local_states, start_states, state,
                       seq_slot, seq_start, cu_new, heads, D, V, pieces);
    else
      e = launch_plain(carry_matrix_kernel<16>, grid, dim3(256), smem, stream, (const float*)local_states, start_states, state,
                       seq_slot, seq_start, cu_new, heads, D, V, pieces);
  }
  if (e != cudaSuccess) return ember_fail("%s (carry): %s", name, cudaGetErrorString(e));
  return launch_walk<T, RULE>(kFromStart, pieces, proj, stride, q_col, k_col, v_col, a_col, a_bias, z, coef, unit_eps, state, out,
                              seq_slot, seq_start, cu_new, n_seqs, heads, D, V, local_states, start_states, stream, name);
}

// grid (ceil(T / kLowRankTokens), tiles of 128 outputs): lr = `rank` columns from `col` of a row of `in`; w2t is the
// second matrix transposed, [rank, n_out], so that a warp's outputs lie side by side in every row of it; a block
// takes kLowRankTokens tokens through each weight it reads.
constexpr int kLowRankTokens = 8;

template <typename T>
__global__ void __launch_bounds__(128)
low_rank_out_kernel(const T* __restrict__ in, long long stride, int col, int rank, const float* __restrict__ w2t,
                    const float* __restrict__ bias, float* __restrict__ out, int T_tokens, int n_out, int act) {
  extern __shared__ float lr[];      // [kLowRankTokens][rank]
  const int t0 = blockIdx.x * kLowRankTokens, nt = min(kLowRankTokens, T_tokens - t0);
  for (int i = threadIdx.x; i < nt * rank; i += blockDim.x) {
    const float v = to_float(in[(size_t)(t0 + i / rank) * stride + col + i % rank]);
    lr[i] = act ? tanhf(v) : v;
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= n_out) return;
  float acc[kLowRankTokens];
#pragma unroll
  for (int k = 0; k < kLowRankTokens; ++k) acc[k] = 0.f;
  for (int r = 0; r < rank; ++r) {
    const float w = w2t[(size_t)r * n_out + c];
#pragma unroll
    for (int k = 0; k < kLowRankTokens; ++k)
      if (k < nt) acc[k] = fmaf(lr[k * rank + r], w, acc[k]);
  }
  const float b = bias[c];
#pragma unroll
  for (int k = 0; k < kLowRankTokens; ++k)
    if (k < nt) out[(size_t)(t0 + k) * n_out + c] = acc[k] + b;
}

}  // namespace

// in [T, *] (dtype, row stride in elements), w2t float32 [rank, n_out] (the second matrix transposed), bias float32
// [n_out], out float32 [T, n_out]; act: 0 none, 1 tanh on the low-rank values.  A token's sums run over the rank in order.
EMBER_API int ember_low_rank_out(const void* in, long long stride, int col, int rank, const float* w2, const float* bias,
                                 float* out, int T, int n_out, int act, int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_out > 0 && rank >= 1 && rank <= 256, "low_rank_out: %d rows, %d outputs, rank %d (at most 256)", T, n_out, rank);
  EMBER_CHECK(act == 0 || act == 1, "low_rank_out: activation %d", act);
  cudaError_t e;
  const dim3 grid((T + kLowRankTokens - 1) / kLowRankTokens, (n_out + 127) / 128);
  const size_t smem = (size_t)kLowRankTokens * rank * sizeof(float);
  EMBER_CHECK(grid.y <= 65535, "low_rank_out: %d outputs exceed one launch", n_out);
  if (dtype == EMBER_F32)
    e = launch_plain(low_rank_out_kernel<float>, grid, dim3(128), smem, stream, (const float*)in, stride, col, rank, w2, bias, out, T,
                     n_out, act);
  else if (dtype == EMBER_BF16)
    e = launch_plain(low_rank_out_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)in, stride, col, rank, w2,
                     bias, out, T, n_out, act);
  else
    return ember_fail("low_rank_out: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("low_rank_out: %s", cudaGetErrorString(e));
  return 0;
}

// proj [T, *] (dtype): q, k of heads x dim from q_col, k_col, v of heads x vdim from v_col; z float32 [T, heads * dim];
// state float32 [slots, heads, dim, vdim]; out float32 [T, heads * vdim].
EMBER_API int ember_recurrence_piece(void) { return kPiece; }
// rule 0: gated linear attention, 1: the generalized delta rule
EMBER_API size_t ember_recurrence_scratch(int rule, int n_seqs, int pieces, int heads, int dim, int vdim) {
  return pieces_scratch(rule, n_seqs, pieces, heads, dim, vdim);
}

// pieces 0: every sequence in one walk; else the count of pieces of ember_recurrence_piece() tokens that the longest
// sequence's new tokens make, and scratch of ember_recurrence_scratch(...) floats.
EMBER_API int ember_gla_scan(const void* proj, long long stride, int q_col, int k_col, int v_col, const float* z, float tau,
                             float* state, float* out, const int* seq_slot, const int* seq_start, const int* cu_new,
                             int n_seqs, int heads, int dim, int vdim, int pieces, float* scratch, int dtype,
                             cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && heads <= 65535 && dim >= 1 && dim <= 256 && vdim >= 1,
              "gla_scan: %d sequences, %d heads of %d x %d (key size at most 256)", n_seqs, heads, dim, vdim);
  EMBER_CHECK(tau > 0.f, "gla_scan: tau %g", (double)tau);
  if (dtype == EMBER_F32)
    return launch_recurrence<float, kRuleGla>(proj, stride, q_col, k_col, v_col, 0, nullptr, z, 1.0f / tau, 0.f, state, out,
                                              seq_slot, seq_start, cu_new, n_seqs, heads, dim, vdim, pieces, scratch, stream, "gla_scan");
  if (dtype == EMBER_BF16)
    return launch_recurrence<__nv_bfloat16, kRuleGla>(proj, stride, q_col, k_col, v_col, 0, nullptr, z, 1.0f / tau, 0.f, state,
                                                      out, seq_slot, seq_start, cu_new, n_seqs, heads, dim, vdim, pieces, scratch,
                                                      stream, "gla_scan");
  return ember_fail("gla_scan: element type %d", dtype);
}

// proj [T, *] (dtype): r, k, v, a_in of heads x dim from their columns; a_bias float32 [heads * dim]; z float32
// [T, heads * dim] (the decay's logits); state float32 [slots, heads, dim, dim]; out float32 [T, heads * dim].
EMBER_API int ember_generalized_delta_rule(const void* proj, long long stride, int r_col, int k_col, int v_col, int a_col,
                                           const float* a_bias, const float* z, float decay_coef, float unit_eps,
                                           float* state, float* out, const int* seq_slot, const int* seq_start,
                                           const int* cu_new, int n_seqs, int heads, int dim, int pieces, float* scratch,
                                           int dtype, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && heads <= 65535 && dim >= 1 && dim <= 256,
              "generalized_delta_rule: %d sequences, %d heads of %d (at most 256)", n_seqs, heads, dim);
  if (dtype == EMBER_F32)
    return launch_recurrence<float, kRuleDelta>(proj, stride, r_col, k_col, v_col, a_col, a_bias, z, decay_coef, unit_eps,
                                                state, out, seq_slot, seq_start, cu_new, n_seqs, heads, dim, dim, pieces, scratch,
                                                stream, "generalized_delta_rule");
  if (dtype == EMBER_BF16)
    return launch_recurrence<__nv_bfloat16, kRuleDelta>(proj, stride, r_col, k_col, v_col, a_col, a_bias, z, decay_coef,
                                                        unit_eps, state, out, seq_slot, seq_start, cu_new, n_seqs, heads,
                                                        dim, dim, pieces, scratch, stream, "generalized_delta_rule");
  return ember_fail("generalized_delta_rule: element type %d", dtype);
}
