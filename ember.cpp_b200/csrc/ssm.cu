// Mamba-2's two sequence operations over a step's packed tokens: the short causal convolution with
// its silu, and the recurrence S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t.
//
// A step holds the new tokens of several sequences back to back (cu_new gives each sequence's
// first row); what a sequence carries from earlier steps lies in per-slot state rows: the last
// taps - 1 rows that entered the convolution, and S of every head.  A sequence that starts at
// position 0 starts from zeros whatever its slot's rows hold.  Sequences of slot -1 are padding:
// their rows are set to zero and no state is touched.
//
// Step sizes, decays, the recurrence and the state are float32 in every mode; x, B and C come in
// the step's element type (the convolution's output).  A token's result depends on its sequence
// alone: every sum is made in an order that sizes fix, not the batch or the step's cut.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
// what follows the convolution's sum: silu (act 0) or nothing (act 1)
__device__ __forceinline__ float conv_act(float v, int act) { return act == 0 ? silu_f(v) : v; }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ---------------------------------------------------------------------------- convolution
// A thread takes one channel through a run of 32 tokens of one sequence, the last taps - 1 inputs in registers;
// grid (sequences * runs, channel tiles).  in: `channels` columns from col0 of a matrix with row stride in_stride.
// w [channels, taps] (the last tap is the current token's), bias [channels].  state [slots, taps - 1, channels]:
// the rows before the step's first, oldest first.  The sum starts from the bias and takes the taps oldest first,
// as the one-token kernel below does.
constexpr int kConvRun = 32;

template <typename T, int TMAX>
__global__ void conv_silu_kernel(const T* __restrict__ in, long long in_stride, int col0, int channels, int taps,
                                 const float* __restrict__ w, const float* __restrict__ bias,
                                 const float* __restrict__ state, T* __restrict__ out, const int* __restrict__ seq_slot,
                                 const int* __restrict__ seq_start, const int* __restrict__ cu_new, int runs, int act) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int s = blockIdx.x / runs, run = blockIdx.x % runs;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const int i0 = run * kConvRun, i1 = min(n, i0 + kConvRun);
  if (i0 >= n) return;
  const int slot = seq_slot[s];
  if (slot < 0) {
    for (int i = i0; i < i1; ++i) out[(size_t)(t0 + i) * channels + c] = from_float<T>(0.f);
    return;
  }
  const bool carried = seq_start[s] > 0;
  const float* st = state + (size_t)slot * (taps - 1) * channels + c;
  const T* src = in + (size_t)t0 * in_stride + col0 + c;
  // hist[TMAX - 1 - m]: the input m tokens back; wt: its tap, zero beyond the filter's length
  float hist[TMAX], wt[TMAX];
#pragma unroll
  for (int m = 0; m < TMAX; ++m) {
    wt[TMAX - 1 - m] = m < taps ? w[(size_t)c * taps + taps - 1 - m] : 0.f;
    float v = 0.f;
    if (m >= 1 && m < taps) {
      const int at = i0 - m;
      if (at >= 0)
        v = to_float(src[(size_t)at * in_stride]);
      else if (carried)
        v = st[(size_t)(taps - 1 + at) * channels];
    }
    hist[TMAX - 1 - m] = v;
  }
  const float b = bias[c];
#pragma unroll 8
  for (int i = i0; i < i1; ++i) {   // (unrolled: eight tokens' loads are on their way together)
    hist[TMAX - 1] = to_float(src[(size_t)i * in_stride]);
    float acc = b;
#pragma unroll
    for (int k = 0; k < TMAX; ++k) acc = fmaf(wt[k], hist[k], acc);
    out[(size_t)(t0 + i) * channels + c] = from_float<T>(conv_act(acc, act));
#pragma unroll
    for (int k = 0; k + 1 < TMAX; ++k) hist[k] = hist[k + 1];
  }
}

// The same with two neighbouring channels a thread (4- or 8-byte loads and stores: half the instructions for the
// same bytes), where the number of channels, the first column and the row stride are even.
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename T, int TMAX>
__global__ void conv_silu2_kernel(const T* __restrict__ in, long long in_stride, int col0, int channels, int taps,
                                  const float* __restrict__ w, const float* __restrict__ bias,
                                  const float* __restrict__ state, T* __restrict__ out, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_start, const int* __restrict__ cu_new, int runs, int act) {
  const int c = 2 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (c >= channels) return;
  const int s = blockIdx.x / runs, run = blockIdx.x % runs;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const int i0 = run * kConvRun, i1 = min(n, i0 + kConvRun);
  if (i0 >= n) return;
  const int slot = seq_slot[s];
  if (slot < 0) {
    for (int i = i0; i < i1; ++i) store2(out + (size_t)(t0 + i) * channels + c, 0.f, 0.f);
    return;
  }
  const bool carried = seq_start[s] > 0;
  const float* st = state + (size_t)slot * (taps - 1) * channels + c;
  const T* src = in + (size_t)t0 * in_stride + col0 + c;
  float2 hist[TMAX], wt[TMAX];
#pragma unroll
  for (int m = 0; m < TMAX; ++m) {
    wt[TMAX - 1 - m] = m < taps ? make_float2(w[(size_t)c * taps + taps - 1 - m], w[(size_t)(c + 1) * taps + taps - 1 - m])
                                : make_float2(0.f, 0.f);
    float2 v = make_float2(0.f, 0.f);
    if (m >= 1 && m < taps) {
      const int at = i0 - m;
      if (at >= 0)
        v = load2(src + (size_t)at * in_stride);
      else if (carried)
        v = load2(st + (size_t)(taps - 1 + at) * channels);
    }
    hist[TMAX - 1 - m] = v;
  }
  const float2 b = load2(bias + c);
#pragma unroll 8
  for (int i = i0; i < i1; ++i) {
    hist[TMAX - 1] = load2(src + (size_t)i * in_stride);
    float a0 = b.x, a1 = b.y;
#pragma unroll
    for (int k = 0; k < TMAX; ++k) {
      a0 = fmaf(wt[k].x, hist[k].x, a0);
      a1 = fmaf(wt[k].y, hist[k].y, a1);
    }
    store2(out + (size_t)(t0 + i) * channels + c, conv_act(a0, act), conv_act(a1, act));
#pragma unroll
    for (int k = 0; k + 1 < TMAX; ++k) hist[k] = hist[k + 1];
  }
}

// The state after the step: its row k is the input taps - 1 - k rows before the sequence's new end.
// One thread per (sequence, channel), rows in ascending order (row k is read from a later row only).
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ in, long long in_stride, int col0, int channels, int taps,
                                  float* __restrict__ state, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_start, const int* __restrict__ cu_new) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int s = blockIdx.x;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const bool carried = seq_start[s] > 0;
  float* st = state + (size_t)slot * (taps - 1) * channels + c;
  for (int k = 0; k < taps - 1; ++k) {
    const int src = n - (taps - 1) + k;
    float v = 0.f;
    if (src >= 0)
      v = to_float(in[(size_t)(t0 + src) * in_stride + col0 + c]);
    else if (carried && k + n < taps - 1)
      v = st[(size_t)(k + n) * channels];
    st[(size_t)k * channels] = v;
  }
}

// One token per sequence (token t is sequence t): the convolution and the state's shift in one launch.
template <typename T>
__global__ void conv_step_kernel(const T* __restrict__ in, long long in_stride, int col0, int channels, int taps,
                                 const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ state,
                                 T* __restrict__ out, const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int act) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int t = blockIdx.x;
  const int slot = seq_slot[t];
  T* o = out + (size_t)t * channels + c;
  if (slot < 0) {
    *o = from_float<T>(0.f);
    return;
  }
  const bool carried = seq_start[t] > 0;
  float* st = state + (size_t)slot * (taps - 1) * channels + c;
  const float cur = to_float(in[(size_t)t * in_stride + col0 + c]);
  float acc = bias[c];
  for (int j = 0; j < taps - 1; ++j) {
    const float v = carried ? st[(size_t)j * channels] : 0.f;
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
    if (j > 0) st[(size_t)(j - 1) * channels] = v;
  }
  acc = fmaf(w[(size_t)c * taps + taps - 1], cur, acc);
  if (taps > 1) st[(size_t)(taps - 2) * channels] = cur;
  *o = from_float<T>(conv_act(acc, act));
}

// ---------------------------------------------------------------------------- recurrence
constexpr int kLanes = 8;      // lanes that share a value channel: lane l holds the states n = l, l + 8, l + 16, ...
constexpr int kPer = 2;        // value channels a thread
constexpr int kChannels = 16 * kPer;  // value channels a block
constexpr int kScanThreads = 128;
constexpr int kSplit = 128;    // tokens of a piece when a long sequence is scanned in pieces

// How many tokens a block stages in shared memory at a time (B and C of N states each, padded to 8 R).
inline int scan_stage(int R) { return max(4, min(32, 4096 / (kLanes * R))); }

// Modes of the scan.  A short sequence (and a decode step) is one pass: kWhole.  A long one is cut into pieces
// of kSplit tokens that are scanned side by side: kLocal scans every piece from a state of zeros and leaves the
// piece's end state and the product of its decays in scratch; ssd_carry_kernel walks the pieces of a sequence
// in order and turns the scratch into every piece's true starting state (and the slot's state after the step);
// kFinal scans every piece again from there and writes y.  The recurrence is linear in the state, so this is
// the same sum in another order.
enum : int { kWhole = 0, kLocal = 1, kFinal = 2 };

// grid (ceil(vdim / 32), heads, sequences * pieces).  xbc [T, inner | groups*N | groups*N] (x, B, C), dt: `heads`
// columns from dt_col of a matrix with row stride dt_stride, state [slots, heads, vdim, N], y float32 [T, inner],
// piece_state [sequences * pieces, heads, vdim, N], piece_decay [sequences * pieces, heads].
// V values of T (16 bytes) as floats
template <typename T>
__device__ __forceinline__ void load16(const T* src, float* dst);
template <>
__device__ __forceinline__ void load16<float>(const float* src, float* dst) {
  const float4 v = *reinterpret_cast<const float4*>(src);
  dst[0] = v.x, dst[1] = v.y, dst[2] = v.z, dst[3] = v.w;
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* src, float* dst) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    dst[2 * i] = f.x, dst[2 * i + 1] = f.y;
  }
}

// VEC: the rows of x, B and C are brought in 16 bytes at a time (N a multiple of 8; inner, vdim and groups * N
// multiples of the 16-byte piece), else value by value.
template <typename T, int RMAX, bool VEC>
__global__ void __launch_bounds__(kScanThreads)
ssd_scan_kernel(const T* __restrict__ xbc, const T* __restrict__ dt_in, long long dt_stride, int dt_col,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ skip,
                float* __restrict__ state, float* __restrict__ y, const int* __restrict__ seq_slot,
                const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads, int vdim, int groups,
                int N, int stage, int mode, int pieces, float* __restrict__ piece_state, float* __restrict__ piece_decay) {
  extern __shared__ __align__(16) float sm[];
  const int R = (N + kLanes - 1) / kLanes;
  const int row = kLanes * R;          // padded length of a token's B (or C)
  float* sB = sm;                      // [stage][row]
  float* sC = sB + stage * row;        // [stage][row]
  float* sX = sC + stage * row;        // [stage][kChannels]
  float* sDt = sX + stage * kChannels;
  float* sA = sDt + stage;

  const int s = blockIdx.z / pieces, piece = blockIdx.z % pieces;
  const int h = blockIdx.y, p0 = blockIdx.x * kChannels;
  const int slot = seq_slot[s];
  int t0 = cu_new[s], t1 = cu_new[s + 1];
  const int inner = heads * vdim, gn = groups * N;
  const int pl = threadIdx.x / kLanes, nl = threadIdx.x % kLanes;
  const int p = p0 + pl * kPer;        // this thread's first value channel
  if (slot < 0) {
    if (mode != kLocal && piece == 0 && nl == 0)
      for (int t = t0; t < t1; ++t)
#pragma unroll
        for (int c = 0; c < kPer; ++c)
          if (p + c < vdim) y[(size_t)t * inner + h * vdim + p + c] = 0.f;
    return;
  }
  if (mode != kWhole) {
    t0 += piece * kSplit;
    t1 = min(t1, t0 + kSplit);
    if (t0 >= t1) return;
  }
  const int g = h / (heads / groups);
  const size_t xbc_stride = (size_t)inner + 2 * gn;
  const size_t at_piece = ((size_t)blockIdx.z * heads + h) * vdim;
  float S[kPer][RMAX];
  {
    const float* from = mode == kFinal ? piece_state + at_piece * N : state + ((size_t)slot * heads + h) * vdim * N;
    const bool have = mode == kFinal || (mode == kWhole && seq_start[s] > 0);
#pragma unroll
    for (int c = 0; c < kPer; ++c)
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        const int n = r * kLanes + nl;
        S[c][r] = (have && r < R && n < N && p + c < vdim) ? from[(size_t)(p + c) * N + n] : 0.f;
      }
  }
  const float A = -expf(a_log[h]), D = skip[h], bias = dt_bias[h];
  float decay = 1.f;

  for (int tc = t0; tc < t1; tc += stage) {
    const int cnt = min(stage, t1 - tc);
    __syncthreads();  // the tokens staged before have been used
    if constexpr (VEC) {
      constexpr int V = 16 / (int)sizeof(T);
      const int per_row = N / V;  // pieces of a token's B (and of its C); row == N here
#pragma unroll 4
      for (int e = threadIdx.x; e < cnt * 2 * per_row; e += kScanThreads) {
        const int tt = e / (2 * per_row), k = e % (2 * per_row);
        const int which = k / per_row, j = k % per_row;
        float v[V];
        load16<T>(xbc + (size_t)(tc + tt) * xbc_stride + inner + (size_t)which * gn + (size_t)g * N + j * V, v);
        float4* dst = reinterpret_cast<float4*>((which ? sC : sB) + tt * row + j * V);
#pragma unroll
        for (int i = 0; i < V / 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
      for (int e = threadIdx.x; e < cnt * (kChannels / V); e += kScanThreads) {
        const int tt = e / (kChannels / V), j = e % (kChannels / V);
        float v[V];
#pragma unroll
        for (int i = 0; i < V; ++i) v[i] = 0.f;
        if (p0 + j * V < vdim) load16<T>(xbc + (size_t)(tc + tt) * xbc_stride + h * vdim + p0 + j * V, v);
        float4* dst = reinterpret_cast<float4*>(sX + tt * kChannels + j * V);
#pragma unroll
        for (int i = 0; i < V / 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
    } else {
      for (int e = threadIdx.x; e < cnt * row; e += kScanThreads) {
        const int tt = e / row, n = e % row;
        const T* src = xbc + (size_t)(tc + tt) * xbc_stride + inner + (size_t)g * N + n;
        sB[e] = n < N ? to_float(src[0]) : 0.f;
        sC[e] = n < N ? to_float(src[gn]) : 0.f;
      }
      for (int e = threadIdx.x; e < cnt * kChannels; e += kScanThreads) {
        const int tt = e / kChannels, pp = e % kChannels;
        sX[e] = p0 + pp < vdim ? to_float(xbc[(size_t)(tc + tt) * xbc_stride + h * vdim + p0 + pp]) : 0.f;
      }
    }
    if ((int)threadIdx.x < cnt) {
      const float dt = softplus_f(to_float(dt_in[(size_t)(tc + threadIdx.x) * dt_stride + dt_col + h]) + bias);
      sDt[threadIdx.x] = dt;
      sA[threadIdx.x] = expf(A * dt);
    }
    __syncthreads();
    for (int tt = 0; tt < cnt; ++tt) {
      const float a = sA[tt], dt = sDt[tt];
      decay *= a;
      float xv[kPer], dtx[kPer], acc[kPer][2];
#pragma unroll
      for (int c = 0; c < kPer; ++c) {
        xv[c] = sX[tt * kChannels + pl * kPer + c];
        dtx[c] = dt * xv[c];
        acc[c][0] = acc[c][1] = 0.f;
      }
      const float* B = sB + tt * row + nl;
      const float* C = sC + tt * row + nl;
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        if (r < R) {
          const float b = B[r * kLanes], cc = C[r * kLanes];
#pragma unroll
          for (int c = 0; c < kPer; ++c) {
            S[c][r] = fmaf(a, S[c][r], dtx[c] * b);
            acc[c][r & 1] = fmaf(S[c][r], cc, acc[c][r & 1]);
          }
        }
      }
      if (mode != kLocal) {
#pragma unroll
        for (int c = 0; c < kPer; ++c) {
          float v = acc[c][0] + acc[c][1];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          if (nl == 0 && p + c < vdim) y[(size_t)(tc + tt) * inner + h * vdim + p + c] = fmaf(D, xv[c], v);
        }
      }
    }
  }
  if (mode == kFinal) return;  // (the carry kernel has written the slot's state)
  float* to = mode == kLocal ? piece_state + at_piece * N : state + ((size_t)slot * heads + h) * vdim * N;
#pragma unroll
  for (int c = 0; c < kPer; ++c)
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      const int n = r * kLanes + nl;
      if (r < R && n < N && p + c < vdim) to[(size_t)(p + c) * N + n] = S[c][r];
    }
  if (mode == kLocal && blockIdx.x == 0 && threadIdx.x == 0) piece_decay[(size_t)blockIdx.z * heads + h] = decay;
}

// One thread per state value of a (sequence, head): the pieces in order.  piece_state[i] comes in as piece i's end
// state from zeros and leaves as its starting state; the slot's state becomes the state after the last piece.
__global__ void ssd_carry_kernel(float* __restrict__ state, float* __restrict__ piece_state,
                                 const float* __restrict__ piece_decay, const int* __restrict__ seq_slot,
                                 const int* __restrict__ seq_start, const int* __restrict__ cu_new, int heads,
                                 int per_head, int pieces, int piece_len) {
  const int s = blockIdx.z, h = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = seq_slot[s];
  if (e >= per_head || slot < 0) return;
  const int n_pieces = min(pieces, (cu_new[s + 1] - cu_new[s] + piece_len - 1) / piece_len);
  float* st = state + ((size_t)slot * heads + h) * per_head + e;
  float S = seq_start[s] > 0 ? *st : 0.f;
  // eight pieces at a time: their values are asked for together (one trip to memory, not eight), then chained
  constexpr int kBatch = 8;
  const size_t step = (size_t)heads * per_head;
  float* ps = piece_state + ((size_t)s * pieces * heads + h) * per_head + e;
  const float* pd = piece_decay + (size_t)s * pieces * heads + h;
  for (int i0 = 0; i0 < n_pieces; i0 += kBatch) {
    float local[kBatch], decay[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const bool in = i0 + k < n_pieces;
      local[k] = in ? __ldcs(ps + (size_t)(i0 + k) * step) : 0.f;
      decay[k] = in ? pd[(size_t)(i0 + k) * heads] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      if (i0 + k < n_pieces) {
        ps[(size_t)(i0 + k) * step] = S;
        S = fmaf(decay[k], S, local[k]);
      }
    }
  }
  *st = S;
}

template <typename T>
int launch_scan(const void* xbc, const void* dt_in, long long dt_stride, int dt_col, const float* dt_bias,
                const float* a_log, const float* skip, float* state, float* y, const int* seq_slot, const int* seq_start,
                const int* cu_new, int n_seqs, int heads, int vdim, int groups, int N, int pieces, float* piece_state,
                float* piece_decay, cudaStream_t stream) {
  const int R = (N + kLanes - 1) / kLanes;
  const int stage = scan_stage(R);
  const size_t smem = (size_t)(2 * stage * kLanes * R + stage * kChannels + 2 * stage) * sizeof(float);
  const dim3 grid((vdim + kChannels - 1) / kChannels, heads, n_seqs * pieces);
  constexpr int V = 16 / (int)sizeof(T);
  const bool vec = N % 8 == 0 && (heads * vdim) % V == 0 && vdim % V == 0 && (groups * N) % V == 0;
#define EMBER_SCAN_ARGS                                                                                                \
  (const T*)xbc, (const T*)dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start, cu_new, heads, \
      vdim, groups, N, stage
#define EMBER_SCAN_MODE(RMAX, MODE)                                                                                    \
  do {                                                                                                                 \
    if (vec)                                                                                                           \
      launch_plain(ssd_scan_kernel<T, RMAX, true>, grid, dim3(kScanThreads), smem, stream, EMBER_SCAN_ARGS, MODE, pieces, \
                 piece_state, piece_decay);                                                                           \
    else                                                                                                               \
      launch_plain(ssd_scan_kernel<T, RMAX, false>, grid, dim3(kScanThreads), smem, stream, EMBER_SCAN_ARGS, MODE, pieces, \
                 piece_state, piece_decay);                                                                           \
  } while (0)
#define EMBER_SCAN(MODE)                 \
  do {                                   \
    if (R <= 1) EMBER_SCAN_MODE(1, MODE); \
    else if (R <= 2) EMBER_SCAN_MODE(2, MODE); \
    else if (R <= 4) EMBER_SCAN_MODE(4, MODE); \
    else if (R <= 8) EMBER_SCAN_MODE(8, MODE); \
    else if (R <= 16) EMBER_SCAN_MODE(16, MODE); \
    else EMBER_SCAN_MODE(32, MODE);       \
  } while (0)
  if (pieces <= 1) {
    EMBER_SCAN(kWhole);
  } else {
    EMBER_SCAN(kLocal);
    const int per_head = vdim * N;
    ssd_carry_kernel<<<dim3((per_head + 255) / 256, heads, n_seqs), 256, 0, stream>>>(
        state, piece_state, piece_decay, seq_slot, seq_start, cu_new, heads, per_head, pieces, kSplit);
    EMBER_SCAN(kFinal);
  }
#undef EMBER_SCAN
#undef EMBER_SCAN_MODE
#undef EMBER_SCAN_ARGS
  EMBER_LAUNCH_OK("ssd_scan");
  return 0;
}


// ---------------------------------------------------------------------------- recurrence on the tensor cores
// For prompts in bfloat16 the recurrence of a piece of 64 tokens is three matrix products (the form that gives
// Mamba-2 its name).  With la_t the running sum of log decays inside the piece (la_t = A * sum_{s<=t} dt_s <= 0):
//   end state from zeros   E[p][n] = sum_s x_s[p] * (exp(la_end - la_s) dt_s B_s[n])
//   inside the piece       y_t    += sum_{s<=t} (C_t . B_s) exp(la_t - la_s) dt_s x_s
//   from the piece's start y_t    += exp(la_t) * (C_t . S_start)
// x, B and C are bfloat16 values, so their products are exact in float32 accumulators (mma.sync m16n8k16).  The
// factors that are float32 (the decays times B, the decayed scores, the state) enter as two bfloat16 terms, the
// value rounded and what the rounding left (hi + lo: about 16 bits of mantissa, two products instead of one), so
// the float32 quantities of the recurrence keep far more than bfloat16's precision; sums and the state itself are
// float32.  Every exponent is of a difference <= 0.  The pieces' starting states come from the same carry kernel
// as the scalar scan's.  Instantiated for states of 64 and 128 rows and 64 value channels; other sizes, float32
// and short steps take the scalar scan.
constexpr int kL = 64;

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* smem) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// v as a rounded bfloat16 and the bfloat16 of what the rounding left
__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(v);
  lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}
__device__ __forceinline__ unsigned pack2(__nv_bfloat16 a, __nv_bfloat16 b) {
  return (unsigned)__bfloat16_as_ushort(a) | ((unsigned)__bfloat16_as_ushort(b) << 16);
}

// Step sizes and running log decays of the piece's tokens (zero steps past its end), by the first warp.
__device__ __forceinline__ void piece_decays(const __nv_bfloat16* __restrict__ dt_in, long long dt_stride, int dt_col, int h,
                                             float bias, float A, int tc, int cnt, float* s_la, float* s_dt) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float d[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int tt = lane + 32 * k;
      d[k] = tt < cnt ? softplus_f(__bfloat162float(dt_in[(size_t)(tc + tt) * dt_stride + dt_col + h]) + bias) : 0.f;
    }
    float run[2] = {d[0], d[1]};
#pragma unroll
    for (int k = 0; k < 2; ++k)
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, run[k], off);
        if (lane >= off) run[k] += v;
      }
    run[1] += __shfl_sync(0xffffffffu, run[0], 31);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      s_dt[lane + 32 * k] = d[k];
      s_la[lane + 32 * k] = A * run[k];
    }
  }
}

// grid (1, heads, sequences * pieces): the end state of a piece from zeros, transposed [p][n], and its decay.
template <int N, int P>
__global__ void __launch_bounds__(128)
ssd_piece_state_kernel(const __nv_bfloat16* __restrict__ xbc, const __nv_bfloat16* __restrict__ dt_in, long long dt_stride,
                       int dt_col, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                       const int* __restrict__ seq_slot, const int* __restrict__ cu_new, int heads, int groups, int pieces,
                       float* __restrict__ piece_state, float* __restrict__ piece_decay) {
  constexpr int LDN = N + 8, LDL = kL + 8;
  extern __shared__ __align__(16) unsigned char raw[];
  __nv_bfloat16* sXt = reinterpret_cast<__nv_bfloat16*>(raw);  // [P][LDL]: x transposed
  __nv_bfloat16* sBh = sXt + P * LDL;                           // [kL][LDN]: decayed B, rounded
  __nv_bfloat16* sBl = sBh + kL * LDN;                          //            and what the rounding left
  __shared__ float s_la[kL], s_dt[kL];
  const int s = blockIdx.z / pieces, piece = blockIdx.z % pieces, h = blockIdx.y;
  if (seq_slot[s] < 0) return;
  const int tc = cu_new[s] + piece * kL, cnt = min(kL, cu_new[s + 1] - tc);
  if (cnt <= 0) return;
  const int inner = heads * P, gn = groups * N, g = h / (heads / groups);
  const size_t stride = (size_t)inner + 2 * gn;
  piece_decays(dt_in, dt_stride, dt_col, h, dt_bias[h], -expf(a_log[h]), tc, cnt, s_la, s_dt);
  __syncthreads();
  const float la_end = s_la[kL - 1];
#pragma unroll 4
  for (int e = threadIdx.x; e < kL * (N / 8); e += 128) {
    const int tt = e / (N / 8), j = e % (N / 8);
    __nv_bfloat16 hi[8], lo[8];
    if (tt < cnt) {
      const uint4 v = *reinterpret_cast<const uint4*>(xbc + (size_t)(tc + tt) * stride + inner + (size_t)g * N + j * 8);
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
      const float w = expf(la_end - s_la[tt]) * s_dt[tt];
#pragma unroll
      for (int i = 0; i < 8; ++i) split_bf16(__bfloat162float(b[i]) * w, hi[i], lo[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) hi[i] = lo[i] = __float2bfloat16_rn(0.f);
    }
    *reinterpret_cast<uint4*>(sBh + tt * LDN + j * 8) = *reinterpret_cast<const uint4*>(hi);
    *reinterpret_cast<uint4*>(sBl + tt * LDN + j * 8) = *reinterpret_cast<const uint4*>(lo);
  }
  for (int e = threadIdx.x; e < kL * (P / 8); e += 128) {
    const int tt = e % kL, j = e / kL;  // (consecutive threads, consecutive tokens: the transposed stores do not collide)
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tt < cnt) v = *reinterpret_cast<const uint4*>(xbc + (size_t)(tc + tt) * stride + (size_t)h * P + j * 8);
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) sXt[(j * 8 + i) * LDL + tt] = x[i];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int PW = P / 16;  // bands of 16 value channels; the four warps take them in turn
  for (int band = warp; band < PW; band += 4) {
    float acc[N / 8][4];
#pragma unroll
    for (int i = 0; i < N / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < kL / 16; ++ks) {
      unsigned af[4];
      ldsm_x4(af, sXt + (band * 16 + (lane & 15)) * LDL + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int dn = 0; dn < N / 16; ++dn) {
        unsigned b[4];
        const int at = (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDN + dn * 16 + (lane >> 4) * 8;
        ldsm_x4_trans(b, sBh + at);
        mma_16816(acc[2 * dn], af, b[0], b[1]);
        mma_16816(acc[2 * dn + 1], af, b[2], b[3]);
        ldsm_x4_trans(b, sBl + at);
        mma_16816(acc[2 * dn], af, b[0], b[1]);
        mma_16816(acc[2 * dn + 1], af, b[2], b[3]);
      }
    }
    const int gq = lane >> 2, c2 = (lane & 3) * 2;
    float* dst = piece_state + ((size_t)blockIdx.z * heads + h) * P * N;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int pch = band * 16 + gq + r * 8;
#pragma unroll
      for (int i = 0; i < N / 8; ++i)
        *reinterpret_cast<float2*>(dst + (size_t)pch * N + i * 8 + c2) = make_float2(acc[i][2 * r], acc[i][2 * r + 1]);
    }
  }
  if (threadIdx.x == 0) piece_decay[(size_t)blockIdx.z * heads + h] = expf(la_end);
}

// grid (1, heads, sequences * pieces): y of a piece from its starting state (piece_state, as the carry kernel left it).
template <int N, int P>
__global__ void __launch_bounds__(128)
ssd_piece_out_kernel(const __nv_bfloat16* __restrict__ xbc, const __nv_bfloat16* __restrict__ dt_in, long long dt_stride,
                     int dt_col, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                     const float* __restrict__ skip, float* __restrict__ y, const int* __restrict__ seq_slot,
                     const int* __restrict__ cu_new, int heads, int groups, int pieces,
                     const float* __restrict__ piece_state) {
  constexpr int LDN = N + 8, LDP = P + 8, KN = N / 16, KP = P / 16;
  extern __shared__ __align__(16) unsigned char raw[];
  __nv_bfloat16* sC = reinterpret_cast<__nv_bfloat16*>(raw);  // [kL][LDN]
  __nv_bfloat16* sB = sC + kL * LDN;                           // [kL][LDN]
  __nv_bfloat16* sX = sB + kL * LDN;                           // [kL][LDP]
  __nv_bfloat16* sSh = sX + kL * LDP;                          // [P][LDN]: the starting state, rounded
  __nv_bfloat16* sSl = sSh + P * LDN;                          //           and what the rounding left
  __shared__ float s_la[kL], s_dt[kL];
  const int s = blockIdx.z / pieces, piece = blockIdx.z % pieces, h = blockIdx.y;
  const int inner = heads * P, gn = groups * N, g = h / (heads / groups);
  const int t_first = cu_new[s] + piece * kL, cnt = min(kL, cu_new[s + 1] - t_first);
  if (cnt <= 0) return;
  if (seq_slot[s] < 0) {
    for (int e = threadIdx.x; e < cnt * P; e += 128) y[(size_t)(t_first + e / P) * inner + h * P + e % P] = 0.f;
    return;
  }
  const int tc = t_first;
  const size_t stride = (size_t)inner + 2 * gn;
  piece_decays(dt_in, dt_stride, dt_col, h, dt_bias[h], -expf(a_log[h]), tc, cnt, s_la, s_dt);
#pragma unroll 4
  for (int e = threadIdx.x; e < kL * (N / 8); e += 128) {
    const int tt = e / (N / 8), j = e % (N / 8);
    uint4 b = make_uint4(0, 0, 0, 0), c = make_uint4(0, 0, 0, 0);
    if (tt < cnt) {
      const __nv_bfloat16* src = xbc + (size_t)(tc + tt) * stride + inner + (size_t)g * N + j * 8;
      b = *reinterpret_cast<const uint4*>(src);
      c = *reinterpret_cast<const uint4*>(src + gn);
    }
    *reinterpret_cast<uint4*>(sB + tt * LDN + j * 8) = b;
    *reinterpret_cast<uint4*>(sC + tt * LDN + j * 8) = c;
  }
  for (int e = threadIdx.x; e < kL * (P / 8); e += 128) {
    const int tt = e / (P / 8), j = e % (P / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tt < cnt) v = *reinterpret_cast<const uint4*>(xbc + (size_t)(tc + tt) * stride + (size_t)h * P + j * 8);
    *reinterpret_cast<uint4*>(sX + tt * LDP + j * 8) = v;
  }
  {
    const float* src = piece_state + ((size_t)blockIdx.z * heads + h) * P * N;
#pragma unroll 4
    for (int e = threadIdx.x; e < P * (N / 4); e += 128) {
      const int pch = e / (N / 4), j = e % (N / 4);
      const float4 v = *reinterpret_cast<const float4*>(src + (size_t)pch * N + j * 4);
      __nv_bfloat16 hi[4], lo[4];
      split_bf16(v.x, hi[0], lo[0]);
      split_bf16(v.y, hi[1], lo[1]);
      split_bf16(v.z, hi[2], lo[2]);
      split_bf16(v.w, hi[3], lo[3]);
      *reinterpret_cast<uint2*>(sSh + pch * LDN + j * 4) = *reinterpret_cast<const uint2*>(hi);
      *reinterpret_cast<uint2*>(sSl + pch * LDN + j * 4) = *reinterpret_cast<const uint2*>(lo);
    }
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, c2 = (lane & 3) * 2;
  unsigned cf[KN][4];  // this warp's 16 rows of C
#pragma unroll
  for (int ks = 0; ks < KN; ++ks) ldsm_x4(cf[ks], sC + (warp * 16 + (lane & 15)) * LDN + ks * 16 + (lane >> 4) * 8);

  // scores C_t . B_s for the piece's 64 tokens s
  float sc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KN; ++ks) {
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      unsigned b[4];
      ldsm_x4(b, sB + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LDN + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_16816(sc[2 * np], cf[ks], b[0], b[1]);
      mma_16816(sc[2 * np + 1], cf[ks], b[2], b[3]);
    }
  }
  // decayed, causal: m[t][s] = score * exp(la_t - la_s) * dt_s for s <= t; as two bfloat16 terms
  const int row[2] = {warp * 16 + gq, warp * 16 + gq + 8};
  const float la_row[2] = {s_la[row[0]], s_la[row[1]]};
  unsigned mh[4][4], ml[4][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    __nv_bfloat16 hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int sx = i * 8 + c2 + (j & 1), r = j >> 1;
      const float m = sx <= row[r] ? sc[i][j] * expf(la_row[r] - s_la[sx]) * s_dt[sx] : 0.f;
      split_bf16(m, hi[j], lo[j]);
    }
    mh[i >> 1][(i & 1) * 2] = pack2(hi[0], hi[1]);
    mh[i >> 1][(i & 1) * 2 + 1] = pack2(hi[2], hi[3]);
    ml[i >> 1][(i & 1) * 2] = pack2(lo[0], lo[1]);
    ml[i >> 1][(i & 1) * 2 + 1] = pack2(lo[2], lo[3]);
  }
  float o[2 * KP][4], o2[2 * KP][4];
#pragma unroll
  for (int i = 0; i < 2 * KP; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = o2[i][j] = 0.f;
  // inside the piece: m . X
#pragma unroll
  for (int kk = 0; kk < kL / 16; ++kk) {
#pragma unroll
    for (int dn = 0; dn < KP; ++dn) {
      unsigned b[4];
      ldsm_x4_trans(b, sX + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDP + dn * 16 + (lane >> 4) * 8);
      mma_16816(o[2 * dn], mh[kk], b[0], b[1]);
      mma_16816(o[2 * dn + 1], mh[kk], b[2], b[3]);
      mma_16816(o[2 * dn], ml[kk], b[0], b[1]);
      mma_16816(o[2 * dn + 1], ml[kk], b[2], b[3]);
    }
  }
  // from the piece's start: C . S (the state lies transposed, [p][n], as a key matrix would)
#pragma unroll
  for (int ks = 0; ks < KN; ++ks) {
#pragma unroll
    for (int np = 0; np < KP; ++np) {
      unsigned b[4];
      const int at = (np * 16 + (lane & 7) + (lane >> 4) * 8) * LDN + ks * 16 + ((lane >> 3) & 1) * 8;
      ldsm_x4(b, sSh + at);
      mma_16816(o2[2 * np], cf[ks], b[0], b[1]);
      mma_16816(o2[2 * np + 1], cf[ks], b[2], b[3]);
      ldsm_x4(b, sSl + at);
      mma_16816(o2[2 * np], cf[ks], b[0], b[1]);
      mma_16816(o2[2 * np + 1], cf[ks], b[2], b[3]);
    }
  }
  const float D = skip[h];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (row[r] >= cnt) continue;
    const float from_start = expf(la_row[r]);
    float* dst = y + (size_t)(tc + row[r]) * inner + (size_t)h * P;
#pragma unroll
    for (int i = 0; i < 2 * KP; ++i) {
      const int pch = i * 8 + c2;
      const float x0 = __bfloat162float(sX[row[r] * LDP + pch]), x1 = __bfloat162float(sX[row[r] * LDP + pch + 1]);
      *reinterpret_cast<float2*>(dst + pch) = make_float2(fmaf(D, x0, fmaf(from_start, o2[i][2 * r], o[i][2 * r])),
                                                         fmaf(D, x1, fmaf(from_start, o2[i][2 * r + 1], o[i][2 * r + 1])));
    }
  }
}

template <int N, int P>
int launch_pieces(const void* xbc, const void* dt_in, long long dt_stride, int dt_col, const float* dt_bias,
                  const float* a_log, const float* skip, float* state, float* y, const int* seq_slot, const int* seq_start,
                  const int* cu_new, int n_seqs, int heads, int groups, int pieces, float* piece_state, float* piece_decay,
                  cudaStream_t stream) {
  constexpr int smem_state = (P * (kL + 8) + 2 * kL * (N + 8)) * (int)sizeof(__nv_bfloat16);
  constexpr int smem_out = (2 * kL * (N + 8) + kL * (P + 8) + 2 * P * (N + 8)) * (int)sizeof(__nv_bfloat16);
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(ssd_piece_state_kernel<N, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_state);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(ssd_piece_out_kernel<N, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_out);
    if (e != cudaSuccess) return ember_fail("ssd_pieces: %s", cudaGetErrorString(e));
    configured = true;
  }
  const dim3 grid(1, heads, n_seqs * pieces);
  ssd_piece_state_kernel<N, P><<<grid, 128, smem_state, stream>>>(
      (const __nv_bfloat16*)xbc, (const __nv_bfloat16*)dt_in, dt_stride, dt_col, dt_bias, a_log, seq_slot, cu_new, heads,
      groups, pieces, piece_state, piece_decay);
  const int per_head = P * N;
  ssd_carry_kernel<<<dim3((per_head + 255) / 256, heads, n_seqs), 256, 0, stream>>>(
      state, piece_state, piece_decay, seq_slot, seq_start, cu_new, heads, per_head, pieces, kL);
  ssd_piece_out_kernel<N, P><<<grid, 128, smem_out, stream>>>((const __nv_bfloat16*)xbc, (const __nv_bfloat16*)dt_in,
                                                              dt_stride, dt_col, dt_bias, a_log, skip, y, seq_slot, cu_new,
                                                              heads, groups, pieces, piece_state);
  EMBER_LAUNCH_OK("ssd_pieces");
  return 0;
}

}  // namespace

// all_single: every sequence brings one token (token t is sequence t): one launch does the state's shift too.
// max_new: the most tokens one sequence brings (the launch is sized by it).
EMBER_API int ember_conv_act(const void* in, long long in_stride, int col0, int channels, int taps, const float* w,
                             const float* bias, float* state, void* out, const int* token_seq, const int* seq_slot,
                             const int* seq_start, const int* cu_new, int T, int n_seqs, int max_new, int all_single,
                             int dtype, int act, cudaStream_t stream);

EMBER_API int ember_conv_silu(const void* in, long long in_stride, int col0, int channels, int taps, const float* w,
                              const float* bias, float* state, void* out, const int* token_seq, const int* seq_slot,
                              const int* seq_start, const int* cu_new, int T, int n_seqs, int max_new, int all_single,
                              int dtype, cudaStream_t stream) {
  return ember_conv_act(in, in_stride, col0, channels, taps, w, bias, state, out, token_seq, seq_slot, seq_start, cu_new, T,
                        n_seqs, max_new, all_single, dtype, 0, stream);
}

// The same with what follows the convolution's sum as an argument: act 0 silu, 1 nothing.
EMBER_API int ember_conv_act(const void* in, long long in_stride, int col0, int channels, int taps, const float* w,
                             const float* bias, float* state, void* out, const int* token_seq, const int* seq_slot,
                             const int* seq_start, const int* cu_new, int T, int n_seqs, int max_new, int all_single,
                             int dtype, int act, cudaStream_t stream) {
  EMBER_CHECK(act == 0 || act == 1, "conv: activation %d", act);
  EMBER_CHECK(T > 0 && n_seqs > 0 && channels > 0 && taps >= 1 && taps <= 16, "conv_silu: bad sizes");
  EMBER_CHECK(taps == 1 || state != nullptr, "conv_silu: a convolution of %d taps carries state", taps);
  EMBER_CHECK(dtype == EMBER_F32 || dtype == EMBER_BF16, "conv_silu: element type %d", dtype);
  EMBER_CHECK(max_new >= 1, "conv_silu: the longest sequence brings %d tokens", max_new);
  const int bx = (channels + 127) / 128;
  const int runs = (max_new + kConvRun - 1) / kConvRun;  // of the longest sequence
  const int elem = dtype == EMBER_F32 ? 4 : 2;
  const bool pairs = channels % 2 == 0 && col0 % 2 == 0 && in_stride % 2 == 0 && (uintptr_t)in % (2 * elem) == 0 &&
                     (uintptr_t)out % (2 * elem) == 0 && (uintptr_t)bias % 8 == 0 && (taps == 1 || (uintptr_t)state % 8 == 0);
  EMBER_CHECK(bx <= 65535, "conv_silu: %d channels exceed one launch", channels);
#define EMBER_CONV(TT)                                                                                                    \
  do {                                                                                                                    \
    if (all_single && T == n_seqs) {                                                                                      \
      launch_plain(conv_step_kernel<TT>, dim3(T, bx), dim3(128), 0, stream, (const TT*)in, in_stride, col0, channels, taps, \
                 w, bias, state, (TT*)out, seq_slot, seq_start, act);                                                          \
    } else if (taps <= 4 && pairs) {                                                                                      \
      conv_silu2_kernel<TT, 4><<<dim3(n_seqs * runs, (channels / 2 + 127) / 128), 128, 0, stream>>>(                      \
          (const TT*)in, in_stride, col0, channels, taps, w, bias, state, (TT*)out, seq_slot, seq_start, cu_new, runs, act);   \
    } else if (taps <= 4) {                                                                                               \
      conv_silu_kernel<TT, 4><<<dim3(n_seqs * runs, bx), 128, 0, stream>>>(                                               \
          (const TT*)in, in_stride, col0, channels, taps, w, bias, state, (TT*)out, seq_slot, seq_start, cu_new, runs, act);   \
    } else {                                                                                                              \
      conv_silu_kernel<TT, 16><<<dim3(n_seqs * runs, bx), 128, 0, stream>>>(                                              \
          (const TT*)in, in_stride, col0, channels, taps, w, bias, state, (TT*)out, seq_slot, seq_start, cu_new, runs, act);   \
    }                                                                                                                     \
    if (!(all_single && T == n_seqs)) {                                                                                   \
      if (taps > 1)                                                                                                       \
        conv_state_kernel<TT><<<dim3(n_seqs, bx), 128, 0, stream>>>((const TT*)in, in_stride, col0, channels, taps,       \
                                                                    state, seq_slot, seq_start, cu_new);                  \
    }                                                                                                                     \
  } while (0)
  if (dtype == EMBER_F32) EMBER_CONV(float); else EMBER_CONV(__nv_bfloat16);
#undef EMBER_CONV
  EMBER_LAUNCH_OK("conv_silu");
  return 0;
}

// Tokens of a piece, and the floats of scratch that a call with `pieces` pieces a sequence needs (0 for one piece).
EMBER_API int ember_ssd_scan_piece(void) { return kSplit; }
EMBER_API size_t ember_ssd_scan_scratch(int n_seqs, int pieces, int heads, int vdim, int N) {
  return pieces <= 1 ? 0 : (size_t)n_seqs * pieces * heads * ((size_t)vdim * N + 1);
}

// pieces: 1, or (a step whose longest sequence brings many tokens) ceil(longest / ember_ssd_scan_piece()): every
// sequence is then scanned in that many pieces side by side, with `scratch` of ember_ssd_scan_scratch floats.
EMBER_API int ember_ssd_scan(const void* xbc, const void* dt_in, long long dt_stride, int dt_col, const float* dt_bias,
                             const float* a_log, const float* skip, float* state, float* y, const int* seq_slot,
                             const int* seq_start, const int* cu_new, int n_seqs, int heads, int vdim, int groups, int N,
                             int pieces, float* scratch, int dtype, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && vdim > 0 && groups > 0 && heads % groups == 0, "ssd_scan: bad sizes");
  EMBER_CHECK(N >= 1 && N <= 256, "ssd_scan: a state of %d rows is not in [1, 256]", N);
  EMBER_CHECK(pieces >= 1 && (pieces == 1 || scratch != nullptr), "ssd_scan: %d pieces need scratch", pieces);
  EMBER_CHECK((long long)n_seqs * pieces <= 65535 && heads <= 65535, "ssd_scan: %d sequences x %d pieces x %d heads exceed one launch",
              n_seqs, pieces, heads);
  float* piece_state = scratch;
  float* piece_decay = scratch ? scratch + (size_t)n_seqs * pieces * heads * vdim * N : nullptr;
  if (dtype == EMBER_F32)
    return launch_scan<float>(xbc, dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start, cu_new,
                              n_seqs, heads, vdim, groups, N, pieces, piece_state, piece_decay, stream);
  if (dtype == EMBER_BF16)
    return launch_scan<__nv_bfloat16>(xbc, dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start,
                                      cu_new, n_seqs, heads, vdim, groups, N, pieces, piece_state, piece_decay, stream);
  return ember_fail("ssd_scan: element type %d", dtype);
}

// The recurrence of a step of prompts in bfloat16 as matrix products over pieces of 64 tokens (see above).  pieces:
// ceil(longest sequence's new tokens / ember_ssd_pieces_len()); scratch: ember_ssd_scan_scratch(n_seqs, pieces, ...)
// floats.  Returns 2, having launched nothing, for sizes without an instantiation: the caller takes ember_ssd_scan.
EMBER_API int ember_ssd_pieces_len(void) { return kL; }
EMBER_API int ember_ssd_pieces(const void* xbc, const void* dt_in, long long dt_stride, int dt_col, const float* dt_bias,
                               const float* a_log, const float* skip, float* state, float* y, const int* seq_slot,
                               const int* seq_start, const int* cu_new, int n_seqs, int heads, int vdim, int groups, int N,
                               int pieces, float* scratch, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && heads > 0 && groups > 0 && heads % groups == 0 && pieces >= 1 && scratch != nullptr,
              "ssd_pieces: bad sizes");
  if (vdim != 64 || (N != 64 && N != 128) || (groups * N) % 8 || dt_stride <= 0) return 2;
  EMBER_CHECK((long long)n_seqs * pieces <= 65535 && heads <= 65535, "ssd_pieces: %d sequences x %d pieces x %d heads exceed one launch",
              n_seqs, pieces, heads);
  float* piece_state = scratch;
  float* piece_decay = scratch + (size_t)n_seqs * pieces * heads * vdim * N;
  if (N == 64)
    return launch_pieces<64, 64>(xbc, dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start, cu_new,
                                 n_seqs, heads, groups, pieces, piece_state, piece_decay, stream);
  return launch_pieces<128, 64>(xbc, dt_in, dt_stride, dt_col, dt_bias, a_log, skip, state, y, seq_slot, seq_start, cu_new,
                                n_seqs, heads, groups, pieces, piece_state, piece_decay, stream);
}
