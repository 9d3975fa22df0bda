// minGRU over a step's packed tokens: a recurrence per channel whose gates read the current token alone.
//
//     z_t = sigmoid(a_t + bias_z)      u_t = b_t + bias_x      c_t = u_t + 1/2 where u_t >= 0, sigmoid(u_t) where u_t < 0
//     S_t = (1 - z_t) S_(t-1) + z_t c_t                         out_t = S_t * silu(g_t)
// a, b and g are columns of one projection (the step's rows of z | x | g).  Gates, candidates and the state
// are float32 whatever the element types that come in or go out.
//
// A thread takes a channel through a sequence's tokens in order, so a token's result depends on its
// sequence alone.  A long sequence is cut into pieces that are walked side by side: the recurrence is
// S_t = A_t S_(t-1) + B_t, so a piece walked from zero gives (product of its A, its end value from zero); the
// pieces' start values follow from those in order, and a second walk from each piece's start value writes the
// results.  A sequence that starts at position 0 starts from zeros whatever its slot's state holds; sequences
// of slot -1 are padding: their rows are zero and no state is touched.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;

__device__ __forceinline__ float sigmoidf(float v) { return 1.0f / (1.0f + expf(-v)); }

__device__ __forceinline__ void gate_and_candidate(float a, float b, float& z, float& c) {
  z = sigmoidf(a);
  c = b >= 0.f ? b + 0.5f : sigmoidf(b);
}

// grid (sequences, channel tiles, pieces).  phase 0: the whole walk (one piece).  phase 1: a piece from zero,
// leaving (product of 1 - z, end value) in scratch.  phase 2: the walk from the piece's start value, which the
// carry left in scratch.
template <typename TIN, typename TOUT>
__global__ void __launch_bounds__(kThreads)
mingru_kernel(const TIN* __restrict__ proj, long long stride, int z_col, int x_col, int g_col, const float* __restrict__ bias_z,
              const float* __restrict__ bias_x, float* __restrict__ state, TOUT* __restrict__ out,
              const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ cu_new, int width,
              int piece, int phase, float* __restrict__ scratch) {
  const int s = blockIdx.x, c = blockIdx.y * kThreads + threadIdx.x, p = blockIdx.z;
  if (c >= width) return;
  const int t0 = cu_new[s], n = cu_new[s + 1] - t0;
  const int lo = p * piece, hi = min(n, lo + piece);
  const int slot = seq_slot[s];
  if (slot < 0) {
    if (phase != 1)
      for (int i = lo; i < hi; ++i) out[(size_t)(t0 + i) * width + c] = from_float<TOUT>(0.f);
    return;
  }
  if (lo >= n) return;
  const float bz = bias_z[c], bx = bias_x[c];
  float* mine = scratch ? scratch + (((size_t)s * gridDim.z + p) * width + c) * 2 : nullptr;
  float S = 0.f;
  if (phase == 0) S = seq_start[s] > 0 ? state[(size_t)slot * width + c] : 0.f;
  if (phase == 2) S = mine[1];
  float A = 1.f;
  constexpr int kAhead = 8;      // tokens whose columns are fetched before the chain of the state walks them
  for (int i0 = lo; i0 < hi; i0 += kAhead) {
    float za[kAhead], xa[kAhead], ga[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const bool there = i0 + u < hi;
      const TIN* row = proj + (size_t)(t0 + (there ? i0 + u : lo)) * stride;
      za[u] = to_float(row[z_col + c]);
      xa[u] = to_float(row[x_col + c]);
      ga[u] = phase == 1 ? 0.f : to_float(row[g_col + c]);
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (i0 + u >= hi) break;
      float z, cand;
      gate_and_candidate(za[u] + bz, xa[u] + bx, z, cand);
      S = fmaf(1.0f - z, S, z * cand);
      if (phase == 1) {
        A *= 1.0f - z;
      } else {
        const float g = ga[u];
        out[(size_t)(t0 + i0 + u) * width + c] = from_float<TOUT>(S * (g * sigmoidf(g)));
      }
    }
  }
  if (phase == 1) {
    mine[0] = A;
    mine[1] = S;
  } else if (hi == n) {
    state[(size_t)slot * width + c] = S;
  }
}

// grid (sequences, channel tiles): scratch (A, end from zero) of every piece becomes (A, start value).
__global__ void mingru_carry_kernel(float* __restrict__ scratch, const float* __restrict__ state, const int* __restrict__ seq_slot,
                                    const int* __restrict__ seq_start, const int* __restrict__ cu_new, int width, int piece,
                                    int pieces) {
  const int s = blockIdx.x, c = blockIdx.y * kThreads + threadIdx.x;
  if (c >= width) return;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int n = cu_new[s + 1] - cu_new[s];
  float S = seq_start[s] > 0 ? state[(size_t)slot * width + c] : 0.f;
  for (int p = 0; p < pieces && p * piece < n; ++p) {
    float* mine = scratch + (((size_t)s * pieces + p) * width + c) * 2;
    const float A = mine[0], B = mine[1];
    mine[1] = S;
    S = fmaf(A, S, B);
  }
}

}  // namespace

EMBER_API size_t ember_mingru_scratch(int n_seqs, int pieces, int width) { return (size_t)n_seqs * pieces * width * 2; }

// proj: rows of `stride` values with the gate's, the candidate's and the output gate's `width` columns from z_col, x_col
// and g_col; biases float32 [width]; state float32 [slots, width] (advanced); out [T, width].  pieces 1: one walk;
// more (with scratch of ember_mingru_scratch floats): pieces of `piece` tokens side by side.
EMBER_API int ember_mingru(const void* proj, long long stride, int z_col, int x_col, int g_col, const float* bias_z,
                           const float* bias_x, float* state, void* out, const int* seq_slot, const int* seq_start,
                           const int* cu_new, int n_seqs, int width, int piece, int pieces, float* scratch, int in_dtype,
                           int out_dtype, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && width > 0 && pieces >= 1 && piece >= 1, "mingru: bad sizes");
  EMBER_CHECK(pieces == 1 || scratch != nullptr, "mingru: pieces side by side need scratch");
  EMBER_CHECK(pieces <= 65535, "mingru: %d pieces exceed one launch", pieces);
  const int tiles = (width + kThreads - 1) / kThreads;
  cudaError_t e = cudaSuccess;
#define EMBER_GRU(TIN, TOUT, PHASE, PIECES)                                                                                   \
  launch_plain(mingru_kernel<TIN, TOUT>, dim3(n_seqs, tiles, PIECES), dim3(kThreads), 0, stream, (const TIN*)proj, stride, z_col, \
               x_col, g_col, bias_z, bias_x, state, (TOUT*)out, seq_slot, seq_start, cu_new, width, piece, PHASE, scratch)
#define EMBER_GRU_ANY(PHASE, PIECES)                                                             \
  (in_dtype == EMBER_F32 && out_dtype == EMBER_F32     ? EMBER_GRU(float, float, PHASE, PIECES)   \
   : in_dtype == EMBER_F32 && out_dtype == EMBER_BF16  ? EMBER_GRU(float, __nv_bfloat16, PHASE, PIECES) \
                                                       : EMBER_GRU(__nv_bfloat16, __nv_bfloat16, PHASE, PIECES))
  EMBER_CHECK((in_dtype == EMBER_F32 || in_dtype == EMBER_BF16) && (out_dtype == EMBER_F32 || out_dtype == EMBER_BF16) &&
                  !(in_dtype == EMBER_BF16 && out_dtype == EMBER_F32),
              "mingru: element types %d -> %d", in_dtype, out_dtype);
  if (pieces == 1) {
    e = EMBER_GRU_ANY(0, 1);
  } else {
    e = EMBER_GRU_ANY(1, pieces);
    if (e == cudaSuccess)
      e = launch_plain(mingru_carry_kernel, dim3(n_seqs, tiles), dim3(kThreads), 0, stream, scratch, (const float*)state, seq_slot,
                       seq_start, cu_new, width, piece, pieces);
    if (e == cudaSuccess) e = EMBER_GRU_ANY(2, pieces);
  }
#undef EMBER_GRU_ANY
#undef EMBER_GRU
  if (e != cudaSuccess) return ember_fail("mingru: %s", cudaGetErrorString(e));
  return 0;
}
