// Experts chosen by a table: the step's (token, choice) pairs sorted by expert, and the two grouped
// products that run every expert over its own pairs.
//
// Pair q = t * top + k is choice k of token t; its expert is table[token id][k].  `moe_route` makes,
// in one launch, the pairs' experts, each expert's count as a running sum (offsets[experts + 1]) and the
// pairs in expert order (sorted[pairs]; the order inside an expert is whatever the atomics gave, which no
// result depends on: every pair's row is computed by itself).  The products:
//   gate_up   inner[q, :] = silu(Wg_e a_t) * (Wu_e a_t)     (W_e = [gate | up] stacked, [2 * inner, width])
//   down      y[q, :]     = Wd_e inner[q, :]                (float32)
// Few pairs (a decode step): a warp per output value streams the expert's rows once, which is all the
// traffic there is.  Many pairs (a prompt): tiles of one expert's pairs and outputs on mma.sync
// m16n8k16 with cp.async double buffering (tiles of 128 pairs x 64 outputs).  float32 takes the streaming form at every size: one
// fixed order of additions per output value, no reduced-precision matrix mode.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------- routing
__global__ void __launch_bounds__(1024)
moe_route_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int n_pairs, int top, int experts,
                 int vocab, int* __restrict__ pair_expert, int* __restrict__ offsets, int* __restrict__ sorted) {
  extern __shared__ int sm_i[];  // count[experts], cursor[experts]
  int* count = sm_i;
  int* cursor = sm_i + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int q = threadIdx.x; q < n_pairs; q += blockDim.x) {
    int tok = tokens ? tokens[q / top] : q / top;     // (no ids: the table's row t is token t's choice)
    tok = min(max(tok, 0), vocab - 1);
    int e = table[(size_t)tok * top + q % top];
    e = min(max(e, 0), experts - 1);
    pair_expert[q] = e;
    atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      run += count[e];
    }
    offsets[experts] = run;
  }
  __syncthreads();
  for (int q = threadIdx.x; q < n_pairs; q += blockDim.x) sorted[atomicAdd(&cursor[pair_expert[q]], 1)] = q;
}

// ---------------------------------------------------------------------------- streaming form
// The dot product of two rows of K values by one warp: lanes take 16-byte pieces in turn where the rows
// allow it, single values else; the lanes' sums are added by warp_sum.  The order depends on K alone.
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const T* a, int K, int lane) {
  constexpr int V = 16 / (int)sizeof(T);
  float acc = 0.f;
  if (K % V == 0) {
    for (int k = lane * V; k < K; k += 32 * V) {
      const uint4 wr = *reinterpret_cast<const uint4*>(w + k);
      const uint4 ar = __ldcg(reinterpret_cast<const uint4*>(a + k));
      const T* wv = reinterpret_cast<const T*>(&wr);
      const T* av = reinterpret_cast<const T*>(&ar);
#pragma unroll
      for (int i = 0; i < V; ++i) acc = fmaf(to_float(wv[i]), to_float(av[i]), acc);
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(to_float(w[k]), to_float(__ldcg(a + k)), acc);
  }
  return warp_sum(acc);
}

// silu(g) * u, or with limit > 0 the clamped form: g capped at limit, u within +-limit, g * sigmoid(alpha g) * (u + shift)
__device__ __forceinline__ float gate_value(float g, float u, float limit, float alpha, float shift) {
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + shift);
  }
  return g / (1.0f + expf(-g)) * u;
}

constexpr int kStreamWarps = 8;
constexpr int kStreamOutputs = 4;  // per warp

// grid (pairs, ceil(inner / 32))
template <typename T>
__global__ void __launch_bounds__(kStreamWarps * 32)
moe_gate_up_stream_kernel(const T* __restrict__ a, const T* __restrict__ w, const int* __restrict__ pair_expert,
                          T* __restrict__ out, int top, int width, int inner, float limit, float alpha, float shift) {
  const int q = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* row = a + (size_t)(q / top) * width;
  const T* we = w + (size_t)pair_expert[q] * 2 * inner * width;
  for (int i = 0; i < kStreamOutputs; ++i) {
    const int f = (blockIdx.y * kStreamWarps + warp) * kStreamOutputs + i;
    if (f >= inner) return;
    const float g = warp_dot(we + (size_t)f * width, row, width, lane);
    const float u = warp_dot(we + (size_t)(inner + f) * width, row, width, lane);
    if (lane == 0) out[(size_t)q * inner + f] = from_float<T>(gate_value(g, u, limit, alpha, shift));
  }
}

// grid (pairs, ceil(width / 32))
template <typename T>
__global__ void __launch_bounds__(kStreamWarps * 32)
moe_down_stream_kernel(const T* __restrict__ a, const T* __restrict__ w, const int* __restrict__ pair_expert,
                       float* __restrict__ out, int width, int inner) {
  const int q = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* row = a + (size_t)q * inner;
  const T* we = w + (size_t)pair_expert[q] * width * inner;
  for (int i = 0; i < kStreamOutputs; ++i) {
    const int n = (blockIdx.y * kStreamWarps + warp) * kStreamOutputs + i;
    if (n >= width) return;
    const float v = warp_dot(we + (size_t)n * inner, row, inner, lane);
    if (lane == 0) out[(size_t)q * width + n] = v;
  }
}

// ---------------------------------------------------------------------------- tiled form (bfloat16)
constexpr int kTileM = 128;  // pairs a tile
constexpr int kTileN = 64;   // outputs a tile
constexpr int kStep = 64;    // of the summed dimension per trip
constexpr int kLd = kStep + 8;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATED>
constexpr int tile_smem() {
  return (2 * kTileM * kLd + 2 * (GATED ? 2 : 1) * kTileN * kLd) * (int)sizeof(__nv_bfloat16);
}

// GATED: W_e = [gate | up] of n_out rows each, the result silu(gate) * up in bfloat16 and the input rows are
// the tokens' (pair / top); else W_e has n_out rows, the result is float32 and the input rows are the pairs'.
// grid (tiles of pairs: an upper bound, ceil(n_out / 64)); a block finds its expert and its tile of that
// expert's pairs from the offsets, and leaves if there is none.  Four warps, each 32 pairs x 64 outputs.
template <bool GATED>
__global__ void __launch_bounds__(128)
moe_tile_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, const int* __restrict__ offsets,
                const int* __restrict__ sorted, void* __restrict__ out, int experts, int top, int K, int n_out, float limit,
                float alpha, float shift) {
  constexpr int NW = GATED ? 2 : 1;
  extern __shared__ __align__(16) unsigned char tile_raw[];
  __nv_bfloat16* sA = reinterpret_cast<__nv_bfloat16*>(tile_raw);  // [2][kTileM * kLd]
  __nv_bfloat16* sW = sA + 2 * kTileM * kLd;                       // [2][NW][kTileN * kLd]
  __shared__ int s_rows[kTileM];  // the input row of each of the tile's pairs, -1 past the expert's last
  __shared__ int s_pair[kTileM];
  __shared__ int s_expert, s_tile;

  if (threadIdx.x == 0) {
    int tile = blockIdx.x, found = -1;
    for (int e = 0; e < experts; ++e) {
      const int tiles = (offsets[e + 1] - offsets[e] + kTileM - 1) / kTileM;
      if (tile < tiles) {
        found = e;
        break;
      }
      tile -= tiles;
    }
    s_expert = found;
    s_tile = tile;
  }
  __syncthreads();
  const int e = s_expert;
  if (e < 0) return;
  const int first = offsets[e] + s_tile * kTileM, count = min(kTileM, offsets[e + 1] - first);
  {
    const int q = (int)threadIdx.x < count ? sorted[first + threadIdx.x] : -1;
    s_pair[threadIdx.x] = q;
    s_rows[threadIdx.x] = q < 0 ? -1 : (GATED ? q / top : q);
  }
  __syncthreads();

  const int n0 = blockIdx.y * kTileN;
  const __nv_bfloat16* we = w + (size_t)e * NW * n_out * K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  auto load = [&](int buf, int k0) {
    constexpr int CPR = kStep / 8;  // 16-byte pieces a row
    for (int id = threadIdx.x; id < kTileM * CPR; id += 128) {
      const int r = id / CPR, c = id % CPR;
      const int src = s_rows[r];
      const bool ok = src >= 0 && k0 + c * 8 < K;
      cp_async_16(sA + (size_t)buf * kTileM * kLd + r * kLd + c * 8, a + (ok ? (size_t)src * K + k0 + c * 8 : 0), ok);
    }
    for (int id = threadIdx.x; id < kTileN * CPR; id += 128) {
      const int r = id / CPR, c = id % CPR;
      const bool ok = n0 + r < n_out && k0 + c * 8 < K;
#pragma unroll
      for (int m = 0; m < NW; ++m)
        cp_async_16(sW + ((size_t)buf * NW + m) * kTileN * kLd + r * kLd + c * 8,
                    we + (ok ? ((size_t)m * n_out + n0 + r) * K + k0 + c * 8 : 0), ok);
    }
  };

  float acc[NW][2][8][4];
#pragma unroll
  for (int m = 0; m < NW; ++m)
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[m][f][i][j] = 0.f;

  const int trips = (K + kStep - 1) / kStep;
  load(0, 0);
  cp_async_commit();
  for (int trip = 0; trip < trips; ++trip) {
    const int buf = trip & 1;
    if (trip + 1 < trips) {
      load(buf ^ 1, (trip + 1) * kStep);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* tA = sA + (size_t)buf * kTileM * kLd;
#pragma unroll
    for (int ks = 0; ks < kStep / 16; ++ks) {
      unsigned af[2][4];
#pragma unroll
      for (int f = 0; f < 2; ++f)
        ldmatrix_x4(af[f], tA + (warp * 32 + f * 16 + (lane & 15)) * kLd + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int m = 0; m < NW; ++m) {
        const __nv_bfloat16* tW = sW + ((size_t)buf * NW + m) * kTileN * kLd;
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          unsigned b[4];
          ldmatrix_x4(b, tW + (np * 16 + (lane & 7) + (lane >> 4) * 8) * kLd + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
          for (int f = 0; f < 2; ++f) {
            mma_bf16(acc[m][f][2 * np], af[f], b[0], b[1]);
            mma_bf16(acc[m][f][2 * np + 1], af[f], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();  // the other buffer is refilled at the top of the next trip
  }

  const int g = lane >> 2, c2 = (lane & 3) * 2;
#pragma unroll
  for (int f = 0; f < 2; ++f) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int q = s_pair[warp * 32 + f * 16 + g + r * 8];
      if (q < 0) continue;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int n = n0 + i * 8 + c2;  // this thread's two outputs: n and n + 1 (n_out is even where rows are 16-byte pieces)
        if (n >= n_out) continue;
        if constexpr (GATED) {
          const float g0 = acc[0][f][i][2 * r], g1 = acc[0][f][i][2 * r + 1];
          const float y0 = gate_value(g0, acc[1][f][i][2 * r], limit, alpha, shift), y1 = gate_value(g1, acc[1][f][i][2 * r + 1], limit, alpha, shift);
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(out) + (size_t)q * n_out + n;
          if (n + 1 < n_out)
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(y0, y1);
          else
            *dst = __float2bfloat16_rn(y0);
        } else {
          float* dst = static_cast<float*>(out) + (size_t)q * n_out + n;
          if (n + 1 < n_out)
            *reinterpret_cast<float2*>(dst) = make_float2(acc[0][f][i][2 * r], acc[0][f][i][2 * r + 1]);
          else
            *dst = acc[0][f][i][2 * r];
        }
      }
    }
  }
}

template <bool GATED>
int launch_tiles(const void* a, const void* w, const int* offsets, const int* sorted, void* out, long long pairs, int experts,
                 int top, int K, int n_out, cudaStream_t stream, const char* name, float limit = 0.f, float alpha = 1.f,
                 float shift = 0.f) {
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_tile_kernel<GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, tile_smem<GATED>());
    if (e != cudaSuccess) return ember_fail("%s: %s", name, cudaGetErrorString(e));
    configured = true;
  }
  const dim3 grid((unsigned)((pairs + kTileM - 1) / kTileM + experts), (n_out + kTileN - 1) / kTileN);
  EMBER_CHECK(grid.y <= 65535, "%s: %d outputs exceed one launch", name, n_out);
  moe_tile_kernel<GATED><<<grid, 128, tile_smem<GATED>(), stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w, offsets,
                                                                    sorted, out, experts, top, K, n_out, limit, alpha, shift);
  EMBER_LAUNCH_OK(name);
  return 0;
}

// ---------------------------------------------------------------------------- the router's choice
// A warp a token.  s = sigmoid(z); the choice is made on s + correction among the experts of the `keep` groups
// whose two largest choice scores add up to the most; weights = s of the chosen, over their sum (+ 1e-20), times
// `scale`.  Among equal scores the lower index wins.  Dynamic shared memory: per warp 2 * experts + groups floats.
constexpr int kPickWarps = 4;

__device__ __forceinline__ void warp_argmax(float& best, int& at) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, at, off);
    if (ov > best || (ov == best && oi < at)) {
      best = ov;
      at = oi;
    }
  }
}

__global__ void __launch_bounds__(32 * kPickWarps)
moe_pick_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction, int T, int experts, int top,
                int groups, int keep, float scale, int* __restrict__ chosen, float* __restrict__ weights) {
  extern __shared__ float pick_sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kPickWarps + warp;
  if (t >= T) return;
  float* sc = pick_sm + (size_t)warp * (2 * experts + groups);
  float* ch = sc + experts;
  float* gs = ch + experts;
  for (int e = lane; e < experts; e += 32) {
    const float s = 1.0f / (1.0f + expf(-logits[(size_t)t * ld + e]));
    sc[e] = s;
    ch[e] = s + correction[e];
  }
  __syncwarp();
  if (groups > 1) {
    const int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {
      float m1 = -INFINITY, m2 = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = ch[e];
        if (v > m1) {
          m2 = m1;
          m1 = v;
        } else if (v > m2) {
          m2 = v;
        }
      }
      gs[g] = per >= 2 ? m1 + m2 : m1;
    }
    __syncwarp();
    for (int it = 0; it < keep; ++it) {     // a kept group's score becomes +inf, which is never picked again
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (v > best || (v == best && g < at))) {
          best = v;
          at = g;
        }
      }
      warp_argmax(best, at);
      if (lane == 0 && at < groups) gs[at] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gs[e / per] != INFINITY) ch[e] = -INFINITY;
    __syncwarp();
  }
  float sum = 0.f;      // (every lane keeps the same sum)
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = ch[e];
      if (v > best || (v == best && e < at)) {
        best = v;
        at = e;
      }
    }
    warp_argmax(best, at);
    if (at >= experts) at = 0;
    sum += sc[at];
    if (lane == 0) {
      chosen[(size_t)t * top + k] = at;
      weights[(size_t)t * top + k] = sc[at];
      ch[at] = -INFINITY;
    }
    __syncwarp();
  }
  const float f = scale / (sum + 1e-20f);
  for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] *= f;
}

// grid (T): out = x + sum_k weights[t, k] y[t, k, :] (k ascending) + sigmoid(gate) * shared[t, :]
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ weights,
                   const float* __restrict__ shared, const float* __restrict__ logits, int ld, int gate_col,
                   float* __restrict__ out, int top, int width) {
  const int t = blockIdx.x;
  const float* w = weights + (size_t)t * top;
  const float sg = shared == nullptr ? 0.f : (logits == nullptr ? 1.f : 1.0f / (1.0f + expf(-logits[(size_t)t * ld + gate_col])));
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(w[k], y[((size_t)t * top + k) * width + c], acc);
    if (shared != nullptr) acc = fmaf(sg, shared[(size_t)t * width + c], acc);
    out[(size_t)t * width + c] = x[(size_t)t * width + c] + acc;
  }
}

}  // namespace

// logits float32 [T, ld] (the first `experts` columns are the router's), correction float32 [experts];
// chosen int32 [T, top], weights float32 [T, top].
EMBER_API int ember_moe_pick(const float* logits, int ld, const float* correction, int T, int experts, int top, int groups,
                             int keep, float scale, int* chosen, float* weights, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && experts > 0 && experts <= 1024 && top >= 1 && top <= experts && ld >= experts,
              "moe_pick: %d tokens, top %d of %d experts (at most 1024)", T, top, experts);
  EMBER_CHECK(groups >= 1 && experts % groups == 0 && keep >= 1 && keep <= groups && (long long)keep * (experts / groups) >= top,
              "moe_pick: %d groups of which %d are kept do not hold %d choices", groups, keep, top);
  const size_t smem = (size_t)kPickWarps * (2 * experts + groups) * sizeof(float);
  const cudaError_t e = launch_plain(moe_pick_kernel, dim3((T + kPickWarps - 1) / kPickWarps), dim3(32 * kPickWarps), smem, stream,
                                     logits, ld, correction, T, experts, top, groups, keep, scale, chosen, weights);
  if (e != cudaSuccess) return ember_fail("moe_pick: %s", cudaGetErrorString(e));
  return 0;
}

// x, out float32 [T, width]; y float32 [T, top, width]; weights float32 [T, top]; shared float32 [T, width] or null;
// logits float32 [T, ld] or null (then the shared rows are added as they are): the shared rows' gate is column gate_col.
EMBER_API int ember_moe_combine(const float* x, const float* y, const float* weights, const float* shared, const float* logits,
                                int ld, int gate_col, float* out, int T, int top, int width, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && top > 0 && width > 0, "moe_combine: bad sizes");
  EMBER_CHECK(logits == nullptr || (gate_col >= 0 && gate_col < ld), "moe_combine: gate column %d of %d", gate_col, ld);
  const cudaError_t e = launch_plain(moe_combine_kernel, dim3(T), dim3(256), 0, stream, x, y, weights, shared, logits, ld, gate_col,
                                     out, top, width);
  if (e != cudaSuccess) return ember_fail("moe_combine: %s", cudaGetErrorString(e));
  return 0;
}

// tokens [T] (ids; null: the table's row t is token t's choice), table [vocab, top]; pair_expert [T * top], offsets [experts + 1], sorted [T * top]
EMBER_API int ember_moe_route(const int* tokens, const int* table, int T, int top, int experts, int vocab, int* pair_expert,
                              int* offsets, int* sorted, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && top > 0 && experts > 0 && vocab > 0 && top <= experts && (tokens != nullptr || vocab >= T), "moe_route: bad sizes");
  EMBER_CHECK(experts <= 4096, "moe_route: %d experts (at most 4096)", experts);
  EMBER_CHECK((long long)T * top < (1ll << 30), "moe_route: %d tokens x %d choices", T, top);
  const cudaError_t e = launch_plain(moe_route_kernel, dim3(1), dim3(1024), 2 * experts * sizeof(int), stream, tokens, table,
                                   T * top, top, experts, vocab, pair_expert, offsets, sorted);
  if (e != cudaSuccess) return ember_fail("moe_route: %s", cudaGetErrorString(e));
  return 0;
}

// a [T, width] (dtype), w [experts, 2 * inner, width], out [T * top, inner] (dtype).  tiled != 0 (bfloat16 only):
// the tensor-core tiles; else the streaming form.
EMBER_API int ember_moe_gate_up_act(const void* a, const void* w, const int* pair_expert, const int* offsets, const int* sorted,
                                    void* out, int T, int top, int experts, int width, int inner, int tiled, int dtype,
                                    float limit, float alpha, float shift, cudaStream_t stream);

EMBER_API int ember_moe_gate_up(const void* a, const void* w, const int* pair_expert, const int* offsets, const int* sorted,
                                void* out, int T, int top, int experts, int width, int inner, int tiled, int dtype,
                                cudaStream_t stream) {
  return ember_moe_gate_up_act(a, w, pair_expert, offsets, sorted, out, T, top, experts, width, inner, tiled, dtype, 0.f, 1.f, 0.f,
                               stream);
}

// The same with the gate's form as arguments: limit 0: silu(g) * u; limit > 0: g capped at limit, u within +-limit,
// g * sigmoid(alpha g) * (u + shift).
EMBER_API int ember_moe_gate_up_act(const void* a, const void* w, const int* pair_expert, const int* offsets, const int* sorted,
                                    void* out, int T, int top, int experts, int width, int inner, int tiled, int dtype,
                                    float limit, float alpha, float shift, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && top > 0 && experts > 0 && width > 0 && inner > 0 && limit >= 0.f, "moe_gate_up: bad sizes");
  const long long pairs = (long long)T * top;
  if (tiled) {
    EMBER_CHECK(dtype == EMBER_BF16 && width % 8 == 0 && inner % 2 == 0,
                "moe_gate_up: tiles take bfloat16 rows that are multiples of 8 and an even number of outputs");
    return launch_tiles<true>(a, w, offsets, sorted, out, pairs, experts, top, width, inner, stream, "moe_gate_up", limit, alpha, shift);
  }
  const dim3 grid((unsigned)pairs, (inner + kStreamWarps * kStreamOutputs - 1) / (kStreamWarps * kStreamOutputs));
  EMBER_CHECK(grid.y <= 65535, "moe_gate_up: %d outputs exceed one launch", inner);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(moe_gate_up_stream_kernel<float>, grid, dim3(kStreamWarps * 32), 0, stream, (const float*)a, (const float*)w,
                   pair_expert, (float*)out, top, width, inner, limit, alpha, shift);
  else if (dtype == EMBER_BF16)
    e = launch_plain(moe_gate_up_stream_kernel<__nv_bfloat16>, grid, dim3(kStreamWarps * 32), 0, stream, (const __nv_bfloat16*)a,
                   (const __nv_bfloat16*)w, pair_expert, (__nv_bfloat16*)out, top, width, inner, limit, alpha, shift);
  else
    return ember_fail("moe_gate_up: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("moe_gate_up: %s", cudaGetErrorString(e));
  return 0;
}

// a [T * top, inner] (dtype), w [experts, width, inner], out float32 [T * top, width]
EMBER_API int ember_moe_down(const void* a, const void* w, const int* pair_expert, const int* offsets, const int* sorted,
                             float* out, int T, int top, int experts, int width, int inner, int tiled, int dtype,
                             cudaStream_t stream) {
  EMBER_CHECK(T > 0 && top > 0 && experts > 0 && width > 0 && inner > 0, "moe_down: bad sizes");
  const long long pairs = (long long)T * top;
  if (tiled) {
    EMBER_CHECK(dtype == EMBER_BF16 && inner % 8 == 0 && width % 2 == 0,
                "moe_down: tiles take bfloat16 rows that are multiples of 8 and an even number of outputs");
    return launch_tiles<false>(a, w, offsets, sorted, out, pairs, experts, top, inner, width, stream, "moe_down");
  }
  const dim3 grid((unsigned)pairs, (width + kStreamWarps * kStreamOutputs - 1) / (kStreamWarps * kStreamOutputs));
  EMBER_CHECK(grid.y <= 65535, "moe_down: %d outputs exceed one launch", width);
  cudaError_t e;
  if (dtype == EMBER_F32)
    e = launch_plain(moe_down_stream_kernel<float>, grid, dim3(kStreamWarps * 32), 0, stream, (const float*)a, (const float*)w,
                   pair_expert, out, width, inner);
  else if (dtype == EMBER_BF16)
    e = launch_plain(moe_down_stream_kernel<__nv_bfloat16>, grid, dim3(kStreamWarps * 32), 0, stream, (const __nv_bfloat16*)a,
                   (const __nv_bfloat16*)w, pair_expert, out, width, inner);
  else
    return ember_fail("moe_down: element type %d", dtype);
  if (e != cudaSuccess) return ember_fail("moe_down: %s", cudaGetErrorString(e));
  return 0;
}
