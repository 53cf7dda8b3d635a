// A routed feed-forward (mixture of experts): every token runs `top` of E small feed-forwards and adds their
// results with weights from a router.
//
//   route          logits = W x in float32, scores = softmax(logits) over all experts, the `top` largest, their
//                  scores divided by their sum (+ eps); ties go to the smaller index.  (`route_topk`: from given logits.)
//   expert_plan    sorts the (token, choice) entries by expert: offsets per expert, a permutation slot -> entry and
//                  its inverse, and the list of row tiles (expert, first slot) that the products walk.  The order
//                  of entries inside an expert is whatever the atomics give; no result depends on it, since every
//                  entry's rows are computed on their own and added per token in the order of the choices.
//   grouped_gemm   C[slot, :] = act(A[row(slot), :] . W[expert(slot)]^T): one launch for all experts, a block per
//                  (row tile, column tile); blocks past the last tile leave.  bfloat16 on mma.sync tensor cores
//                  with float32 accumulators, float32 on the CUDA cores in k order.
//   expert_combine out[n, :] = sum_j weight[n, j] * Y[slot(n, j), :] (+ shared[n, :]), float32, in the order of j.
//
// Nothing here synchronises with the host or sizes a launch by the routing, so a step with routed layers can
// be recorded and replayed.
#include "common.cuh"

namespace {

constexpr int kMaxExperts = 1024;
constexpr int kMaxTop = 32;

// The choice of one token by one warp with scores sigmoid(logit): the `top` largest logits are chosen (the order of
// the scores, without the ties that a saturated sigmoid would make; equal logits go to the smaller index), and the
// weights are the chosen scores, divided by their sum + eps unless eps < 0, times `factor`.
template <typename F>
__device__ __forceinline__ void choose_experts_sigmoid(F logit, int E, int top, float eps, float factor, int lane,
                                                       int32_t* __restrict__ ids, float* __restrict__ weights) {
  constexpr int kPer = kMaxExperts / 32;
  float s[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) s[i] = (lane + 32 * i) < E ? logit(lane + 32 * i) : -INFINITY;
  float chosen_w = 0.f, total = 0.f;
  int chosen_e = -1;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPer; ++i)
      if (s[i] > best) {                 // ascending e within a lane: the first maximum is the smallest index
        best = s[i];
        best_e = lane + 32 * i;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kPer; ++i)
        if (lane + 32 * i == best_e) s[i] = -INFINITY;    // taken
    }
    const float score = 1.0f / (1.0f + expf(-best));
    if (lane == j) {
      chosen_w = score;
      chosen_e = best_e;
    }
    total += score;
  }
  if (lane < top) {
    ids[lane] = chosen_e;
    weights[lane] = (eps < 0.f ? chosen_w : chosen_w / (total + eps)) * factor;
  }
}

// The choice of one token by one warp: softmax over `logit(e)`, the `top` largest, renormalised.
template <typename F>
__device__ __forceinline__ void choose_experts(F logit, int E, int top, float eps, float factor, int lane,
                                               int32_t* __restrict__ ids, float* __restrict__ weights, int sigmoid = 0) {
  if (sigmoid) {
    choose_experts_sigmoid(logit, E, top, eps, factor, lane, ids, weights);
    return;
  }
  constexpr int kPer = kMaxExperts / 32;
  float s[kPer];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = lane + 32 * i;
    s[i] = e < E ? logit(e) : -INFINITY;
    m = fmaxf(m, s[i]);
  }
  m = warp_max(m);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    s[i] = (lane + 32 * i) < E ? expf(s[i] - m) : -1.f;    // -1: not an expert, never chosen
    if (s[i] > 0.f) sum += s[i];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int i = 0; i < kPer; ++i)
    if (s[i] >= 0.f) s[i] = s[i] / sum;
  float chosen_w = 0.f, total = 0.f;     // lane j keeps the j-th choice
  int chosen_e = -1;
  for (int j = 0; j < top; ++j) {
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPer; ++i)
      if (s[i] > best) {                 // ascending e within a lane: the first maximum is the smallest index
        best = s[i];
        best_e = lane + 32 * i;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kPer; ++i)
        if (lane + 32 * i == best_e) s[i] = -1.f;
    }
    if (lane == j) {
      chosen_w = best;
      chosen_e = best_e;
    }
    total += best;                       // the same on every lane, in the order of the choices
  }
  if (lane < top) {
    ids[lane] = chosen_e;
    // eps < 0: the chosen scores stand as they are (no division by their sum); `factor` multiplies either form
    weights[lane] = (eps < 0.f ? chosen_w : chosen_w / (total + eps)) * factor;
  }
}

// From given logits: one warp per token.
__global__ void route_topk_kernel(const float* __restrict__ logits, int E, int top, float eps, float factor,
                                  const int32_t* __restrict__ req_of_token, int32_t* __restrict__ ids,
                                  float* __restrict__ weights, int n_tokens, int sigmoid) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= n_tokens) return;
  if (req_of_token && req_of_token[n] < 0) {
    for (int j = lane; j < top; j += 32) {
      ids[(size_t)n * top + j] = -1;
      weights[(size_t)n * top + j] = 0.f;
    }
    return;
  }
  const float* z = logits + (size_t)n * E;
  choose_experts([&](int e) { return z[e]; }, E, top, eps, factor, lane, ids + (size_t)n * top, weights + (size_t)n * top, sigmoid);
}

// Four consecutive values of a row kept in shared memory (the address a multiple of four elements).
__device__ __forceinline__ void load4(const float* p, float& a, float& b, float& c, float& d) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  a = v.x; b = v.y; c = v.z; d = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float& a, float& b, float& c, float& d) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  a = lo.x; b = lo.y; c = hi.x; d = hi.y;
}

// The router whole: logits = W x in float32 (x may be bfloat16; sums per lane in k order, then a fixed butterfly) and
// the choice.  A block takes TOK tokens: their rows wait in shared memory in their own dtype, the warps share out
// the experts, and a row of the router read once serves all TOK tokens (each token's sum has the same order whatever
// TOK is); then warp t chooses for token t.
template <typename T, int TOK>
__global__ void route_kernel(const T* __restrict__ x, long x_stride, const float* __restrict__ w, int E, int K, int top,
                             float eps, float factor, const int32_t* __restrict__ req_of_token, int32_t* __restrict__ ids,
                             float* __restrict__ weights, int n_tokens, int sigmoid, const float* __restrict__ side,
                             float* __restrict__ side_out) {
  extern __shared__ __align__(16) unsigned char route_smem[];   // [TOK][K] rows (T), then [TOK][E] logits (float)
  T* xs = reinterpret_cast<T*>(route_smem);
  float* z = reinterpret_cast<float*>(route_smem + (((size_t)TOK * K * sizeof(T) + 15) & ~(size_t)15));
  pdl_launch_dependents();
  pdl_wait();
  const int n0 = blockIdx.x * TOK, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int here = min(TOK, n_tokens - n0);
  constexpr int kPiece = 16 / (int)sizeof(T);       // elements of a 16-byte piece
  if (K % kPiece == 0 && x_stride % kPiece == 0 && ((uintptr_t)x & 15) == 0) {
    const int pieces = K / kPiece;
    for (int i = threadIdx.x; i < TOK * pieces; i += blockDim.x) {
      const int t = i / pieces, k = (i - t * pieces) * kPiece;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);           // sixteen zero bytes are zeros in both types
      if (t < here) v = *reinterpret_cast<const uint4*>(x + (size_t)(n0 + t) * x_stride + k);
      *reinterpret_cast<uint4*>(xs + (size_t)t * K + k) = v;
    }
  } else {
    for (int i = threadIdx.x; i < TOK * K; i += blockDim.x) {
      const int t = i / K, k = i - t * K;
      xs[i] = t < here ? x[(size_t)(n0 + t) * x_stride + k] : from_f32<T>(0.f);
    }
  }
  __syncthreads();
  // four k a lane and load where rows allow it (k = 4 lane + 128 i: one order of sums for every TOK), else one
  const bool vec = (K & 3) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)side & 15) == 0;
  // `side` [K]: one more row beside the router's, whose sigmoid goes to side_out[n] (a gate per token that reads
  // the same rows; same order of sums as an expert's logit)
  for (int e = warp; e < E + (side ? 1 : 0); e += warps) {
    const float* wr = e < E ? w + (size_t)e * K : side;
    float acc[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[t] = 0.f;
    if (vec) {
#pragma unroll 2
      for (int k = 4 * lane; k < K; k += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(wr + k);
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          float x0, x1, x2, x3;
          load4(xs + (size_t)t * K + k, x0, x1, x2, x3);
          acc[t] = __fmaf_rn(wv.x, x0, acc[t]);
          acc[t] = __fmaf_rn(wv.y, x1, acc[t]);
          acc[t] = __fmaf_rn(wv.z, x2, acc[t]);
          acc[t] = __fmaf_rn(wv.w, x3, acc[t]);
        }
      }
    } else {
#pragma unroll 4
      for (int k = lane; k < K; k += 32) {
        const float wv = wr[k];
#pragma unroll
        for (int t = 0; t < TOK; ++t) acc[t] = __fmaf_rn(wv, to_f32<T>(xs[t * K + k]), acc[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      const float v = warp_sum(acc[t]);
      if (lane == 0) {
        if (e < E) z[t * E + e] = v;
        else if (t < here) side_out[n0 + t] = 1.0f / (1.0f + expf(-v));
      }
    }
  }
  __syncthreads();
  for (int t = warp; t < here; t += warps) {
    const int n = n0 + t;
    if (req_of_token && req_of_token[n] < 0) {
      for (int j = lane; j < top; j += 32) {
        ids[(size_t)n * top + j] = -1;
        weights[(size_t)n * top + j] = 0.f;
      }
      continue;
    }
    const float* zt = z + t * E;
    choose_experts([&](int e) { return zt[e]; }, E, top, eps, factor, lane, ids + (size_t)n * top, weights + (size_t)n * top, sigmoid);
  }
}

template <typename T, int TOK>
int launch_route(const void* x, long x_stride, const float* w, int n_tokens, int E, int K, int top, float eps, float factor,
                 const int32_t* req_of_token, int32_t* ids, float* weights, int sigmoid, const float* side, float* side_out,
                 cudaStream_t stream) {
  const size_t smem = (((size_t)TOK * K * sizeof(T) + 15) & ~(size_t)15) + (size_t)TOK * E * sizeof(float);
  if (smem > 200 * 1024) return YALIS_ERR_SHAPE;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(route_kernel<T, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return YALIS_ERR_LAUNCH;
    configured = smem;
  }
  return yalis_launch(route_kernel<T, TOK>, dim3((n_tokens + TOK - 1) / TOK), dim3(256), smem, stream, (const T*)x, x_stride, w, E, K,
                      top, eps, factor, req_of_token, ids, weights, n_tokens, sigmoid, side, side_out);
}

// One block.  entries = n_tokens * top.  tiles: (expert, first slot) per row tile of `bm` slots, ended by n_tiles.
__global__ void expert_plan_kernel(const int32_t* __restrict__ ids, int entries, int E, int bm, int32_t* __restrict__ offsets,
                                   int32_t* __restrict__ perm, int32_t* __restrict__ inv, int32_t* __restrict__ tile_expert,
                                   int32_t* __restrict__ tile_slot, int32_t* __restrict__ n_tiles) {
  __shared__ int count[kMaxExperts], start[kMaxExperts + 1], tile0[kMaxExperts + 1];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      tile0[e] = tiles;
      at += count[e];
      tiles += (count[e] + bm - 1) / bm;
    }
    start[E] = at;
    tile0[E] = tiles;
    *n_tiles = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = start[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int nt = tile0[e + 1] - tile0[e];
    for (int t = 0; t < nt; ++t) {
      tile_expert[tile0[e] + t] = e;
      tile_slot[tile0[e] + t] = start[e] + t * bm;
    }
    count[e] = 0;      // now the cursor
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) {
      const int slot = start[e] + atomicAdd(&count[e], 1);
      perm[slot] = i;
      inv[i] = slot;
    } else {
      inv[i] = -1;
    }
  }
}

// xg[slot, :] = x[perm[slot] / top, :] for the slots in use (16-byte pieces): the rows of every expert side by side,
// as a product that reads its rows as one box needs them.
__global__ void gather_rows_kernel(const uint4* __restrict__ x, long x_stride16, const int32_t* __restrict__ perm, int top,
                                   const int32_t* __restrict__ offsets, int E, uint4* __restrict__ out, int cols16) {
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x;
  if (slot >= offsets[E]) return;
  const int row = perm[slot] / top;
  for (int c = threadIdx.x; c < cols16; c += blockDim.x) out[(size_t)slot * cols16 + c] = x[(size_t)row * x_stride16 + c];
}

// xg[slot, :] = x[perm[slot] / top, :] * weights[perm[slot]] in any dtype: the rows of every expert side by side,
// each times the weight of its (token, choice) entry (weights null: 1), float32 product, one rounding.
template <typename T>
__global__ void gather_scale_rows_kernel(const T* __restrict__ x, long x_stride, const int32_t* __restrict__ perm, int top,
                                         const float* __restrict__ weights, const int32_t* __restrict__ offsets, int E,
                                         T* __restrict__ out, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x;
  if (slot >= offsets[E]) return;
  const int entry = perm[slot], row = entry / top;
  const float wgt = weights ? weights[entry] : 1.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    out[(size_t)slot * cols + c] = from_f32<T>(to_f32<T>(x[(size_t)row * x_stride + c]) * wgt);
}

// The same for bfloat16 rows on 16-byte boundaries, eight columns a thread (same product and rounding per element).
__global__ void gather_scale_rows_bf16x8_kernel(const uint4* __restrict__ x, long x_stride16, const int32_t* __restrict__ perm,
                                                int top, const float* __restrict__ weights, const int32_t* __restrict__ offsets,
                                                int E, uint4* __restrict__ out, int cols16) {
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x;
  if (slot >= offsets[E]) return;
  const int entry = perm[slot], row = entry / top;
  const float wgt = weights ? weights[entry] : 1.0f;
  for (int c = threadIdx.x; c < cols16; c += blockDim.x) {
    uint4 raw = x[(size_t)row * x_stride16 + c];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      h[i] = __floats2bfloat162_rn(v.x * wgt, v.y * wgt);
    }
    out[(size_t)slot * cols16 + c] = raw;
  }
}

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) {            // the square of relu
    v = fmaxf(v, 0.f);
    return v * v;
  }
  return v;
}

struct GroupedArgs {
  const void* a; long a_stride;       // [rows, K]
  const int32_t* perm; int top;       // row of slot s: perm[s] / top (perm null: the slot itself)
  const void* w;                      // [E, n_out, K]
  void* c; long c_stride;             // [slots, n_out]
  const int32_t* offsets; const int32_t* tile_expert; const int32_t* tile_slot; const int32_t* n_tiles;
  int n_out, K, act;
};

// float32 (or any dtype without alignment demands): 32 x 64 tile, 256 threads, 2 x 4 outputs a thread.
template <typename T>
__global__ void grouped_gemm_simt_kernel(const GroupedArgs g) {
  constexpr int BM = 32, BN = 64, BK = 16;
  __shared__ float As[BM][BK + 1], Bs[BN][BK + 1];
  __shared__ int rows[BM];
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.x >= *g.n_tiles) return;
  const int e = g.tile_expert[blockIdx.x], slot0 = g.tile_slot[blockIdx.x];
  const int m_rows = min(BM, g.offsets[e + 1] - slot0);
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  if (tid < BM) rows[tid] = tid < m_rows ? (g.perm ? g.perm[slot0 + tid] / g.top : slot0 + tid) : -1;
  __syncthreads();
  const T* A = reinterpret_cast<const T*>(g.a);
  const T* W = reinterpret_cast<const T*>(g.w) + (size_t)e * g.n_out * g.K;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < g.K; k0 += BK) {
    for (int i = tid; i < BM * BK; i += 256) {
      const int r = i / BK, k = i % BK;
      As[r][k] = (rows[r] >= 0 && k0 + k < g.K) ? to_f32<T>(A[(size_t)rows[r] * g.a_stride + k0 + k]) : 0.f;
    }
    for (int i = tid; i < BN * BK; i += 256) {
      const int r = i / BK, k = i % BK;
      Bs[r][k] = (n0 + r < g.n_out && k0 + k < g.K) ? to_f32<T>(W[(size_t)(n0 + r) * g.K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(As[ty * 2 + i][k], Bs[tx + 16 * j][k], acc[i][j]);
    }
    __syncthreads();
  }
  T* C = reinterpret_cast<T*>(g.c);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= m_rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx + 16 * j;
      if (c < g.n_out) C[(size_t)(slot0 + r) * g.c_stride + c] = from_f32<T>(apply_act(acc[i][j], g.act));
    }
  }
}

// bfloat16 on mma.sync.m16n8k16 with ldmatrix-fed fragments: a BM x BN tile per block, K in steps of 64 through a
// ring of cp.async stages.  Two shapes: 128 x 128 with 8 warps (64 x 32 each) and 3 stages for steps in which an
// expert gets many tokens, and 32 x 64 (5 stages) or 16 x 64 (8 stages) with 4 warps for steps of few tokens, where
// the weights stream through once and what counts is how many bytes are in flight (16 rows: 112 KB an SM).  Needs K % 8 == 0 and 16-byte
// aligned rows of A and W.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}

template <int BM, int BN, int BK, int WARPS_M, int WARPS_N, int STAGES>
__global__ void __launch_bounds__(32 * WARPS_M * WARPS_N) grouped_gemm_mma_kernel(const GroupedArgs g) {
  constexpr int LD = BK + 8, CH = BK / 8;               // rows of 80 or 144 bytes: ldmatrix reads 8 distinct 16-byte lanes
  constexpr int THREADS = 32 * WARPS_M * WARPS_N;
  constexpr int WTM = BM / WARPS_M, WTN = BN / WARPS_N, MT = WTM / 16, NT = WTN / 8;
  static_assert(WTM % 16 == 0 && WTN % 16 == 0, "warp tiles are made of 16 x 16 pieces");
  extern __shared__ __align__(16) unsigned char gg_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(gg_smem);                 // [STAGES][BM][LD]
  __nv_bfloat16* Bs = As + (size_t)STAGES * BM * LD;                            // [STAGES][BN][LD]
  int* rows = reinterpret_cast<int*>(Bs + (size_t)STAGES * BN * LD);            // [BM]
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.x >= *g.n_tiles) return;
  const int e = g.tile_expert[blockIdx.x], slot0 = g.tile_slot[blockIdx.x];
  const int m_rows = min(BM, g.offsets[e + 1] - slot0);
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / WARPS_N, wn = warp % WARPS_N;
  for (int i = tid; i < BM; i += THREADS) rows[i] = i < m_rows ? (g.perm ? g.perm[slot0 + i] / g.top : slot0 + i) : -1;
  __syncthreads();
  const __nv_bfloat16* A = reinterpret_cast<const __nv_bfloat16*>(g.a);
  const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(g.w) + (size_t)e * g.n_out * g.K;
  const int steps = (g.K + BK - 1) / BK;

  auto load = [&](int step) {
    if (step < steps) {
      const int stage = step % STAGES, k0 = step * BK;
      __nv_bfloat16* as = As + (size_t)stage * BM * LD;
      __nv_bfloat16* bs = Bs + (size_t)stage * BN * LD;
      for (int i = tid; i < BM * CH; i += THREADS) {
        const int r = i / CH, ch = i % CH;
        const bool ok = rows[r] >= 0 && k0 + ch * 8 < g.K;
        cp_async16(as + r * LD + ch * 8, ok ? A + (size_t)rows[r] * g.a_stride + k0 + ch * 8 : A, ok);
      }
      for (int i = tid; i < BN * CH; i += THREADS) {
        const int r = i / CH, ch = i % CH;
        const bool ok = n0 + r < g.n_out && k0 + ch * 8 < g.K;
        cp_async16(bs + r * LD + ch * 8, ok ? W + (size_t)(n0 + r) * g.K + k0 + ch * 8 : W, ok);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // a group per step, empty past the end: the count below holds
  };

  float acc[MT][NT][4] = {};
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) load(st);
  for (int step = 0; step < steps; ++step) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();                                       // step's tile is in place; everyone is done with step - 1
    load(step + STAGES - 1);                               // into the stage that step - 1 used
    const __nv_bfloat16* as = As + (size_t)(step % STAGES) * BM * LD;
    const __nv_bfloat16* bs = Bs + (size_t)(step % STAGES) * BN * LD;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t af[MT][4], bf[NT][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const unsigned addr = (unsigned)__cvta_generic_to_shared(as + (wm * WTM + mt * 16 + (lane & 15)) * LD + kk + (lane >> 4) * 8);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(af[mt][0]), "=r"(af[mt][1]), "=r"(af[mt][2]), "=r"(af[mt][3]) : "r"(addr));
      }
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        const unsigned addr = (unsigned)__cvta_generic_to_shared(
            bs + (wn * WTN + np * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + kk + ((lane >> 3) & 1) * 8);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(bf[2 * np][0]), "=r"(bf[2 * np][1]), "=r"(bf[2 * np + 1][0]), "=r"(bf[2 * np + 1][1]) : "r"(addr));
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                       : "+f"(acc[mt][nt][0]), "+f"(acc[mt][nt][1]), "+f"(acc[mt][nt][2]), "+f"(acc[mt][nt][3])
                       : "r"(af[mt][0]), "r"(af[mt][1]), "r"(af[mt][2]), "r"(af[mt][3]), "r"(bf[nt][0]), "r"(bf[nt][1]));
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(g.c);
  const int gq = lane >> 2, tq = lane & 3;
  const bool pairs = (g.c_stride & 1) == 0 && ((uintptr_t)C & 3) == 0;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * WTM + mt * 16 + gq + half * 8;
      if (r >= m_rows) continue;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int c = n0 + wn * WTN + nt * 8 + 2 * tq;
        __nv_bfloat16* dst = C + (size_t)(slot0 + r) * g.c_stride + c;
        const float v0 = apply_act(acc[mt][nt][half * 2], g.act), v1 = apply_act(acc[mt][nt][half * 2 + 1], g.act);
        if (pairs && c + 1 < g.n_out) {
          *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);
        } else {
          if (c < g.n_out) dst[0] = __float2bfloat16_rn(v0);
          if (c + 1 < g.n_out) dst[1] = __float2bfloat16_rn(v1);
        }
      }
    }
}

template <int BM, int BN, int BK, int WARPS_M, int WARPS_N, int STAGES>
int launch_grouped_mma(const GroupedArgs& g, int max_tiles, cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * (BM + BN) * (BK + 8) * 2 + BM * 4;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(grouped_gemm_mma_kernel<BM, BN, BK, WARPS_M, WARPS_N, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return YALIS_ERR_LAUNCH;
    configured = true;
  }
  const dim3 grid(max_tiles, (g.n_out + BN - 1) / BN);
  if (grid.y > 65535) return YALIS_ERR_SHAPE;
  return yalis_launch(grouped_gemm_mma_kernel<BM, BN, BK, WARPS_M, WARPS_N, STAGES>, grid, dim3(32 * WARPS_M * WARPS_N), smem, stream, g);
}

// out[n, :] = sum_j weights[n, j] * y[inv[n * top + j], :] + shared[n, :]
template <typename T>
__global__ void expert_combine_kernel(const T* __restrict__ y, long y_stride, const int32_t* __restrict__ inv,
                                      const float* __restrict__ weights, int top, const T* __restrict__ shared,
                                      long shared_stride, T* __restrict__ out, long out_stride, int cols,
                                      const float* __restrict__ shared_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < cols; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const int slot = inv[(size_t)n * top + j];
      if (slot >= 0) acc = __fmaf_rn(weights ? weights[(size_t)n * top + j] : 1.0f, to_f32<T>(y[(size_t)slot * y_stride + c]), acc);
    }
    if (shared) acc = __fmaf_rn(shared_scale ? shared_scale[n] : 1.0f, to_f32<T>(shared[(size_t)n * shared_stride + c]), acc);
    out[(size_t)n * out_stride + c] = from_f32<T>(acc);
  }
}

// The same for bfloat16 rows on 16-byte boundaries: 8 columns a thread, the same order of sums per column.
__global__ void expert_combine_bf16x8_kernel(const __nv_bfloat16* __restrict__ y, long y_stride, const int32_t* __restrict__ inv,
                                             const float* __restrict__ weights, int top, const __nv_bfloat16* __restrict__ shared,
                                             long shared_stride, __nv_bfloat16* __restrict__ out, long out_stride, int cols,
                                             const float* __restrict__ shared_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= cols) return;
  float acc[8] = {};
  for (int j = 0; j < top; ++j) {
    const int slot = inv[(size_t)n * top + j];
    if (slot < 0) continue;
    const float wj = weights ? weights[(size_t)n * top + j] : 1.0f;
    const uint4 raw = *reinterpret_cast<const uint4*>(y + (size_t)slot * y_stride + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      acc[2 * i] = __fmaf_rn(wj, v.x, acc[2 * i]);
      acc[2 * i + 1] = __fmaf_rn(wj, v.y, acc[2 * i + 1]);
    }
  }
  if (shared) {
    const uint4 raw = *reinterpret_cast<const uint4*>(shared + (size_t)n * shared_stride + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float ws = shared_scale ? shared_scale[n] : 1.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      acc[2 * i] = __fmaf_rn(ws, v.x, acc[2 * i]);
      acc[2 * i + 1] = __fmaf_rn(ws, v.y, acc[2 * i + 1]);
    }
  }
  uint4 res;
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  *reinterpret_cast<uint4*>(out + (size_t)n * out_stride + c) = res;
}

}  // namespace

YALIS_API int yalis_route_topk(const float* logits, int n_tokens, int E, int top, float eps, float factor, const int32_t* req_of_token,
                               int32_t* ids, float* weights, int sigmoid, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (E <= 0 || E > kMaxExperts || top <= 0 || top > kMaxTop || top > E) return YALIS_ERR_SHAPE;
  const int warps = 4;
  return yalis_launch(route_topk_kernel, dim3((n_tokens + warps - 1) / warps), dim3(32 * warps), 0, stream, logits, E, top,
                      eps, factor, req_of_token, ids, weights, n_tokens, sigmoid);
}

// The router and the choice in one launch.  x: [n_tokens, K] float32 or bfloat16; w: float32 [E, K].  Steps of a
// thousand tokens and more take eight to a block where their rows fit shared memory (fewer tokens would leave SMs
// without a block: 64 tokens in 8 blocks took 48 us, in 64 blocks 13).
YALIS_API int yalis_route(const void* x, int x_dtype, long x_stride, const float* w, int n_tokens, int E, int K, int top, float eps, float factor,
                          const int32_t* req_of_token, int32_t* ids, float* weights, int sigmoid, const float* side,
                          float* side_out, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (E <= 0 || E > kMaxExperts || top <= 0 || top > kMaxTop || top > E || K <= 0) return YALIS_ERR_SHAPE;
  if ((side == nullptr) != (side_out == nullptr)) return YALIS_ERR_SHAPE;
  const size_t elt = x_dtype == YALIS_BF16 ? 2 : 4;
  const bool many = n_tokens >= 1024 && 8 * ((size_t)K * elt + (size_t)E * 4) + 16 <= 96 * 1024;
  YALIS_DISPATCH_DTYPE(x_dtype, T,
                       return many ? launch_route<T, 8>(x, x_stride, w, n_tokens, E, K, top, eps, factor, req_of_token, ids, weights, sigmoid, side, side_out, stream)
                                   : launch_route<T, 1>(x, x_stride, w, n_tokens, E, K, top, eps, factor, req_of_token, ids, weights, sigmoid, side, side_out, stream));
  return YALIS_OK;
}

YALIS_API int yalis_expert_plan(const int32_t* ids, int entries, int E, int bm, int32_t* offsets, int32_t* perm,
                                int32_t* inv, int32_t* tile_expert, int32_t* tile_slot, int32_t* n_tiles,
                                cudaStream_t stream) {
  if (entries <= 0) return YALIS_OK;
  if (E <= 0 || E > kMaxExperts || bm <= 0) return YALIS_ERR_SHAPE;
  return yalis_launch(expert_plan_kernel, dim3(1), dim3(1024), 0, stream, ids, entries, E, bm, offsets, perm, inv,
                      tile_expert, tile_slot, n_tiles);
}

// bm: the row tile the plan was made for (16, 32 or 128 for the tensor-core form, 32 for the other).
YALIS_API int yalis_grouped_gemm(const void* a, long a_stride, const int32_t* perm, int top, const void* w, void* c,
                                 long c_stride, int dtype, const int32_t* offsets, const int32_t* tile_expert,
                                 const int32_t* tile_slot, const int32_t* n_tiles, int max_tiles, int n_out, int K, int act,
                                 int bm, int tensor_cores, cudaStream_t stream) {
  if (max_tiles <= 0) return YALIS_OK;
  if (n_out <= 0 || K <= 0 || top <= 0 || (n_out + 63) / 64 > 65535) return YALIS_ERR_SHAPE;
  GroupedArgs g;
  g.a = a; g.a_stride = a_stride; g.perm = perm; g.top = top; g.w = w; g.c = c; g.c_stride = c_stride; g.offsets = offsets;
  g.tile_expert = tile_expert; g.tile_slot = tile_slot; g.n_tiles = n_tiles; g.n_out = n_out; g.K = K; g.act = act;
  const dim3 grid(max_tiles, (n_out + 63) / 64);
  if (tensor_cores) {
    if (dtype != YALIS_BF16) return YALIS_ERR_DTYPE;
    if (K % 8 || a_stride % 8 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return YALIS_ERR_ALIGN;
    if (bm == 16) return launch_grouped_mma<16, 64, 64, 1, 4, 8>(g, max_tiles, stream);
    if (bm == 32) return launch_grouped_mma<32, 64, 64, 1, 4, 5>(g, max_tiles, stream);
    if (bm == 128) return launch_grouped_mma<128, 128, 64, 2, 4, 3>(g, max_tiles, stream);
    return YALIS_ERR_SHAPE;
  }
  if (bm != 32) return YALIS_ERR_SHAPE;
  YALIS_DISPATCH_DTYPE(dtype, T, return yalis_launch(grouped_gemm_simt_kernel<T>, grid, dim3(256), 0, stream, g));
  return YALIS_OK;
}

// bfloat16 rows of K % 8 == 0 columns on 16-byte boundaries; out contiguous [entries, K].
YALIS_API int yalis_gather_rows(const void* x, long x_stride, const int32_t* perm, int top, const int32_t* offsets, int E,
                                void* out, int entries, int K, cudaStream_t stream) {
  if (entries <= 0) return YALIS_OK;
  if (K % 8 || x_stride % 8 || ((uintptr_t)x & 15) || ((uintptr_t)out & 15) || top <= 0) return YALIS_ERR_ALIGN;
  return yalis_launch(gather_rows_kernel, dim3(entries), dim3(K / 8 < 256 ? ((K / 8 + 31) / 32) * 32 : 256), 0, stream,
                      (const uint4*)x, x_stride / 8, perm, top, offsets, E, (uint4*)out, K / 8);
}

// Any dtype; `weights` float32 [n_tokens * top] or null.
YALIS_API int yalis_gather_scale_rows(const void* x, long x_stride, int dtype, const int32_t* perm, int top, const float* weights,
                                      const int32_t* offsets, int E, void* out, int entries, int K, cudaStream_t stream) {
  if (entries <= 0) return YALIS_OK;
  if (top <= 0 || K <= 0) return YALIS_ERR_SHAPE;
  if (dtype == YALIS_BF16 && K % 8 == 0 && x_stride % 8 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)out & 15))
    return yalis_launch(gather_scale_rows_bf16x8_kernel, dim3(entries), dim3(K / 8 < 256 ? ((K / 8 + 31) / 32) * 32 : 256), 0, stream,
                        (const uint4*)x, x_stride / 8, perm, top, weights, offsets, E, (uint4*)out, K / 8);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(gather_scale_rows_kernel<T>, dim3(entries), dim3(K < 256 ? ((K + 31) / 32) * 32 : 256), 0,
                                           stream, (const T*)x, x_stride, perm, top, weights, offsets, E, (T*)out, K));
  return YALIS_OK;
}

// `weights` null: every choice counts once.  `shared_scale` float32 [n_tokens] or null: a factor per token on `shared`.
YALIS_API int yalis_expert_combine(const void* y, long y_stride, const int32_t* inv, const float* weights, int top,
                                   const void* shared, long shared_stride, void* out, long out_stride, int dtype,
                                   int n_tokens, int cols, const float* shared_scale, cudaStream_t stream) {
  if (n_tokens <= 0 || cols <= 0) return YALIS_OK;
  if (top <= 0) return YALIS_ERR_SHAPE;
  const bool aligned = dtype == YALIS_BF16 && cols % 8 == 0 && y_stride % 8 == 0 && out_stride % 8 == 0 && shared_stride % 8 == 0 &&
                       !((uintptr_t)y & 15) && !((uintptr_t)out & 15) && !((uintptr_t)shared & 15);
  if (aligned)
    return yalis_launch(expert_combine_bf16x8_kernel, dim3(n_tokens, (cols / 8 + 127) / 128), dim3(128), 0, stream,
                        (const __nv_bfloat16*)y, y_stride, inv, weights, top, (const __nv_bfloat16*)shared, shared_stride,
                        (__nv_bfloat16*)out, out_stride, cols, shared_scale);
  const int col_blocks = (cols + 1023) / 1024;
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(expert_combine_kernel<T>, dim3(n_tokens, col_blocks), dim3(256), 0, stream, (const T*)y,
                                           y_stride, inv, weights, top, (const T*)shared, shared_stride, (T*)out,
                                           out_stride, cols, shared_scale));
  return YALIS_OK;
}
