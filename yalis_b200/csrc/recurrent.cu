// Mixers that keep a matrix per head instead of keys and values: linear recurrences
// over a float32 state S [dim, vdim] per (request, head),
//
//   S <- diag(g_t) S                      g_t: a constant per head, a scalar per token, or a vector over dim
//   u  = beta_t (v_t - S^T k_t)           (delta rule)        or   u = v_t   (plain outer-product write)
//   S <- S + k_t u^T
//   o_t = S^T q_t                         (the read-out sees the token's own write)
//
// and the generalized delta rule, whose decay and removal both read the OLD state,
//
//   S <- diag(g_t) S - (a_t * u_t)(u_t^T S) + k_t v_t^T,   o_t = S^T q_t
//
// with a unit key u_t and a removal rate a_t per head and key channel,
//
// with the short causal convolution that feeds some of them and the per-head norm and gate
// that follow them.  Everything here is float32 arithmetic whatever the model's dtype; the
// state and the convolution's tail live in the per-request slot memory of the cache manager.
//
// The columns of S are independent of one another (column j only ever meets v_j), so a thread
// owns 8 (or 16) rows of one column in registers, the lanes that share a column sit in one warp, and
// a block walks the tokens of one request in order: a portion of a prompt and a single
// decoded token are the same loop, and the result for a token does not depend on how the
// request was cut into steps or on what else is in the batch.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---- what the delta rule reads: convolution, unit length, decay and write strength ------------------
//   y_t[c] = silu(sum_j w[c][K-1-j] x_(t-j)[c]),  x before the request's start = 0
// The last K-1 inputs of every request are kept in its slot: tail[c][0..K-2], oldest first.
// With kv_heads > 0 the first 2 * kv_heads * dim channels are the heads of q and then of k: each head is
// brought to unit length, x / sqrt(sum x^2 + eps), and q multiplied by q_scale.  With a_raw the decay
// g = exp(-exp(a_log[h]) * softplus(a_raw + dt_bias)) (per head, or per head and key channel) and the write
// strength beta = sigmoid(b_raw) are computed beside it, in float32.
constexpr int kMaxTaps = 16;

template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                                     const float* __restrict__ tail, size_t slot_stride,
                                     const int32_t* __restrict__ req_of_token, const int32_t* __restrict__ q_start,
                                     const int32_t* __restrict__ slots, float* __restrict__ out, int out_stride,
                                     int channels, int taps, int kv_heads, int dim, float q_scale, float unit_eps,
                                     const T* __restrict__ a_raw, int a_stride, int a_cols,
                                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     const T* __restrict__ b_raw, int b_stride, int heads, float* __restrict__ g_out,
                                     float* __restrict__ beta_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int req = req_of_token[n];
  if (req < 0) return;
  const int i = n - q_start[req];                 // index of the token in its request's portion
  const float* tl = tail + (size_t)slots[req] * slot_stride;
  float* row = out + (size_t)n * out_stride;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    float acc = 0.f;
    for (int j = taps - 1; j >= 0; --j) {         // oldest input first: a fixed order of additions
      float xv;
      if (i - j >= 0) xv = to_f32<T>(x[(size_t)(n - j) * x_stride + c]);
      else xv = tl[(size_t)c * (taps - 1) + (taps - 1 + i - j)];
      acc = __fmaf_rn(w[(size_t)c * taps + (taps - 1 - j)], xv, acc);
    }
    row[c] = silu_exact(acc);
  }
  if (a_raw != nullptr) {
    const int per = a_cols / heads;               // 1, or dim
    for (int c = threadIdx.x; c < a_cols; c += blockDim.x) {
      const float a = to_f32<T>(a_raw[(size_t)n * a_stride + c]) + dt_bias[c];
      g_out[(size_t)n * a_cols + c] = expf(-expf(a_log[c / per]) * softplus_f(a));
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x)
      beta_out[(size_t)n * heads + h] = sigmoid_f(to_f32<T>(b_raw[(size_t)n * b_stride + h]));
  }
  if (kv_heads > 0) {
    __syncthreads();                              // the block reads back what it wrote itself
    const int lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int hh = threadIdx.x >> 5; hh < 2 * kv_heads; hh += nw) {     // q heads, then k heads
      float* v = row + (size_t)hh * dim;
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = __fmaf_rn(v[d], v[d], ss);
      ss = warp_sum(ss);
      const float r = (hh < kv_heads ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
      for (int d = lane; d < dim; d += 32) v[d] *= r;
    }
  }
}

// After the step: the tail becomes the last K-1 inputs the request has seen.
template <typename T>
__global__ void short_conv_tail_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ tail,
                                       size_t slot_stride, const int32_t* __restrict__ q_start,
                                       const int32_t* __restrict__ slots, int channels, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int req = blockIdx.x;
  const int a = q_start[req], q_len = q_start[req + 1] - a;
  if (q_len <= 0) return;
  float* tl = tail + (size_t)slots[req] * slot_stride;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float nv[kMaxTaps];
#pragma unroll
    for (int m = 0; m < kMaxTaps; ++m) {
      if (m < keep) {
        const int i = q_len - keep + m;           // index in the portion of the input that lands at place m
        nv[m] = i >= 0 ? to_f32<T>(x[(size_t)(a + i) * x_stride + c]) : tl[(size_t)c * keep + (m + q_len)];
      }
    }
#pragma unroll
    for (int m = 0; m < kMaxTaps; ++m)
      if (m < keep) tl[(size_t)c * keep + m] = nv[m];
  }
}

// ---- the recurrence ------------------------------------------------------------------------------
constexpr int kScanThreads = 128;
constexpr int kMaxTile = 16;         // tokens staged in shared memory at a time

struct ScanParams {
  const float* q; int q_stride;      // [N, kv_heads * dim]
  const float* k; int k_stride;
  const float* v; int v_stride;      // [N, heads * vdim]
  const float* decay;                // DECAY 0: [heads]; 1: [N, heads]; 2: [N, heads * dim]
  const float* beta;                 // RULE 1: [N, heads]
  const float* unit;                 // RULE 2: unit keys u [N, heads * dim]
  const float* removal;              // RULE 2: a * u [N, heads * dim]
  float* state; size_t slot_stride;  // per slot: [heads][vdim][dim_padded]
  float* out; int out_stride;        // [N, heads * vdim]
  const int32_t* q_start; const int32_t* slots;
  int heads, kv_heads, dim, dim_padded, vdim, lanes, tile;
  int wide;                          // 1: rows of q, k and the decay may be copied 16 bytes at a time
};

__device__ __forceinline__ void copy_async4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void copy_async16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// RULE: 0 plain outer-product write, 1 delta rule, 2 generalized delta rule (needs DECAY 2).
// DECAY: 0 constant per head, 1 scalar per token and head, 2 vector per token, head and key channel.
// ROWS: rows of a column that a thread keeps (8: twice the warps, which hide each other's waits; 16: dim up to 512).
// The tokens of a request are staged through two buffers in shared memory: while one tile is walked, the
// asynchronous copies of the next are in flight.
// LANES: lanes that share a column (a power of two up to 32; ROWS * LANES >= dim).
template <int ROWS, int LANES, int RULE, int DECAY>
__global__ void __launch_bounds__(kScanThreads) state_scan_kernel(const ScanParams p) {
  extern __shared__ __align__(16) float sm[];
  constexpr int Q = ROWS / 4;          // 16-byte pieces of a column per thread
  pdl_launch_dependents();
  pdl_wait();
  const int req = blockIdx.z, h = blockIdx.y;
  const int t_begin = p.q_start[req], q_len = p.q_start[req + 1] - t_begin;
  if (q_len <= 0) return;
  constexpr int L = LANES, cols = kScanThreads / L, width = ROWS * L;
  const int tid = threadIdx.x, l = tid % L, c = tid / L;
  const int j = blockIdx.x * cols + c;
  const bool live = j < p.vdim;
  const int kvh = h / (p.heads / p.kv_heads);
  const int D = p.dim, Dp = p.dim_padded, V = p.vdim, TT = p.tile;
  constexpr bool DELTA = RULE == 1;
  // one buffer: q [TT][width], k [TT][width], decay vectors [TT][width] (DECAY 2), unit keys and removal vectors
  // [TT][width] each (RULE 2), v [TT][cols], beta [TT], decay [TT]
  constexpr int vec_cols = RULE == 2 ? 5 : (DECAY == 2 ? 3 : 2);
  const size_t buf_floats = ((size_t)vec_cols * TT * width + (size_t)TT * cols + 2 * TT + 3) & ~(size_t)3;
  // behind the two buffers: every lane's share of a read-out, [TT][cols][L + 1]; the shares are added after the
  // tile is walked, off the chain from one token's state to the next
  float* shares = sm + 2 * buf_floats;

  // what no copy ever writes: the rows past dim (zeros; ones for the decay)
  const int pad = width - D;
  for (int e = tid; e < 2 * vec_cols * TT * pad; e += kScanThreads) {
    const int row = e / pad, d = D + (e - row * pad);          // row: (buffer, array, token)
    const int b = row / (vec_cols * TT), r = row - b * (vec_cols * TT);
    sm[(size_t)b * buf_floats + (size_t)r * width + d] = (r / TT) == 2 ? 1.f : 0.f;
  }

  auto issue = [&](int t0, int b) {
    float* qs = sm + (size_t)b * buf_floats;
    float* ks = qs + (size_t)TT * width;
    float* gv = ks + (size_t)TT * width;
    float* uv = gv + (size_t)TT * width;
    float* av = uv + (size_t)TT * width;
    float* vs = qs + (size_t)vec_cols * TT * width;
    float* bs = vs + (size_t)TT * cols;
    float* gs = bs + TT;
    const int tt = min(TT, q_len - t0);
    if (p.wide) {
      const int quads = D >> 2;
      for (int e = tid; e < tt * quads; e += kScanThreads) {
        const int t = e / quads, d = (e - t * quads) << 2;
        const size_t n = (size_t)(t_begin + t0 + t);
        copy_async16(qs + t * width + d, p.q + n * p.q_stride + (size_t)kvh * D + d);
        copy_async16(ks + t * width + d, p.k + n * p.k_stride + (size_t)kvh * D + d);
        if (DECAY == 2) copy_async16(gv + t * width + d, p.decay + (n * p.heads + h) * D + d);
        if (RULE == 2) {
          copy_async16(uv + t * width + d, p.unit + (n * p.heads + h) * D + d);
          copy_async16(av + t * width + d, p.removal + (n * p.heads + h) * D + d);
        }
      }
    } else {
      for (int e = tid; e < tt * D; e += kScanThreads) {
        const int t = e / D, d = e - t * D;
        const size_t n = (size_t)(t_begin + t0 + t);
        copy_async4(qs + t * width + d, p.q + n * p.q_stride + (size_t)kvh * D + d);
        copy_async4(ks + t * width + d, p.k + n * p.k_stride + (size_t)kvh * D + d);
        if (DECAY == 2) copy_async4(gv + t * width + d, p.decay + (n * p.heads + h) * D + d);
        if (RULE == 2) {
          copy_async4(uv + t * width + d, p.unit + (n * p.heads + h) * D + d);
          copy_async4(av + t * width + d, p.removal + (n * p.heads + h) * D + d);
        }
      }
    }
    for (int e = tid; e < tt * cols; e += kScanThreads) {
      const int t = e / cols, cc = e - t * cols;
      const int jj = blockIdx.x * cols + cc;
      if (jj < V) copy_async4(vs + e, p.v + (size_t)(t_begin + t0 + t) * p.v_stride + (size_t)h * V + jj);
      else vs[e] = 0.f;
    }
    if (tid < tt) {
      const size_t n = (size_t)(t_begin + t0 + tid);
      if (DELTA) copy_async4(bs + tid, p.beta + n * p.heads + h);
      if (DECAY == 1) copy_async4(gs + tid, p.decay + n * p.heads + h);
    }
    copy_async_commit();
  };

  float* sp = p.state + (size_t)p.slots[req] * p.slot_stride + ((size_t)h * V + (live ? j : 0)) * Dp;
  float S[ROWS];
#pragma unroll
  for (int i = 0; i < Q; ++i) {
    const int d = (i * L + l) * 4;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && d < Dp) x = *reinterpret_cast<const float4*>(sp + d);
    S[4 * i] = x.x; S[4 * i + 1] = x.y; S[4 * i + 2] = x.z; S[4 * i + 3] = x.w;
  }
  const float g_const = DECAY == 0 ? p.decay[h] : 1.f;

  issue(0, 0);
  int b = 0;
  for (int t0 = 0; t0 < q_len; t0 += TT, b ^= 1) {
    const int tt = min(TT, q_len - t0);
    if (t0 + TT < q_len) {
      issue(t0 + TT, b ^ 1);
      copy_async_wait<1>();
    } else {
      copy_async_wait<0>();
    }
    __syncthreads();
    const float* qs = sm + (size_t)b * buf_floats;
    const float* vs = qs + (size_t)vec_cols * TT * width;
    const float* bs = vs + (size_t)TT * cols;
    const float* gs = bs + TT;
    const float* qp = qs + l * 4;                          // this lane's first piece of q; k and the decay follow
    const float* kp = qp + (size_t)TT * width;
    const float* gp = kp + (size_t)TT * width;
    for (int t = 0; t < tt; ++t, qp += width, kp += width, gp += width) {
      float kr[ROWS], qr[ROWS];
#pragma unroll
      for (int i = 0; i < Q; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(kp + i * L * 4);
        const float4 bq = *reinterpret_cast<const float4*>(qp + i * L * 4);
        kr[4 * i] = a.x; kr[4 * i + 1] = a.y; kr[4 * i + 2] = a.z; kr[4 * i + 3] = a.w;
        qr[4 * i] = bq.x; qr[4 * i + 1] = bq.y; qr[4 * i + 2] = bq.z; qr[4 * i + 3] = bq.w;
      }
      if (RULE == 2) {
        // both the decay and the removal read the old state: the dot product u . S first (pairs, then a fixed tree
        // and a butterfly over the lanes), then every row in one expression, then the read-out as in the other rules
        const float* up = gp + (size_t)TT * width;
        const float* ap = up + (size_t)TT * width;
        float ur[ROWS], ar[ROWS], gr[ROWS];
#pragma unroll
        for (int i = 0; i < Q; ++i) {
          const float4 a = *reinterpret_cast<const float4*>(up + i * L * 4);
          const float4 b2 = *reinterpret_cast<const float4*>(ap + i * L * 4);
          const float4 g = *reinterpret_cast<const float4*>(gp + i * L * 4);
          ur[4 * i] = a.x; ur[4 * i + 1] = a.y; ur[4 * i + 2] = a.z; ur[4 * i + 3] = a.w;
          ar[4 * i] = b2.x; ar[4 * i + 1] = b2.y; ar[4 * i + 2] = b2.z; ar[4 * i + 3] = b2.w;
          gr[4 * i] = g.x; gr[4 * i + 1] = g.y; gr[4 * i + 2] = g.z; gr[4 * i + 3] = g.w;
        }
        float part[ROWS / 2];
#pragma unroll
        for (int i = 0; i < ROWS / 2; ++i) part[i] = __fmaf_rn(S[2 * i + 1], ur[2 * i + 1], S[2 * i] * ur[2 * i]);
#pragma unroll
        for (int w = ROWS / 4; w >= 1; w >>= 1)
#pragma unroll
          for (int i = 0; i < w; ++i) part[i] += part[i + w];
        float dot = part[0];
#pragma unroll
        for (int o = 1; o < L; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float vj = vs[t * cols + c];
#pragma unroll
        for (int i = 0; i < ROWS / 2; ++i) {
          S[2 * i] = __fmaf_rn(kr[2 * i], vj, __fmaf_rn(-ar[2 * i], dot, S[2 * i] * gr[2 * i]));
          S[2 * i + 1] = __fmaf_rn(kr[2 * i + 1], vj, __fmaf_rn(-ar[2 * i + 1], dot, S[2 * i + 1] * gr[2 * i + 1]));
          part[i] = __fmaf_rn(S[2 * i + 1], qr[2 * i + 1], S[2 * i] * qr[2 * i]);
        }
#pragma unroll
        for (int w = ROWS / 4; w >= 1; w >>= 1)
#pragma unroll
          for (int i = 0; i < w; ++i) part[i] += part[i + w];
        shares[(t * cols + c) * (L + 1) + l] = part[0];
        continue;
      }
      if (DECAY == 2) {
#pragma unroll
        for (int i = 0; i < Q; ++i) {
          const float4 g = *reinterpret_cast<const float4*>(gp + i * L * 4);
          S[4 * i] *= g.x; S[4 * i + 1] *= g.y; S[4 * i + 2] *= g.z; S[4 * i + 3] *= g.w;
        }
      } else {
        const float g = DECAY == 1 ? gs[t] : g_const;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) S[r] *= g;
      }
      float u = vs[t * cols + c];
      if (DELTA) {
        // sums of pairs, then a fixed tree: short chains, and the same order of additions for every token
        float part[ROWS / 2];
#pragma unroll
        for (int i = 0; i < ROWS / 2; ++i) part[i] = __fmaf_rn(S[2 * i + 1], kr[2 * i + 1], S[2 * i] * kr[2 * i]);
#pragma unroll
        for (int w = ROWS / 4; w >= 1; w >>= 1)
#pragma unroll
          for (int i = 0; i < w; ++i) part[i] += part[i + w];
        float dot = part[0];
#pragma unroll
        for (int o = 1; o < L; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        u = bs[t] * (u - dot);
      }
      float part[ROWS / 2];
#pragma unroll
      for (int i = 0; i < ROWS / 2; ++i) {
        S[2 * i] = __fmaf_rn(kr[2 * i], u, S[2 * i]);
        S[2 * i + 1] = __fmaf_rn(kr[2 * i + 1], u, S[2 * i + 1]);
        part[i] = __fmaf_rn(S[2 * i + 1], qr[2 * i + 1], S[2 * i] * qr[2 * i]);
      }
#pragma unroll
      for (int w = ROWS / 4; w >= 1; w >>= 1)
#pragma unroll
        for (int i = 0; i < w; ++i) part[i] += part[i + w];
      shares[(t * cols + c) * (L + 1) + l] = part[0];
    }
    __syncthreads();                // the next round's copies overwrite the other buffer, which the round after reads
    for (int e = tid; e < tt * cols; e += kScanThreads) {
      const int t = e / cols, cc = e - t * cols;
      const int jj = blockIdx.x * cols + cc;
      const float* sh = shares + (size_t)e * (L + 1);
      float o_acc = sh[0];
#pragma unroll
      for (int i = 1; i < L; ++i) o_acc += sh[i];          // lane order: the same sum for every token
      if (jj < V) p.out[(size_t)(t_begin + t0 + t) * p.out_stride + (size_t)h * V + jj] = o_acc;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < Q; ++i) {
      const int d = (i * L + l) * 4;
      if (d < Dp) *reinterpret_cast<float4*>(sp + d) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
    }
  }
}

// ---- per-head norm, weight and gate of a mixer's read-out ---------------------------------------------
//   y[n, h, :] = o / sqrt(mean(o^2) + eps) * weight * act(gate[n, h, :]) * out_scale
// GATE: 0 none, 1 silu, 2 sigmoid.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ weight,
                                      const T* __restrict__ gate, int gate_stride, int gate_kind, T* __restrict__ y,
                                      int y_stride, const int32_t* __restrict__ req_of_token, int heads, int vdim,
                                      float eps, float out_scale, int weight_stride) {
  pdl_launch_dependents();
  pdl_wait();
  // a warp per (token, head): the sum of squares in a fixed order whatever the block holds
  const int n = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= heads || req_of_token[n] < 0) return;
  const float* op = o + (size_t)n * o_stride + (size_t)h * vdim;
  float ss = 0.f;
  for (int d = lane; d < vdim; d += 32) ss = __fmaf_rn(op[d], op[d], ss);
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int d = lane; d < vdim; d += 32) {
    float val = op[d] * r;
    if (weight) val *= weight[(size_t)h * weight_stride + d];
    if (gate_kind) {
      const float z = to_f32<T>(gate[(size_t)n * gate_stride + (size_t)h * vdim + d]);
      val *= gate_kind == 1 ? silu_exact(z) : sigmoid_f(z);
    }
    y[(size_t)n * y_stride + (size_t)h * vdim + d] = from_f32<T>(val * out_scale);
  }
}

// ---- what the generalized delta rule reads ------------------------------------------------------------
// From the projections of a token (model dtype): q, k, v as float32; per head and key channel the decay
// g = exp(-rate * sigmoid(w_raw + w_bias)), the unit key u = k / sqrt(sum k^2 + unit_eps) of each head and the
// removal vector sigmoid(a_raw + a_bias) * u.  A block per token, a warp per head in turn; float32 throughout.
template <typename T>
__global__ void general_delta_prepare_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                             int in_stride, const T* __restrict__ a_raw, int a_stride,
                                             const float* __restrict__ a_bias, const T* __restrict__ w_raw, int w_stride,
                                             const float* __restrict__ w_bias, float rate, float unit_eps,
                                             const int32_t* __restrict__ req_of_token, int heads, int dim,
                                             float* __restrict__ out, size_t plane) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  if (req_of_token[n] < 0) return;
  const int lane = threadIdx.x & 31, nw = blockDim.x >> 5, width = heads * dim;
  float* row = out + (size_t)n * width;           // six planes [N, width]: q, k, v, decay, unit, removal
  for (int h = blockIdx.y * nw + (threadIdx.x >> 5); h < heads; h += nw * gridDim.y) {   // a warp per head
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) {
      const float kv = to_f32<T>(k[(size_t)n * in_stride + h * dim + d]);
      ss = __fmaf_rn(kv, kv, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + unit_eps);
    for (int d = lane; d < dim; d += 32) {
      const int c = h * dim + d;
      const float kv = to_f32<T>(k[(size_t)n * in_stride + c]);
      const float u = kv * inv;
      row[c] = to_f32<T>(q[(size_t)n * in_stride + c]);
      row[1 * plane + c] = kv;
      row[2 * plane + c] = to_f32<T>(v[(size_t)n * in_stride + c]);
      row[3 * plane + c] = expf(-rate * sigmoid_f(to_f32<T>(w_raw[(size_t)n * w_stride + c]) + w_bias[c]));
      row[4 * plane + c] = u;
      row[5 * plane + c] = sigmoid_f(to_f32<T>(a_raw[(size_t)n * a_stride + c]) + a_bias[c]) * u;
    }
  }
}

}  // namespace

// out: float32 [6, n_tokens, heads * dim]: q, k, v, decay, unit key, removal vector.
YALIS_API int yalis_general_delta_prepare(const void* q, const void* k, const void* v, int in_stride, const void* a_raw,
                                          int a_stride, const float* a_bias, const void* w_raw, int w_stride,
                                          const float* w_bias, float rate, float unit_eps, const int32_t* req_of_token,
                                          int n_tokens, int heads, int dim, int dtype, float* out,
                                          cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || dim <= 0) return YALIS_ERR_SHAPE;
  // steps of few tokens: two heads a block, so that a decode step of 8 tokens fills more than 8 SMs
  const int per_block = n_tokens >= 512 ? 8 : 2;
  const int warps = heads < per_block ? heads : per_block;
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(general_delta_prepare_kernel<T>, dim3(n_tokens, (heads + warps - 1) / warps), dim3(32 * warps), 0, stream,
                                           (const T*)q, (const T*)k, (const T*)v, in_stride, (const T*)a_raw, a_stride, a_bias,
                                           (const T*)w_raw, w_stride, w_bias, rate, unit_eps, req_of_token, heads, dim, out,
                                           (size_t)n_tokens * heads * dim));
  return YALIS_OK;
}

// a_raw null: no decay and write strength are computed.  kv_heads 0: no head is brought to unit length.
YALIS_API int yalis_delta_prepare(const void* x, int dtype, int x_stride, const float* w, float* tail,
                                  int64_t slot_stride, const int32_t* req_of_token, const int32_t* q_start,
                                  const int32_t* slots, float* out, int out_stride, int n_tokens, int n_requests,
                                  int channels, int taps, int kv_heads, int dim, float q_scale, float unit_eps,
                                  const void* a_raw, int a_stride, int a_cols, const float* a_log, const float* dt_bias,
                                  const void* b_raw, int b_stride, int heads, float* g_out, float* beta_out,
                                  cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (taps < 1 || taps > kMaxTaps || channels <= 0 || kv_heads < 0 || 2 * kv_heads * dim > channels) return YALIS_ERR_SHAPE;
  if (a_raw && (heads <= 0 || a_cols % heads || !a_log || !dt_bias || !b_raw || !g_out || !beta_out)) return YALIS_ERR_SHAPE;
  const int by = (channels + 127) / 128;
  const int threads = channels >= 1024 ? 256 : 128;
  YALIS_DISPATCH_DTYPE(dtype, T, {
    int st = yalis_launch(delta_prepare_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, (const T*)x, x_stride, w,
                          (const float*)tail, (size_t)slot_stride, req_of_token, q_start, slots, out, out_stride, channels,
                          taps, kv_heads, dim, q_scale, unit_eps, (const T*)a_raw, a_stride, a_cols, a_log, dt_bias,
                          (const T*)b_raw, b_stride, heads, g_out, beta_out);
    if (st != YALIS_OK || taps == 1) return st;
    return yalis_launch(short_conv_tail_kernel<T>, dim3(n_requests, by), dim3(128), 0, stream, (const T*)x, x_stride,
                        tail, (size_t)slot_stride, q_start, slots, channels, taps);
  });
  return YALIS_OK;
}

// Rows of a column that a thread keeps: 8 up to dim 256, 16 beyond (up to 512).
static int scan_rows(int dim) { return dim <= 256 ? 8 : 16; }

// Lanes that share a column of the state: the smallest power of two with rows * lanes >= dim.
YALIS_API int yalis_state_scan_lanes(int dim) {
  int lanes = 1;
  while (lanes * scan_rows(dim) < dim) lanes <<= 1;
  return lanes;
}

template <int ROWS, int LANES, int RULE, int DECAY>
static int launch_scan(const ScanParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    if (cudaFuncSetAttribute(state_scan_kernel<ROWS, LANES, RULE, DECAY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess)
      return YALIS_ERR_LAUNCH;
    allowed = 200 * 1024;
  }
  return yalis_launch(state_scan_kernel<ROWS, LANES, RULE, DECAY>, grid, dim3(kScanThreads), smem, stream, p);
}

template <int ROWS, int LANES>
static int launch_scan_kind(const ScanParams& p, dim3 grid, size_t smem, int delta, int decay_kind, cudaStream_t stream) {
  if (delta == 2) return launch_scan<ROWS, LANES, 2, 2>(p, grid, smem, stream);
  if (delta && decay_kind == 1) return launch_scan<ROWS, LANES, 1, 1>(p, grid, smem, stream);
  if (delta && decay_kind == 2) return launch_scan<ROWS, LANES, 1, 2>(p, grid, smem, stream);
  if (delta) return launch_scan<ROWS, LANES, 1, 0>(p, grid, smem, stream);
  if (decay_kind == 0) return launch_scan<ROWS, LANES, 0, 0>(p, grid, smem, stream);
  if (decay_kind == 1) return launch_scan<ROWS, LANES, 0, 1>(p, grid, smem, stream);
  return launch_scan<ROWS, LANES, 0, 2>(p, grid, smem, stream);
}

// decay_kind 0: decay [heads]; 1: decay [N, heads]; 2: decay [N, heads * dim].  delta 1: the delta rule with beta
// [N, heads]; delta 2: the generalized delta rule with unit keys and removal vectors [N, heads * dim] (contiguous,
// kv_heads = heads, decay_kind 2).
// max_q_len: the longest portion of the step if the caller knows it (0: not known); it only bounds the staging tile.
YALIS_API int yalis_state_scan(const float* q, int q_stride, const float* k, int k_stride, const float* v, int v_stride,
                               const float* decay, int decay_kind, const float* beta, const float* unit,
                               const float* removal, float* state, int64_t slot_stride,
                               float* out, int out_stride, const int32_t* q_start, const int32_t* slots, int n_requests,
                               int heads, int kv_heads, int dim, int vdim, int delta, int max_q_len, cudaStream_t stream) {
  if (n_requests <= 0) return YALIS_OK;
  if (dim <= 0 || vdim <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || heads > 65535 || n_requests > 65535)
    return YALIS_ERR_SHAPE;
  const int lanes = yalis_state_scan_lanes(dim);
  if (lanes > 32) return YALIS_ERR_SHAPE;           // dim <= 512
  if (decay_kind < 0 || decay_kind > 2 || !decay || delta < 0 || delta > 2 || (delta == 1 && !beta)) return YALIS_ERR_SHAPE;
  if (delta == 2 && (decay_kind != 2 || !unit || !removal || kv_heads != heads)) return YALIS_ERR_SHAPE;
  const int dim_padded = (dim + 3) & ~3;
  if ((slot_stride & 3) || ((uintptr_t)state & 15)) return YALIS_ERR_ALIGN;
  const int rows = scan_rows(dim);
  const int cols = kScanThreads / lanes, width = rows * lanes;
  const size_t per_token = ((delta == 2 ? 5 : (decay_kind == 2 ? 3 : 2)) * (size_t)width + cols + 2) * sizeof(float);
  int tile = (int)((180 * 1024) / (2 * per_token));
  tile = tile > kMaxTile ? kMaxTile : (tile < 1 ? 1 : tile);
  if (max_q_len > 0 && tile > max_q_len) tile = max_q_len;      // single tokens: small blocks, many of them per SM
  ScanParams p;
  p.q = q; p.q_stride = q_stride; p.k = k; p.k_stride = k_stride; p.v = v; p.v_stride = v_stride;
  p.decay = decay; p.beta = beta; p.unit = unit; p.removal = removal; p.state = state; p.slot_stride = (size_t)slot_stride; p.out = out;
  p.out_stride = out_stride; p.q_start = q_start; p.slots = slots; p.heads = heads; p.kv_heads = kv_heads;
  p.dim = dim; p.dim_padded = dim_padded; p.vdim = vdim; p.lanes = lanes; p.tile = tile;
  p.wide = (dim % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && !((uintptr_t)q & 15) && !((uintptr_t)k & 15) &&
            (decay_kind != 2 || !((uintptr_t)decay & 15)) &&
            (delta != 2 || (!((uintptr_t)unit & 15) && !((uintptr_t)removal & 15)))) ? 1 : 0;
  const dim3 grid((vdim + cols - 1) / cols, heads, n_requests);
  const size_t smem = 2 * ((per_token * tile + 15) & ~(size_t)15) + (size_t)tile * cols * (lanes + 1) * sizeof(float);
  if (rows == 16) return launch_scan_kind<16, 32>(p, grid, smem, delta, decay_kind, stream);
  switch (lanes) {
    case 1: return launch_scan_kind<8, 1>(p, grid, smem, delta, decay_kind, stream);
    case 2: return launch_scan_kind<8, 2>(p, grid, smem, delta, decay_kind, stream);
    case 4: return launch_scan_kind<8, 4>(p, grid, smem, delta, decay_kind, stream);
    case 8: return launch_scan_kind<8, 8>(p, grid, smem, delta, decay_kind, stream);
    case 16: return launch_scan_kind<8, 16>(p, grid, smem, delta, decay_kind, stream);
    default: return launch_scan_kind<8, 32>(p, grid, smem, delta, decay_kind, stream);
  }
}

YALIS_API int yalis_head_norm_gate(const float* o, int o_stride, const float* weight, const void* gate, int gate_stride,
                                   int gate_kind, void* y, int y_stride, int dtype, const int32_t* req_of_token,
                                   int n_tokens, int heads, int vdim, float eps, float out_scale, int weight_per_head,
                                   cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || heads > 65535 || vdim <= 0 || gate_kind < 0 || gate_kind > 2 || (gate_kind && !gate)) return YALIS_ERR_SHAPE;
  const int warps = heads < 4 ? heads : 4;
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(head_norm_gate_kernel<T>, dim3(n_tokens, (heads + warps - 1) / warps),
                                           dim3(32 * warps), 0, stream, o, o_stride, weight, (const T*)gate, gate_stride,
                                           gate_kind, (T*)y, y_stride, req_of_token, heads, vdim, eps, out_scale,
                                           weight_per_head ? vdim : 0));
  return YALIS_OK;
}
