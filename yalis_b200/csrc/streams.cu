// A residual stream kept in several copies ("hyper-connections"), a norm without statistics, and an embedding row
// chosen by a pair of tokens.
//
// `stream_step` is the one kernel between two sub-layers.  Per token row and column c, with S copies x_1 .. x_S:
//
//   write (optional)   y  = (sum of the given partial results) * layer_scale[c] * sigmoid(gate[c] + gate_bias[c])
//                      x_t <- sum_s mix[s][t] x_s + out[t] * y          (all copies from the old ones)
//   read  (optional)   u  = sum_s in[s] x_s                             (in absent: the plain sum)
//                      h  = tanh(alpha * u) * w[c] + b[c]               (norm absent: h = u)
//
// Nothing here needs a sum over a row, so a thread owns a few columns of one row and the copies stay in registers
// between the write of one sub-layer and the read of the next.  With S = 1, mix = out = in = 1 this is the plain
// "x += y; h = norm(x)" of a pre-norm layer, so the same kernel serves a model with one copy.  All arithmetic is
// float32; y, gate and h are in the model's dtype (the partial results of a split product are float32).
//
// `pair_rows_add` adds row ((previous * mul_prev + token * mul_cur) mod buckets) of a table to every token's row
// of the stream (row `buckets` for the first token of a sequence); the previous token of a portion's first token
// is kept per request slot by `remember_last_tokens`.
#include "common.cuh"

namespace {

constexpr int kMaxCopies = 8;

struct StreamStep {
  float* x; int copies; int width;              // [N, copies, width] float32, updated in place when `store`
  const float* src;                             // [N, width] or null: every copy equals this row (x holds nothing yet)
  const void* y; int y_parts; long y_part_stride; long y_stride; int y_f32;   // [parts][N, width]
  const void* gate; long gate_stride; const float* gate_bias; int gate_f32;  // logits of the gate on y, or null
  const float* layer_scale;                     // [width] or null
  const float* mix; const float* out_w;         // [copies, copies] (from, to) and [copies]; both null: x_t += y
  const float* in_w;                            // [copies] or null (the plain sum)
  const float* alpha; const float* norm_w; const float* norm_b;              // norm: all three or none
  const int32_t* rows; int n_rows;              // rows null: every row, the result of the write is stored
  void* h; long h_stride; int h_f32;            // [n_rows, width] or null
  int store;
  int vec;                                      // V == 4 only: y, gate, h and the per-column vectors take 8- and 16-byte accesses
};

// Four consecutive values of a float32 or bfloat16 array as one access (``vec``: 16- resp. 8-byte aligned), else one by one.
template <int V>
__device__ __forceinline__ void load_values(const void* base, bool f32, size_t at, bool vec, float (&out)[V]) {
  if (V == 4 && vec) {
    if (f32) {
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + at);
      out[0] = v.x; out[1] = v.y; out[V > 1 ? 2 : 0] = v.z; out[V > 1 ? 3 : 0] = v.w;
    } else {
      const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + at);
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
      out[0] = lo.x; out[1] = lo.y; out[V > 1 ? 2 : 0] = hi.x; out[V > 1 ? 3 : 0] = hi.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j)
      out[j] = f32 ? reinterpret_cast<const float*>(base)[at + j] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[at + j]);
  }
}

// SC: the number of copies when the launcher knows a kernel for it (1 to 4), else 0: read from the arguments.
template <int V, int SC>
__global__ void __launch_bounds__(256) stream_step_kernel(const StreamStep a) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int n = a.rows ? a.rows[r] : r;
  if (n < 0) return;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (c0 >= a.width) return;
  const int S = SC ? SC : a.copies, D = a.width;
  float* xr = a.x + (size_t)n * S * D + c0;
  float xs[kMaxCopies][V];
  if (a.src != nullptr) {                         // the stream's first pass: all copies are the entering row
    float e[V];
    load_values<V>(a.src, true, (size_t)n * D + c0, V == 4, e);
#pragma unroll
    for (int s = 0; s < kMaxCopies; ++s)
      if (s < S)
#pragma unroll
        for (int j = 0; j < V; ++j) xs[s][j] = e[j];
  } else {
#pragma unroll
  for (int s = 0; s < kMaxCopies; ++s) {
    if (s < S) {
      if (V == 4) {
        const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)s * D);
        xs[s][0] = v.x; xs[s][1] = v.y; xs[s][V > 1 ? 2 : 0] = v.z; xs[s][V > 1 ? 3 : 0] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) xs[s][j] = xr[(size_t)s * D + j];
      }
    }
  }
  }
  if (a.y != nullptr) {
    float y[V];
    if (a.y_f32) {
#pragma unroll
      for (int j = 0; j < V; ++j) y[j] = 0.f;
      for (int q = 0; q < a.y_parts; ++q) {
        float part[V];
        load_values<V>(a.y, true, (size_t)q * a.y_part_stride + (size_t)n * a.y_stride + c0, a.vec, part);
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] += part[j];
      }
    } else {
      load_values<V>(a.y, false, (size_t)n * a.y_stride + c0, a.vec, y);
    }
    if (a.layer_scale) {
      float sc[V];
      load_values<V>(a.layer_scale, true, c0, a.vec, sc);
#pragma unroll
      for (int j = 0; j < V; ++j) y[j] *= sc[j];
    }
    if (a.gate) {
      float g[V];
      load_values<V>(a.gate, a.gate_f32, (size_t)n * a.gate_stride + c0, a.vec, g);
      if (a.gate_bias) {
        float gb[V];
        load_values<V>(a.gate_bias, true, c0, a.vec, gb);
#pragma unroll
        for (int j = 0; j < V; ++j) g[j] += gb[j];
      }
#pragma unroll
      for (int j = 0; j < V; ++j) y[j] *= 1.0f / (1.0f + expf(-g[j]));
    }
    if (a.mix == nullptr) {
#pragma unroll
      for (int s = 0; s < kMaxCopies; ++s)
        if (s < S)
#pragma unroll
          for (int j = 0; j < V; ++j) xs[s][j] += y[j];
    } else {
      float nx[kMaxCopies][V];
#pragma unroll
      for (int t = 0; t < kMaxCopies; ++t) {
        if (t < S) {
#pragma unroll
          for (int j = 0; j < V; ++j) nx[t][j] = 0.f;
#pragma unroll
          for (int s = 0; s < kMaxCopies; ++s)
            if (s < S) {
              const float m = a.mix[s * S + t];
#pragma unroll
              for (int j = 0; j < V; ++j) nx[t][j] = __fmaf_rn(m, xs[s][j], nx[t][j]);
            }
          const float o = a.out_w[t];
#pragma unroll
          for (int j = 0; j < V; ++j) nx[t][j] = __fmaf_rn(o, y[j], nx[t][j]);
        }
      }
#pragma unroll
      for (int t = 0; t < kMaxCopies; ++t)
        if (t < S)
#pragma unroll
          for (int j = 0; j < V; ++j) xs[t][j] = nx[t][j];
    }
  }
  if (a.store && (a.y != nullptr || a.src != nullptr)) {
#pragma unroll
    for (int s = 0; s < kMaxCopies; ++s)
      if (s < S) {
        if (V == 4) {
          *reinterpret_cast<float4*>(xr + (size_t)s * D) = make_float4(xs[s][0], xs[s][1], xs[s][V > 1 ? 2 : 0], xs[s][V > 1 ? 3 : 0]);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) xr[(size_t)s * D + j] = xs[s][j];
        }
      }
  }
  if (a.h == nullptr) return;
  float u[V];
#pragma unroll
  for (int j = 0; j < V; ++j) u[j] = 0.f;
#pragma unroll
  for (int s = 0; s < kMaxCopies; ++s)
    if (s < S) {
      const float w = a.in_w ? a.in_w[s] : 1.0f;
#pragma unroll
      for (int j = 0; j < V; ++j) u[j] = a.in_w ? __fmaf_rn(w, xs[s][j], u[j]) : u[j] + xs[s][j];
    }
  if (a.alpha != nullptr) {
    const float al = a.alpha[0];
    float nw[V], nb[V];
    load_values<V>(a.norm_w, true, c0, a.vec, nw);
    load_values<V>(a.norm_b, true, c0, a.vec, nb);
#pragma unroll
    for (int j = 0; j < V; ++j) u[j] = __fmaf_rn(tanhf(al * u[j]), nw[j], nb[j]);
  }
  if (V == 4 && a.vec) {
    if (a.h_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.h) + (size_t)r * a.h_stride + c0) =
          make_float4(u[0], u[1], u[V > 1 ? 2 : 0], u[V > 1 ? 3 : 0]);
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(u[0], u[1]), hi = __floats2bfloat162_rn(u[V > 1 ? 2 : 0], u[V > 1 ? 3 : 0]);
      uint2 v;
      v.x = *reinterpret_cast<const uint32_t*>(&lo);
      v.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.h) + (size_t)r * a.h_stride + c0) = v;
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < V; ++j) {
    if (a.h_f32) reinterpret_cast<float*>(a.h)[(size_t)r * a.h_stride + c0 + j] = u[j];
    else reinterpret_cast<__nv_bfloat16*>(a.h)[(size_t)r * a.h_stride + c0 + j] = __float2bfloat16_rn(u[j]);
  }
}

// x[n, :] += table[row(n), :] for every token of a request (float32 stream of one copy).
template <typename T>
__global__ void pair_rows_add_kernel(float* __restrict__ x, int width, const T* __restrict__ table, int buckets,
                                     long long mul_prev, long long mul_cur, const int32_t* __restrict__ ids,
                                     const int32_t* __restrict__ from_slot, const int32_t* __restrict__ chosen,
                                     const int32_t* __restrict__ positions, const int32_t* __restrict__ req_of_token,
                                     const int32_t* __restrict__ q_start, const int32_t* __restrict__ slots,
                                     const int32_t* __restrict__ last_token, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int req = req_of_token[n];
  if (req < 0) return;
  auto token_at = [&](int t) {
    int id = ids[t];
    if (from_slot != nullptr && from_slot[t] >= 0) id = chosen[from_slot[t]];
    return id;
  };
  const int tok = token_at(n);
  if (tok < 0 || tok >= vocab) return;          // the embedding kernel has reported it
  long long row = buckets;                       // the first token of a sequence
  if (positions[n] > 0) {
    const int prev = n > q_start[req] ? token_at(n - 1) : last_token[slots[req]];
    row = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    if (row < 0) row += buckets;
  }
  const T* src = table + (size_t)row * width;
  float* dst = x + (size_t)n * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] += to_f32<T>(src[c]);
}

// last_token[slot of request] = the last token the request brought in this step.
__global__ void remember_last_tokens_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ from_slot,
                                            const int32_t* __restrict__ chosen, const int32_t* __restrict__ q_start,
                                            const int32_t* __restrict__ slots, int n_requests, int32_t* __restrict__ last_token) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_requests) return;
  const int a = q_start[r], b = q_start[r + 1];
  if (b <= a) return;
  int id = ids[b - 1];
  if (from_slot != nullptr && from_slot[b - 1] >= 0) id = chosen[from_slot[b - 1]];
  last_token[slots[r]] = id;
}

}  // namespace

YALIS_API int yalis_stream_step(float* x, int n_tokens, int copies, int width, const void* y, int y_parts, long y_part_stride,
                                long y_stride, int y_f32, const void* gate, long gate_stride, const float* gate_bias,
                                int gate_f32, const float* layer_scale, const float* mix, const float* out_w,
                                const float* in_w, const float* alpha, const float* norm_w, const float* norm_b,
                                const int32_t* rows, int n_rows, void* h, long h_stride, int h_f32, const float* src,
                                cudaStream_t stream) {
  if (copies < 1 || copies > kMaxCopies || width <= 0) return YALIS_ERR_SHAPE;
  if ((mix == nullptr) != (out_w == nullptr)) return YALIS_ERR_SHAPE;
  if ((alpha == nullptr) != (norm_w == nullptr) || (alpha == nullptr) != (norm_b == nullptr)) return YALIS_ERR_SHAPE;
  if (y != nullptr && !y_f32 && y_parts != 1) return YALIS_ERR_SHAPE;
  const int count = rows ? n_rows : n_tokens;
  if (count <= 0) return YALIS_OK;
  StreamStep a;
  a.x = x; a.src = src; a.copies = copies; a.width = width; a.y = y; a.y_parts = y_parts; a.y_part_stride = y_part_stride;
  a.y_stride = y_stride; a.y_f32 = y_f32; a.gate = gate; a.gate_stride = gate_stride; a.gate_bias = gate_bias;
  a.gate_f32 = gate_f32; a.layer_scale = layer_scale; a.mix = mix; a.out_w = out_w; a.in_w = in_w; a.alpha = alpha;
  a.norm_w = norm_w; a.norm_b = norm_b; a.rows = rows; a.n_rows = n_rows; a.h = h; a.h_stride = h_stride; a.h_f32 = h_f32;
  a.store = rows == nullptr ? 1 : 0;
  const bool wide = width % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)src & 15);
  // 8- and 16-byte accesses to everything beside x: every base and row stride must allow them
  auto fits = [](const void* p, bool f32, long stride) {
    return p == nullptr || (!((uintptr_t)p & (f32 ? 15 : 7)) && stride % 4 == 0);
  };
  a.vec = wide && fits(y, y_f32, y_stride) && (y == nullptr || y_part_stride % 4 == 0) && fits(gate, gate_f32, gate_stride) &&
          fits(gate_bias, true, 0) && fits(layer_scale, true, 0) && fits(norm_w, true, 0) && fits(norm_b, true, 0) &&
          fits(h, h_f32, h_stride);
  const int per = wide ? 4 : 1;
  const int threads = 256;
  const dim3 grid((width + threads * per - 1) / (threads * per), count);
  if (!wide) return yalis_launch(stream_step_kernel<1, 0>, grid, dim3(threads), 0, stream, a);
  switch (copies) {
    case 1: return yalis_launch(stream_step_kernel<4, 1>, grid, dim3(threads), 0, stream, a);
    case 2: return yalis_launch(stream_step_kernel<4, 2>, grid, dim3(threads), 0, stream, a);
    case 3: return yalis_launch(stream_step_kernel<4, 3>, grid, dim3(threads), 0, stream, a);
    case 4: return yalis_launch(stream_step_kernel<4, 4>, grid, dim3(threads), 0, stream, a);
    default: return yalis_launch(stream_step_kernel<4, 0>, grid, dim3(threads), 0, stream, a);
  }
}

YALIS_API int yalis_pair_rows_add(float* x, int n_tokens, int width, const void* table, int dtype, int buckets,
                                  long long mul_prev, long long mul_cur, const int32_t* ids, const int32_t* from_slot,
                                  const int32_t* chosen, const int32_t* positions, const int32_t* req_of_token,
                                  const int32_t* q_start, const int32_t* slots, const int32_t* last_token, int vocab,
                                  cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (buckets <= 0 || (from_slot == nullptr) != (chosen == nullptr)) return YALIS_ERR_SHAPE;
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(pair_rows_add_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, x, width,
                                           (const T*)table, buckets, mul_prev, mul_cur, ids, from_slot, chosen, positions,
                                           req_of_token, q_start, slots, last_token, vocab));
  return YALIS_OK;
}

YALIS_API int yalis_remember_last_tokens(const int32_t* ids, const int32_t* from_slot, const int32_t* chosen,
                                         const int32_t* q_start, const int32_t* slots, int n_requests, int32_t* last_token,
                                         cudaStream_t stream) {
  if (n_requests <= 0) return YALIS_OK;
  return yalis_launch(remember_last_tokens_kernel, dim3((n_requests + 127) / 128), dim3(128), 0, stream, ids, from_slot,
                      chosen, q_start, slots, n_requests, last_token);
}
