// What lies between a mixer's input projection and its core, for mixers whose heads are
// prepared in more ways than a full rotation: an added bias, a norm over the head with a
// learned scale, a rotation of only the first `rot_dims` sizes, a constant factor, value heads
// of a size of their own.  Queries go to a plain matrix; keys and values go to the pages of a
// cache or to plain matrices (for mixers that keep a state instead of keys).  Also the
// element-wise activations of dense feed-forwards and the row-wise additions of looped layers.
// All arithmetic is float32; sines and cosines come from sincosf of a float32 angle.
#include "common.cuh"

namespace {

constexpr int kMaxHeadDim = 1024;

struct PrepParams {
  const void* src; int src_stride;           // [N, ...]: q heads at q_off, k heads at k_off, v heads at v_off
  int q_off, k_off, v_off;
  const void* q_bias; const void* k_bias; const void* v_bias;     // model dtype, or null
  const float* q_norm; const float* k_norm; float norm_eps;       // scale over dim, or null: no norm
  const float* inv_freq; int rot_dims;                            // [rot_dims / 2], or null: no rotation
  int rot_interleaved;                                            // pair i is (2i, 2i + 1) instead of (i, i + rot_dims / 2)
  float q_scale, k_scale;
  float q_temp_coef; int q_temp_every;                            // every > 0: q *= 1 + coef * ln(floor((pos + 1) / every) + 1)
  void* q_out; int q_out_stride;             // [N, nq * dim]
  void* k_out; int k_out_stride;             // plain destinations (used when k_pool is null)
  void* v_out; int v_out_stride;
  void* k_pool; void* v_pool;                // [pages, nk, page_size, dim] and [pages, nk, page_size, vdim]
  const int32_t* block_table; int table_width, page_size, num_pages;
  const int32_t* positions; const int32_t* req_of_token;
  int nq, nk, dim, vdim;
  int32_t* bad_page;
};

// One warp per (token, head): heads [0, nq) are queries, [nq, nq + nk) keys, [nq + nk, nq + 2 nk) values.
template <typename T, typename TO>
__global__ void qkv_prepare_kernel(const PrepParams p) {
  extern __shared__ float xs_all[];           // a row of `width_max` floats per warp
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x, head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (head >= p.nq + 2 * p.nk) return;
  float* xs = xs_all + (size_t)(threadIdx.x >> 5) * (p.dim > p.vdim ? p.dim : p.vdim);
  const int req = p.req_of_token[n];
  if (req < 0) return;
  const int pos = p.positions[n];
  const bool is_q = head < p.nq, is_v = head >= p.nq + p.nk;
  const int hh = is_q ? head : (is_v ? head - p.nq - p.nk : head - p.nq);
  const int width = is_v ? p.vdim : p.dim;
  const T* src = reinterpret_cast<const T*>(p.src) + (size_t)n * p.src_stride + (is_q ? p.q_off : (is_v ? p.v_off : p.k_off)) +
                 (size_t)hh * width;
  const T* bias = reinterpret_cast<const T*>(is_q ? p.q_bias : (is_v ? p.v_bias : p.k_bias));
  TO* dst;
  if (is_q) {
    dst = reinterpret_cast<TO*>(p.q_out) + (size_t)n * p.q_out_stride + (size_t)hh * width;
  } else if (p.k_pool != nullptr) {
    const int page_idx = pos / p.page_size;
    const int page = page_idx < p.table_width ? p.block_table[(size_t)req * p.table_width + page_idx] : -1;
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0 && p.bad_page) atomicOr(p.bad_page, YALIS_FLAG_BAD_PAGE);
      return;
    }
    dst = reinterpret_cast<TO*>(is_v ? p.v_pool : p.k_pool) +
          (((size_t)page * p.nk + hh) * p.page_size + (pos - page_idx * p.page_size)) * width;
  } else {
    if (p.k_out == nullptr) return;              // nothing keeps this layer's keys and values: queries only
    dst = is_v ? reinterpret_cast<TO*>(p.v_out) + (size_t)n * p.v_out_stride + (size_t)hh * width
               : reinterpret_cast<TO*>(p.k_out) + (size_t)n * p.k_out_stride + (size_t)hh * width;
  }
  float ss = 0.f;
  for (int d = lane; d < width; d += 32) {
    float x = to_f32<T>(src[d]);
    if (bias) x += to_f32<T>(bias[(size_t)hh * width + d]);
    xs[d] = x;
    ss = __fmaf_rn(x, x, ss);
  }
  if (is_v) {
    for (int d = lane; d < width; d += 32) dst[d] = from_f32<TO>(xs[d]);
    return;
  }
  const float* nw = is_q ? p.q_norm : p.k_norm;
  if (nw) {
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)width + p.norm_eps);
    for (int d = lane; d < width; d += 32) xs[d] = xs[d] * r * nw[d];
  }
  __syncwarp();
  float factor = is_q ? p.q_scale : p.k_scale;
  if (is_q && p.q_temp_every > 0) factor *= 1.0f + p.q_temp_coef * logf((float)((pos + 1) / p.q_temp_every + 1));
  const int half = p.inv_freq ? p.rot_dims >> 1 : 0;
  for (int i = lane; i < half; i += 32) {
    float sn, cs, o1, o2;
    sincosf((float)pos * p.inv_freq[i], &sn, &cs);
    const int a = p.rot_interleaved ? 2 * i : i, b = p.rot_interleaved ? 2 * i + 1 : i + half;
    rotate_pair(xs[a], xs[b], cs, sn, o1, o2);
    dst[a] = from_f32<TO>(o1 * factor);
    dst[b] = from_f32<TO>(o2 * factor);
  }
  for (int d = 2 * half + lane; d < width; d += 32) dst[d] = from_f32<TO>(xs[d] * factor);
}

// ACT: 0 gelu with erf, 1 gelu with tanh, 2 silu, 3 the square of relu, 4 tanh.
template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, int x_stride, T* __restrict__ y, int y_stride, int rows,
                                  int cols, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)rows * cols;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / cols, c = e - r * cols;
    const float z = to_f32<T>(x[r * x_stride + c]);
    float o;
    if (act == 0) o = 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    else if (act == 1) o = 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    else if (act == 2) o = silu_exact(z);
    else if (act == 4) o = tanhf(z);
    else o = fmaxf(z, 0.f) * fmaxf(z, 0.f);
    y[r * y_stride + c] = from_f32<T>(o);
  }
}

// The same, eight elements a thread, for bfloat16 rows that start on 16-byte boundaries and whose width is a
// multiple of 8.  grid: (ceil(cols / 8 / 256), rows).
__device__ __forceinline__ float act_value(float z, int act) {
  if (act == 0) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (act == 1) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  if (act == 3) return fmaxf(z, 0.f) * fmaxf(z, 0.f);
  if (act == 4) return tanhf(z);
  return silu_exact(z);
}

__global__ void activation_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, int x_stride, __nv_bfloat16* __restrict__ y,
                                         int y_stride, int cols, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= cols) return;
  const size_t r = blockIdx.y;
  uint4 raw = *reinterpret_cast<const uint4*>(x + r * x_stride + c);
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 z = __bfloat1622float2(h[i]);
    h[i] = __floats2bfloat162_rn(act_value(z.x, act), act_value(z.y, act));
  }
  *reinterpret_cast<uint4*>(y + r * y_stride + c) = raw;
}

// A gated activation over rows that hold a gate part and an up part (at column offsets of one matrix):
//   kind 0:  y = silu(g) * u
//   kind 1:  g <- min(g, limit), u <- clamp(u, -limit, limit);  y = g * sigmoid(alpha * g) * (u + shift)
// float32 arithmetic, one rounding.
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ x, long x_stride, int gate_off, int up_off, T* __restrict__ y,
                                        long y_stride, int rows, int cols, int kind, float limit, float alpha, float shift) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)rows * cols;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / cols, c = e - r * cols;
    float g = to_f32<T>(x[r * x_stride + gate_off + c]), u = to_f32<T>(x[r * x_stride + up_off + c]);
    float o;
    if (kind == 1) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      o = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + shift);
    } else {
      o = silu_exact(g) * u;
    }
    y[r * y_stride + c] = from_f32<T>(o);
  }
}

// The same, eight elements a thread, for bfloat16 rows whose two parts and whose results start on 16-byte boundaries
// (width and both offsets multiples of 8).  The result is rounded to 8 bits of mantissa at once, so the fast
// exponential and division do not show.  grid: (ceil(cols / 8 / 128), rows).
__global__ void gated_activation_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, long x_stride, int gate_off, int up_off,
                                               __nv_bfloat16* __restrict__ y, long y_stride, int cols, int kind, float limit,
                                               float alpha, float shift) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= cols) return;
  const size_t r = blockIdx.y;
  uint4 graw = *reinterpret_cast<const uint4*>(x + r * x_stride + gate_off + c);
  const uint4 uraw = *reinterpret_cast<const uint4*>(x + r * x_stride + up_off + c);
  __nv_bfloat162* gh = reinterpret_cast<__nv_bfloat162*>(&graw);
  const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uraw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 g = __bfloat1622float2(gh[i]);
    float2 u = __bfloat1622float2(uh[i]);
    if (kind == 1) {
      g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
      u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
      gh[i] = __floats2bfloat162_rn(__fdividef(g.x, 1.0f + __expf(-alpha * g.x)) * (u.x + shift),
                                    __fdividef(g.y, 1.0f + __expf(-alpha * g.y)) * (u.y + shift));
    } else {
      gh[i] = __floats2bfloat162_rn(silu_bf16_path(g.x) * u.x, silu_bf16_path(g.y) * u.y);
    }
  }
  *reinterpret_cast<uint4*>(y + r * y_stride + c) = graw;
}

// x[n, :] += other[n, :] + vec[:]   (either may be absent)
__global__ void add_rows_vector_kernel(float* __restrict__ x, const float* __restrict__ other,
                                       const float* __restrict__ vec, int rows, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)rows * cols;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    float v = x[e];
    if (other) v += other[e];
    if (vec) v += vec[e % cols];
    x[e] = v;
  }
}

}  // namespace

// out_dtype: the dtype of q_out and of the plain k_out / v_out (pools always have the model dtype `dtype`).
YALIS_API int yalis_qkv_prepare(const void* src, int dtype, int src_stride, int q_off, int k_off, int v_off,
                                const void* q_bias, const void* k_bias, const void* v_bias, const float* q_norm,
                                const float* k_norm, float norm_eps, const float* inv_freq, int rot_dims,
                                int rot_interleaved, float q_scale, float k_scale, float q_temp_coef, int q_temp_every,
                                void* q_out, int q_out_stride, void* k_out, int k_out_stride, void* v_out,
                                int v_out_stride, int out_dtype, void* k_pool, void* v_pool,
                                const int32_t* block_table, int table_width, int page_size, int num_pages,
                                const int32_t* positions, const int32_t* req_of_token, int n_tokens, int nq, int nk,
                                int dim, int vdim, int32_t* bad_page, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (dim <= 0 || dim > kMaxHeadDim || vdim <= 0 || vdim > kMaxHeadDim || nq <= 0 || nk <= 0 || nq + 2 * nk > 65535)
    return YALIS_ERR_SHAPE;
  if (inv_freq && (rot_dims <= 0 || (rot_dims & 1) || rot_dims > dim)) return YALIS_ERR_SHAPE;
  if (k_pool && out_dtype != dtype) return YALIS_ERR_DTYPE;
  PrepParams p;
  p.src = src; p.src_stride = src_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
  p.q_bias = q_bias; p.k_bias = k_bias; p.v_bias = v_bias; p.q_norm = q_norm; p.k_norm = k_norm; p.norm_eps = norm_eps;
  p.inv_freq = inv_freq; p.rot_dims = rot_dims; p.rot_interleaved = rot_interleaved; p.q_scale = q_scale; p.k_scale = k_scale;
  p.q_temp_coef = q_temp_coef; p.q_temp_every = q_temp_every;
  p.q_out = q_out; p.q_out_stride = q_out_stride; p.k_out = k_out; p.k_out_stride = k_out_stride;
  p.v_out = v_out; p.v_out_stride = v_out_stride; p.k_pool = k_pool; p.v_pool = v_pool; p.block_table = block_table;
  p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages; p.positions = positions;
  p.req_of_token = req_of_token; p.nq = nq; p.nk = nk; p.dim = dim; p.vdim = vdim; p.bad_page = bad_page;
  const int warps = 4;
  const dim3 grid(n_tokens, (nq + 2 * nk + warps - 1) / warps);
  const size_t smem = (size_t)warps * (dim > vdim ? dim : vdim) * sizeof(float);
  if (dtype == YALIS_F32 && out_dtype == YALIS_F32)
    return yalis_launch(qkv_prepare_kernel<float, float>, grid, dim3(32 * warps), smem, stream, p);
  if (dtype == YALIS_BF16 && out_dtype == YALIS_BF16)
    return yalis_launch(qkv_prepare_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(32 * warps), smem, stream, p);
  if (dtype == YALIS_BF16 && out_dtype == YALIS_F32)
    return yalis_launch(qkv_prepare_kernel<__nv_bfloat16, float>, grid, dim3(32 * warps), smem, stream, p);
  return YALIS_ERR_DTYPE;
}

YALIS_API int yalis_activation(const void* x, int x_stride, void* y, int y_stride, int dtype, int rows, int cols,
                               int act, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return YALIS_OK;
  if (act < 0 || act > 4) return YALIS_ERR_SHAPE;
  const size_t total = (size_t)rows * cols;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == YALIS_BF16 && cols % 8 == 0 && x_stride % 8 == 0 && y_stride % 8 == 0 && !((uintptr_t)x & 15) &&
      !((uintptr_t)y & 15) && rows <= 65535)
    return yalis_launch(activation_bf16x8_kernel, dim3((cols / 8 + 127) / 128, rows), dim3(128), 0, stream,
                        (const __nv_bfloat16*)x, x_stride, (__nv_bfloat16*)y, y_stride, cols, act);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(activation_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)x, x_stride,
                                           (T*)y, y_stride, rows, cols, act));
  return YALIS_OK;
}

YALIS_API int yalis_gated_activation(const void* x, long long x_stride, int gate_off, int up_off, void* y, long long y_stride,
                                     int dtype, int rows, int cols, int kind, float limit, float alpha, float shift,
                                     cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return YALIS_OK;
  if (kind < 0 || kind > 1) return YALIS_ERR_SHAPE;
  if (dtype == YALIS_BF16 && cols % 8 == 0 && x_stride % 8 == 0 && y_stride % 8 == 0 && gate_off % 8 == 0 && up_off % 8 == 0 &&
      !((uintptr_t)x & 15) && !((uintptr_t)y & 15) && rows <= 65535)
    return yalis_launch(gated_activation_bf16x8_kernel, dim3((cols / 8 + 127) / 128, rows), dim3(128), 0, stream,
                        (const __nv_bfloat16*)x, (long)x_stride, gate_off, up_off, (__nv_bfloat16*)y, (long)y_stride, cols, kind,
                        limit, alpha, shift);
  const size_t total = (size_t)rows * cols;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(gated_activation_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)x,
                                           (long)x_stride, gate_off, up_off, (T*)y, (long)y_stride, rows, cols, kind, limit,
                                           alpha, shift));
  return YALIS_OK;
}

YALIS_API int yalis_add_rows_vector(float* x, const float* other, const float* vec, int rows, int cols,
                                    cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return YALIS_OK;
  const size_t total = (size_t)rows * cols;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return yalis_launch(add_rows_vector_kernel, dim3(blocks), dim3(256), 0, stream, x, other, vec, rows, cols);
}
