// Attention over a latent: every token keeps ONE row [c (r) | k_rot (p)] for all heads, where c is a normed
// low-rank projection of the layer's input and k_rot a rotated key part that all heads share.  A head's keys
// and values are linear maps of c (k_h = Uk_h c, v_h = Uv_h c), so they are never formed: with
// a_h = Uk_h^T q_h ("absorbed" queries, r wide)
//
//     score_h(i, j) = (a_h(i) . c(j) + q_rot_h(i) . k_rot(j)) * scale
//     out_h(i)      = Uv_h  sum_j softmax_j(score_h(i, j)) c(j)
//
// which is attention with one key/value head of width r + p whose values are the first r sizes of the keys.
// The pieces here: `latent_prepare` (norm of c, rotation of k_rot and of the queries' rotated parts, page
// write), `head_project` (the per-head maps Uk^T and Uv on the CUDA cores, float32 in k order, with an optional
// sigmoid gate on the result; large bfloat16 steps use the library's batched product and `sigmoid_gate` instead),
// and the attention itself in two forms: an exact one (float32 path, twin of the other) and a tensor-core one
// (bfloat16 pages).  Scores, weights and sums are float32 in every form.
#include "common.cuh"


namespace {

// ---- prepare -----------------------------------------------------------------------------------------------
struct LatentPrep {
  const void* src; int src_stride;    // [N, ...] model dtype: heads [plain d | rotated p] at q_off, [c r | k_rot p] at kv_off
  int q_off, kv_off;                  // kv_off < 0: this layer reads another layer's rows and writes none
  const void* q_src; int q_stride;    // the queries, when they are not columns of src (queries through a latent of their own)
  int heads, d, r, p;
  const float* norm_w; float eps;     // scale of the norm over c
  const float* inv_freq; int rot_dims; int interleaved; float magnitude;   // inv_freq null: no rotation
  float* qc;                          // [N, heads, r + p] float32: this kernel fills the last p of every head
  void* pool;                         // [pages, 1, page_size, r + p] model dtype, or null
  const int32_t* block_table; int table_width, page_size, num_pages;
  const int32_t* positions; const int32_t* req_of_token;
  int32_t* bad_page;
};

// The first rot_dims of src[0..p) turned by position * inv_freq (pairs (2i, 2i+1) or (i, i + rot_dims / 2)),
// the rest copied.  One warp.
template <typename T, typename TO>
__device__ __forceinline__ void rotate_part(const T* __restrict__ src, TO* __restrict__ dst, int p, int pos,
                                            const LatentPrep& a, int lane) {
  const int half = a.inv_freq ? a.rot_dims >> 1 : 0;
  for (int i = lane; i < half; i += 32) {
    float sn, cs, o1, o2;
    sincosf((float)pos * a.inv_freq[i], &sn, &cs);
    sn *= a.magnitude;
    cs *= a.magnitude;
    const int i1 = a.interleaved ? 2 * i : i, i2 = a.interleaved ? 2 * i + 1 : i + half;
    rotate_pair(to_f32<T>(src[i1]), to_f32<T>(src[i2]), cs, sn, o1, o2);
    dst[i1] = from_f32<TO>(o1);
    dst[i2] = from_f32<TO>(o2);
  }
  for (int i = 2 * half + lane; i < p; i += 32) dst[i] = from_f32<TO>(to_f32<T>(src[i]));
}

// One warp per job of a token: jobs [0, heads) rotate a head's query part, job `heads` makes the token's row.
template <typename T>
__global__ void latent_prepare_kernel(const LatentPrep a) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x, job = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (job > a.heads) return;
  const int req = a.req_of_token[n];
  if (req < 0) return;
  const int pos = a.positions[n];
  const T* row = reinterpret_cast<const T*>(a.src) + (size_t)n * a.src_stride;
  if (job < a.heads) {
    const T* qrow = a.q_src ? reinterpret_cast<const T*>(a.q_src) + (size_t)n * a.q_stride : row;
    rotate_part<T, float>(qrow + a.q_off + (size_t)job * (a.d + a.p) + a.d,
                          a.qc + ((size_t)n * a.heads + job) * (a.r + a.p) + a.r, a.p, pos, a, lane);
    return;
  }
  if (a.kv_off < 0 || a.pool == nullptr) return;
  const int page_idx = pos / a.page_size;
  const int page = page_idx < a.table_width ? a.block_table[(size_t)req * a.table_width + page_idx] : -1;
  if (page < 0 || page >= a.num_pages) {
    if (lane == 0 && a.bad_page) atomicOr(a.bad_page, YALIS_FLAG_BAD_PAGE);
    return;
  }
  T* dst = reinterpret_cast<T*>(a.pool) + ((size_t)page * a.page_size + (pos - page_idx * a.page_size)) * (a.r + a.p);
  const T* s = row + a.kv_off;
  float ss = 0.f;
  for (int i = lane; i < a.r; i += 32) {
    const float x = to_f32<T>(s[i]);
    ss = __fmaf_rn(x, x, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)a.r + a.eps);
  for (int i = lane; i < a.r; i += 32) dst[i] = from_f32<T>(to_f32<T>(s[i]) * inv * a.norm_w[i]);
  rotate_part<T, T>(s + a.r, dst + a.r, a.p, pos, a, lane);
}

// y[n, :] = x[n, :] / sqrt(mean(x[n, :]^2) + eps) * w for a column block x [N, width] of a wider matrix (the normed
// latent that queries pass through).  A warp per row; float32 arithmetic, one rounding.
template <typename T>
__global__ void norm_rows_kernel(const T* __restrict__ x, long x_stride, const float* __restrict__ w, float eps, int width,
                                 T* __restrict__ y, long y_stride, int n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= n_rows) return;
  const T* s = x + (size_t)n * x_stride;
  float ss = 0.f;
  for (int i = lane; i < width; i += 32) {
    const float v = to_f32<T>(s[i]);
    ss = __fmaf_rn(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = lane; i < width; i += 32) y[(size_t)n * y_stride + i] = from_f32<T>(to_f32<T>(s[i]) * inv * w[i]);
}

// ---- per-head linear maps -------------------------------------------------------------------------------------
// out[n, h, o] = sum_k w[h, o, k] x[n, h, k]   (optionally times sigmoid(gate[n, h * O + o])), float32 sums in k
// order per lane and a fixed butterfly across lanes.  Block (n, h); a warp per output.
template <typename T, typename TX, typename TO>
__global__ void head_project_kernel(const TX* __restrict__ x, long xs_n, long xs_h, const T* __restrict__ w, int O, int K,
                                    TO* __restrict__ out, long os_n, long os_h, const T* __restrict__ gate, long gs_n,
                                    const int32_t* __restrict__ req_of_token) {
  extern __shared__ float xs[];
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x, h = blockIdx.y;
  if (req_of_token && req_of_token[n] < 0) return;
  const TX* xp = x + (size_t)n * xs_n + (size_t)h * xs_h;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f32<TX>(xp[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const T* wh = w + (size_t)h * O * K;
  // four outputs in flight per warp: their loads and butterflies overlap; each output's own order of sums is fixed
  for (int o0 = warp * 4; o0 < O; o0 += warps * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = lane; k < K; k += 32) {
      const float xv = xs[k];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (o0 + j < O) acc[j] = __fmaf_rn(to_f32<T>(wh[(size_t)(o0 + j) * K + k]), xv, acc[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = warp_sum(acc[j]);
    if (lane < 4 && o0 + lane < O) {
      const int o = o0 + lane;
      float v = lane == 0 ? acc[0] : (lane == 1 ? acc[1] : (lane == 2 ? acc[2] : acc[3]));
      if (gate) v *= 1.0f / (1.0f + expf(-to_f32<T>(gate[(size_t)n * gs_n + (size_t)h * O + o])));
      out[(size_t)n * os_n + (size_t)h * os_h + o] = from_f32<TO>(v);
    }
  }
}

// y[n, h * e + c] = x[n, h, c] * sigmoid(g[n, h * e + c])  (x float32 or model dtype with strides over n and h,
// y and g model dtype)
template <typename T, typename TX>
__global__ void sigmoid_gate_kernel(const TX* __restrict__ x, long xs_n, long xs_h, int e, const T* __restrict__ g, long gs,
                                    T* __restrict__ y, long ys, int rows, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)rows * cols;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols, c = i - r * cols, h = c / e;
    const float v = to_f32<TX>(x[r * xs_n + h * xs_h + (c - h * e)]) / (1.0f + expf(-to_f32<T>(g[r * gs + c])));
    y[r * ys + c] = from_f32<T>(v);
  }
}

// ---- the exact attention -----------------------------------------------------------------------------------------
constexpr int kWarps = 4;
constexpr int kMaxPerLane = 20;   // r + p <= 640

// Block (token, head).  Each warp walks every fourth visible row in ascending order with an online softmax; the
// four partial results are merged in warp order, so a (position, head) has one order of sums whatever the step.
template <typename T>
__global__ void latent_attention_exact_kernel(const float* __restrict__ qc, float* __restrict__ out,
                                              const T* __restrict__ pool, const int32_t* __restrict__ positions,
                                              const int32_t* __restrict__ req_of_token,
                                              const int32_t* __restrict__ block_table, int table_width, int page_size,
                                              int num_pages, int heads, int r, int p, float scale, int window,
                                              const float* __restrict__ sink) {
  extern __shared__ float smem[];   // [kWarps][r] sums, then m[kWarps], l[kWarps]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int req = req_of_token[t];
  if (req < 0) return;
  const int pos = positions[t];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w = r + p;
  float qr[kMaxPerLane], acc[kMaxPerLane];
  const float* qp = qc + ((size_t)t * heads + h) * w;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    qr[i] = d < w ? qp[d] : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int32_t* bt = block_table + (size_t)req * table_width;
  for (int j = lo + warp; j <= pos; j += kWarps) {
    const int pi = j / page_size;
    const int page = pi < table_width ? bt[pi] : -1;
    if (page < 0 || page >= num_pages) continue;
    const T* row = pool + ((size_t)page * page_size + (j - pi * page_size)) * w;
    float x[kMaxPerLane];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      x[i] = d < w ? to_f32<T>(row[d]) : 0.f;
      dot = __fmaf_rn(qr[i], x[i], dot);
    }
    const float s = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float pr = expf(s - m_new);
    l = l * corr + pr;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) acc[i] = acc[i] * corr + pr * x[i];
    m = m_new;
  }
  float* acc_s = smem;
  float* m_s = smem + kWarps * r;
  float* l_s = m_s + kWarps;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < r) acc_s[warp * r + d] = acc[i];
  }
  if (lane == 0) {
    m_s[warp] = m;
    l_s[warp] = l;
  }
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int k = 0; k < kWarps; ++k) mm = fmaxf(mm, m_s[k]);
  // a sink is a score of its own in the denominator: no key, no value, not scaled
  if (sink != nullptr) mm = fmaxf(mm, sink[h]);
  float ll = sink != nullptr ? expf(sink[h] - mm) : 0.f, wgt[kWarps];
#pragma unroll
  for (int k = 0; k < kWarps; ++k) {
    wgt[k] = (m_s[k] == -INFINITY) ? 0.f : expf(m_s[k] - mm);
    ll += l_s[k] * wgt[k];
  }
  float* op = out + ((size_t)t * heads + h) * r;
  for (int d = threadIdx.x; d < r; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < kWarps; ++k) o += acc_s[k * r + d] * wgt[k];
    op[d] = ll > 0.f ? o / ll : 0.f;
  }
}

// ---- the tensor-core attention ------------------------------------------------------------------------------------------
// bfloat16 rows, mma.sync.m16n8k16 with float32 accumulators.  All heads of a token read the same rows, so a tile
// of 32 or 64 query rows is (tokens x heads) of one request in token order: a decode step fills it with the heads of
// one token, a prompt portion with several tokens.  A block walks the rows its tile can see 64 at a time (cp.async,
// two buffers, a page lookup per row).  Per 64 rows and group of 32 queries (4 warps): each warp computes the scores
// of 16 rows for the 32 queries (K = r + p), the row maxima meet in shared memory, the weights exp(s - m) go to
// shared memory as TWO bfloat16 halves (rounding and rounding of the rest: 16 bits of mantissa, since weights are
// 32-bit by the design's rule), and each warp then adds weights x rows[:, its quarter of the r columns] to its
// accumulators (the rows are the B operand through ldmatrix.trans).  Maxima, sums and accumulators are float32.
// In steps of single tokens the 64-row tiles of a request are dealt to `n_splits` blocks in turn (z of the grid);
// each leaves its unnormalised sums, maximum and sum of weights, which `latent_merge` adds in the order of z.
constexpr int kKeyTile = 64;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct LatentMma {
  const void* q_lat; int q_lat_bf16; long ql_n, ql_h;   // [.., r] per (token, head): float32 or bfloat16, any strides
  const float* q_rot; long qr_n, qr_h;                  // [.., p] per (token, head)
  void* out; int out_bf16; long o_n, o_h;               // [.., r] per (token, head)
  const __nv_bfloat16* pool;
  const int32_t* positions; const int32_t* q_start;
  const int32_t* block_table; int table_width, page_size, num_pages;
  int heads, p; float scale; int window;
  const float* sink;                                    // [heads] or null: a score without key and value in every denominator
  int n_splits; float* part_o; float* part_ml;          // [splits, tokens * heads, r] and [.., 2] when n_splits > 1
  int n_tokens;
};

template <int R, int WR>                            // WR groups of 32 queries (4 warps each) share the rows they read
__global__ void __launch_bounds__(128 * WR) latent_attention_mma_kernel(const LatentMma a) {
  constexpr int NT = R / 32;                       // 8-column tiles of the output a warp owns
  constexpr int BM = 32 * WR, THREADS = 128 * WR, TPR = THREADS / kKeyTile;   // threads per row of a tile of keys
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int W = R + a.p, LD = W + 8;               // rows of (W + 8) * 2 bytes: fragment loads hit 32 distinct banks
  constexpr int LDP = kKeyTile + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [BM][LD]
  __nv_bfloat16* Ks = Qs + BM * LD;                                          // [2][64][LD]
  __nv_bfloat16* Ph = Ks + 2 * kKeyTile * LD;                                // [BM][LDP]
  __nv_bfloat16* Pl = Ph + BM * LDP;                                         // [BM][LDP]
  float* red = reinterpret_cast<float*>(Pl + BM * LDP);                      // [4][BM]
  int* row_pos = reinterpret_cast<int*>(red + 4 * BM);                       // [BM]
  pdl_launch_dependents();
  pdl_wait();
  const int req = blockIdx.y;
  const int q0 = a.q_start[req], q_len = a.q_start[req + 1] - q0;
  // the last tiles of a portion see the most rows: they go first, so that the launch does not end on its longest blocks
  const int n_rows = q_len * a.heads, row0 = (int)(gridDim.x - 1 - blockIdx.x) * BM;
  if (row0 >= n_rows) return;
  const int rows_here = min(BM, n_rows - row0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
  const int wc = warp & 3, rb = (warp >> 2) * 32;  // this warp's quarter of keys / columns, its group's first query

  // the tile's queries as bfloat16, and each row's position
  for (int i = tid; i < BM * W; i += THREADS) {
    const int r = i / W, c = i - r * W;
    float v = 0.f;
    if (r < rows_here) {
      const int tok = q0 + (row0 + r) / a.heads, h = (row0 + r) % a.heads;
      if (c < R) {
        v = a.q_lat_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.q_lat)[(size_t)tok * a.ql_n + (size_t)h * a.ql_h + c])
                         : reinterpret_cast<const float*>(a.q_lat)[(size_t)tok * a.ql_n + (size_t)h * a.ql_h + c];
      } else {
        v = a.q_rot[(size_t)tok * a.qr_n + (size_t)h * a.qr_h + (c - R)];
      }
    }
    Qs[r * LD + c] = __float2bfloat16_rn(v);
  }
  if (tid < BM) row_pos[tid] = tid < rows_here ? a.positions[q0 + (row0 + tid) / a.heads] : -1;
  const int pos_first = a.positions[q0 + row0 / a.heads];
  const int pos_last = a.positions[q0 + (row0 + rows_here - 1) / a.heads];
  const int lo = (a.window > 0 && pos_first - a.window + 1 > 0) ? pos_first - a.window + 1 : 0;
  const int n_tiles = (pos_last - lo) / kKeyTile + 1;
  const int32_t* bt = a.block_table + (size_t)req * a.table_width;
  const int chunks = W / 8;
  const int step = a.n_splits, tile_first = blockIdx.z;

  // TPR threads per row of a tile: each looks its row's page up one tile before the tile is asked for (the lookup is a
  // trip to the L2 that would otherwise sit between a tile's arrival and its use), then copies 16-byte pieces in turn
  auto page_of = [&](int tile) {
    const int j = lo + tile * kKeyTile + tid / TPR;
    if (tile >= n_tiles || j > pos_last) return -1;
    const int pi = j / a.page_size;
    return pi < a.table_width ? bt[pi] : -1;
  };
  auto load = [&](int tile, int buf, int page) {
    __nv_bfloat16* dst = Ks + (size_t)buf * kKeyTile * LD;
    const int r = tid / TPR, j = lo + tile * kKeyTile + r;
    const bool ok = page >= 0 && page < a.num_pages;
    const __nv_bfloat16* src = ok ? a.pool + ((size_t)page * a.page_size + (j % a.page_size)) * W : a.pool;
    for (int ch = tid % TPR; ch < chunks; ch += TPR) cp_async_16(dst + r * LD + ch * 8, ok ? src + ch * 8 : a.pool, ok);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float o[2][NT][4] = {};
  float m_run[2][2], l_run[2][2];                  // [m-tile][row g / row g + 8]; l: this warp's share of the sum
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      m_run[mt][hf] = -INFINITY;
      l_run[mt][hf] = 0.f;
    }

  if (tile_first < n_tiles) load(tile_first, 0, page_of(tile_first));
  int buf = 0, page_next = page_of(tile_first + step);
  for (int tile = tile_first; tile < n_tiles; tile += step, buf ^= 1) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                // this tile is in place; everyone is done with the one before
    if (tile + step < n_tiles) load(tile + step, buf ^ 1, page_next);
    page_next = page_of(tile + 2 * step);
    const __nv_bfloat16* Kt = Ks + (size_t)buf * kKeyTile * LD;
    // scores of this warp's 16 rows for its group's 32 queries
    float s[2][2][4] = {}, s2[2][2][4] = {};           // even and odd steps of K apart: twice the MMAs in flight
    for (int k0 = 0; k0 < W; k0 += 16) {
      uint32_t af[2][4], bq[4];                     // fragments by ldmatrix: three instructions feed four MMAs
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const unsigned addr = (unsigned)__cvta_generic_to_shared(Qs + (rb + mt * 16 + (lane & 15)) * LD + k0 + (lane >> 4) * 8);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(af[mt][0]), "=r"(af[mt][1]), "=r"(af[mt][2]), "=r"(af[mt][3]) : "r"(addr));
      }
      {
        const unsigned addr = (unsigned)__cvta_generic_to_shared(
            Kt + (wc * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + k0 + ((lane >> 3) & 1) * 8);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(bq[0]), "=r"(bq[1]), "=r"(bq[2]), "=r"(bq[3]) : "r"(addr));
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const uint32_t b0 = bq[2 * nt], b1 = bq[2 * nt + 1];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          if (k0 & 16) mma_bf16(s2[mt][nt], af[mt], b0, b1);
          else mma_bf16(s[mt][nt], af[mt], b0, b1);
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[mt][nt][e] += s2[mt][nt][e];
    // mask, scale, row maxima of this warp's keys
    const int key0 = lo + tile * kKeyTile + wc * 16;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int pos = row_pos[rb + mt * 16 + gq + hf * 8];
        float m = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = key0 + nt * 8 + 2 * tq + e;
            const bool vis = pos >= 0 && j <= pos && (a.window <= 0 || j > pos - a.window);
            const float v = vis ? s[mt][nt][hf * 2 + e] * a.scale : -INFINITY;
            s[mt][nt][hf * 2 + e] = v;
            m = fmaxf(m, v);
          }
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        if (tq == 0) red[wc * BM + rb + mt * 16 + gq + hf * 8] = m;
      }
    __syncthreads();
    float corr[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int r = rb + mt * 16 + gq + hf * 8;
        const float m_new = fmaxf(fmaxf(m_run[mt][hf], fmaxf(red[r], red[BM + r])), fmaxf(red[2 * BM + r], red[3 * BM + r]));
        corr[mt][hf] = m_new == -INFINITY ? 1.f : expf(m_run[mt][hf] - m_new);
        m_run[mt][hf] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          float pv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float v = s[mt][nt][hf * 2 + e];
            pv[e] = v == -INFINITY ? 0.f : expf(v - m_new);
            sum += pv[e];
          }
          const __nv_bfloat162 hi = __floats2bfloat162_rn(pv[0], pv[1]);
          const __nv_bfloat162 lw = __floats2bfloat162_rn(pv[0] - __bfloat162float(hi.x), pv[1] - __bfloat162float(hi.y));
          const int c = wc * 16 + nt * 8 + 2 * tq;
          *reinterpret_cast<__nv_bfloat162*>(Ph + r * LDP + c) = hi;
          *reinterpret_cast<__nv_bfloat162*>(Pl + r * LDP + c) = lw;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_run[mt][hf] = l_run[mt][hf] * corr[mt][hf] + sum;
      }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        o[mt][nt][0] *= corr[mt][0];
        o[mt][nt][1] *= corr[mt][0];
        o[mt][nt][2] *= corr[mt][1];
        o[mt][nt][3] *= corr[mt][1];
      }
    __syncthreads();                                // the weights of all 64 rows are in place
    // this warp's quarter of the columns: o += P . rows[:, quarter]
#pragma unroll
    for (int kk = 0; kk < kKeyTile; kk += 16) {
      uint32_t ah[2][4], al[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int off = (rb + mt * 16 + (lane & 15)) * LDP + kk + (lane >> 4) * 8;
        const unsigned addr_h = (unsigned)__cvta_generic_to_shared(Ph + off), addr_l = (unsigned)__cvta_generic_to_shared(Pl + off);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(ah[mt][0]), "=r"(ah[mt][1]), "=r"(ah[mt][2]), "=r"(ah[mt][3]) : "r"(addr_h));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(al[mt][0]), "=r"(al[mt][1]), "=r"(al[mt][2]), "=r"(al[mt][3]) : "r"(addr_l));
      }
      // rows kk .. kk + 15 of the tile as the B operand, transposed on the way: two 8-column tiles a load
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        const __nv_bfloat16* vp = Kt + (kk + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + wc * (R / 4) + np * 16 + (lane >> 4) * 8;
        uint32_t b[4];
        const unsigned addr = (unsigned)__cvta_generic_to_shared(vp);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(addr));
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma_bf16(o[mt][2 * np + half], ah[mt], b[2 * half], b[2 * half + 1]);
            mma_bf16(o[mt][2 * np + half], al[mt], b[2 * half], b[2 * half + 1]);
          }
      }
      if constexpr (NT % 2) {                       // an odd tile left over (r = 96)
        constexpr int nt = NT - 1;
        const __nv_bfloat16* vp = Kt + (kk + (lane & 15)) * LD + wc * (R / 4) + nt * 8;
        uint32_t b0, b1;
        const unsigned addr = (unsigned)__cvta_generic_to_shared(vp);
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          mma_bf16(o[mt][nt], ah[mt], b0, b1);
          mma_bf16(o[mt][nt], al[mt], b0, b1);
        }
      }
    }
  }
  // the four warps' shares of the sums, in warp order
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf)
      if (tq == 0) red[wc * BM + rb + mt * 16 + gq + hf * 8] = l_run[mt][hf];
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = rb + mt * 16 + gq + hf * 8;
      if (r >= rows_here) continue;
      const float l = ((red[r] + red[BM + r]) + red[2 * BM + r]) + red[3 * BM + r];
      const int tok = q0 + (row0 + r) / a.heads, h = (row0 + r) % a.heads;
      if (a.n_splits > 1) {                         // this block's share, for the merge
        const size_t row = ((size_t)blockIdx.z * a.n_tokens + tok) * a.heads + h;
        if (wc == 0 && tq == 0) {
          a.part_ml[row * 2] = m_run[mt][hf];
          a.part_ml[row * 2 + 1] = l;
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int c = wc * (R / 4) + nt * 8 + 2 * tq;
          a.part_o[row * R + c] = o[mt][nt][hf * 2];
          a.part_o[row * R + c + 1] = o[mt][nt][hf * 2 + 1];
        }
        continue;
      }
      float inv = l > 0.f ? 1.0f / l : 0.f;
      if (a.sink != nullptr) {                      // the sums stand relative to m_run: bring the sink to the same scale
        const float sk = a.sink[h], mf = fmaxf(m_run[mt][hf], sk);
        const float c = m_run[mt][hf] == -INFINITY ? 0.f : expf(m_run[mt][hf] - mf);
        inv = c / (l * c + expf(sk - mf));
      }
      const size_t base = (size_t)tok * a.o_n + (size_t)h * a.o_h + wc * (R / 4);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const float v0 = o[mt][nt][hf * 2] * inv, v1 = o[mt][nt][hf * 2 + 1] * inv;
        const int c = nt * 8 + 2 * tq;
        if (a.out_bf16) {
          reinterpret_cast<__nv_bfloat16*>(a.out)[base + c] = __float2bfloat16_rn(v0);
          reinterpret_cast<__nv_bfloat16*>(a.out)[base + c + 1] = __float2bfloat16_rn(v1);
        } else {
          reinterpret_cast<float*>(a.out)[base + c] = v0;
          reinterpret_cast<float*>(a.out)[base + c + 1] = v1;
        }
      }
    }
}

// out = sum_z o_z exp(m_z - M) / sum_z l_z exp(m_z - M) in the order of z (at most 32 shares).  One warp per
// (token, head): lane z weighs share z, then every column adds its shares in the order of z.
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int n_splits,
                                    int n_tokens, int heads, int r, const int32_t* __restrict__ req_of_token, void* out,
                                    int out_bf16, long o_n, long o_h, const float* __restrict__ sink) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_tokens * heads) return;
  const int tok = row / heads, h = row - tok * heads;
  if (req_of_token[tok] < 0) return;
  const size_t rows = (size_t)n_tokens * heads;
  const float m = lane < n_splits ? part_ml[((size_t)lane * rows + row) * 2] : -INFINITY;
  const float lz = lane < n_splits ? part_ml[((size_t)lane * rows + row) * 2 + 1] : 0.f;
  float M = warp_max(m);
  if (sink != nullptr) M = fmaxf(M, sink[h]);
  const float wz = m == -INFINITY ? 0.f : expf(m - M);
  float l = warp_sum(lz * wz);
  if (sink != nullptr) l += expf(sink[h] - M);
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  for (int c = lane; c < r; c += 32) {
    float acc = 0.f;
#pragma unroll 8
    for (int z = 0; z < n_splits; ++z) {
      // loaded whether it counts or not (a share without rows holds no numbers), so that the loads go out together
      const float v = part_o[((size_t)z * rows + row) * r + c];
      const float w = __shfl_sync(0xffffffffu, wz, z);
      acc = __fmaf_rn(w > 0.f ? v : 0.f, w, acc);
    }
    const size_t at = (size_t)tok * o_n + (size_t)h * o_h + c;
    if (out_bf16) reinterpret_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(acc * inv);
    else reinterpret_cast<float*>(out)[at] = acc * inv;
  }
}

template <int R, int WR>
size_t latent_mma_smem(int p) {
  const int LD = R + p + 8;
  return (size_t)(32 * WR + 2 * kKeyTile) * LD * 2 + 2 * (size_t)32 * WR * (kKeyTile + 8) * 2 + 5 * 32 * WR * 4;
}

template <int R, int WR>
int launch_latent_mma(const LatentMma& a, int max_rows, int n_requests, cudaStream_t stream) {
  const size_t smem = latent_mma_smem<R, WR>(a.p);
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(latent_attention_mma_kernel<R, WR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return YALIS_ERR_LAUNCH;
    configured = smem;
  }
  const dim3 grid((max_rows + 32 * WR - 1) / (32 * WR), n_requests, a.n_splits);
  return yalis_launch(latent_attention_mma_kernel<R, WR>, grid, dim3(128 * WR), smem, stream, a);
}

// Tiles of 64 queries where a step has that many rows per request and shared memory has the room, else of 32.
template <int R>
int launch_latent_mma_any(const LatentMma& a, int max_rows, int n_requests, cudaStream_t stream) {
  if (max_rows > 32 && latent_mma_smem<R, 2>(a.p) <= 227 * 1024) return launch_latent_mma<R, 2>(a, max_rows, n_requests, stream);
  return launch_latent_mma<R, 1>(a, max_rows, n_requests, stream);
}

}  // namespace

YALIS_API int yalis_latent_prepare(const void* src, int dtype, int src_stride, int q_off, int kv_off, int heads, int d,
                                   int r, int p, const float* norm_w, float eps, const float* inv_freq, int rot_dims,
                                   int interleaved, float magnitude, float* qc, void* pool,
                                   const int32_t* block_table, int table_width, int page_size, int num_pages,
                                   const int32_t* positions, const int32_t* req_of_token, int n_tokens,
                                   int32_t* bad_page, const void* q_src, int q_stride, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || heads > 65535 || d < 0 || r <= 0 || p < 0) return YALIS_ERR_SHAPE;
  if (inv_freq && (rot_dims <= 0 || (rot_dims & 1) || rot_dims > p)) return YALIS_ERR_SHAPE;
  LatentPrep a;
  a.src = src; a.src_stride = src_stride; a.q_off = q_off; a.kv_off = kv_off; a.heads = heads; a.d = d; a.r = r; a.p = p;
  a.norm_w = norm_w; a.eps = eps; a.inv_freq = inv_freq; a.rot_dims = rot_dims; a.interleaved = interleaved;
  a.magnitude = magnitude; a.qc = qc; a.pool = pool; a.block_table = block_table; a.table_width = table_width;
  a.page_size = page_size; a.num_pages = num_pages; a.positions = positions; a.req_of_token = req_of_token;
  a.bad_page = bad_page; a.q_src = q_src; a.q_stride = q_stride;
  const int warps = 4;
  const dim3 grid(n_tokens, (heads + 1 + warps - 1) / warps);
  YALIS_DISPATCH_DTYPE(dtype, T, return yalis_launch(latent_prepare_kernel<T>, grid, dim3(32 * warps), 0, stream, a));
  return YALIS_OK;
}

YALIS_API int yalis_norm_rows(const void* x, long x_stride, const float* w, float eps, int width, void* y, long y_stride,
                              int n_rows, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return YALIS_OK;
  if (width <= 0) return YALIS_ERR_SHAPE;
  const int warps = 4;
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(norm_rows_kernel<T>, dim3((n_rows + warps - 1) / warps), dim3(32 * warps), 0, stream,
                                           (const T*)x, x_stride, w, eps, width, (T*)y, y_stride, n_rows));
  return YALIS_OK;
}

// x_dtype / out_dtype: float32 or the model dtype `dtype` of w and gate.
YALIS_API int yalis_head_project(const void* x, int x_dtype, long xs_n, long xs_h, const void* w, int dtype, int heads,
                                 int O, int K, void* out, int out_dtype, long os_n, long os_h, const void* gate,
                                 long gs_n, const int32_t* req_of_token, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || heads > 65535 || O <= 0 || K <= 0 || K > 12288) return YALIS_ERR_SHAPE;
  const dim3 grid(n_tokens, heads), block(256);
  const size_t smem = (size_t)K * sizeof(float);
#define YALIS_HP(T, TX, TO)                                                                                         \
  return yalis_launch(head_project_kernel<T, TX, TO>, grid, block, smem, stream, (const TX*)x, xs_n, xs_h, (const T*)w, \
                      O, K, (TO*)out, os_n, os_h, (const T*)gate, gs_n, req_of_token)
  if (dtype == YALIS_F32 && x_dtype == YALIS_F32 && out_dtype == YALIS_F32) YALIS_HP(float, float, float);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_BF16 && out_dtype == YALIS_F32) YALIS_HP(__nv_bfloat16, __nv_bfloat16, float);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_F32 && out_dtype == YALIS_BF16) YALIS_HP(__nv_bfloat16, float, __nv_bfloat16);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_F32 && out_dtype == YALIS_F32) YALIS_HP(__nv_bfloat16, float, float);
#undef YALIS_HP
  return YALIS_ERR_DTYPE;
}

YALIS_API int yalis_sigmoid_gate(const void* x, int x_dtype, long xs_n, long xs_h, int e, const void* g, long gs, void* y,
                                 long ys, int dtype, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return YALIS_OK;
  if (e <= 0 || cols % e) return YALIS_ERR_SHAPE;
  const size_t total = (size_t)rows * cols;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == YALIS_F32 && x_dtype == YALIS_F32)
    return yalis_launch(sigmoid_gate_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, xs_n, xs_h, e,
                        (const float*)g, gs, (float*)y, ys, rows, cols);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_F32)
    return yalis_launch(sigmoid_gate_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, xs_n,
                        xs_h, e, (const __nv_bfloat16*)g, gs, (__nv_bfloat16*)y, ys, rows, cols);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_BF16)
    return yalis_launch(sigmoid_gate_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                        (const __nv_bfloat16*)x, xs_n, xs_h, e, (const __nv_bfloat16*)g, gs, (__nv_bfloat16*)y, ys, rows, cols);
  return YALIS_ERR_DTYPE;
}

YALIS_API int yalis_latent_attention_exact(const float* qc, float* out, const void* pool, int dtype,
                                           const int32_t* positions, const int32_t* req_of_token,
                                           const int32_t* block_table, int table_width, int page_size, int num_pages,
                                           int n_tokens, int heads, int r, int p, float scale, int window,
                                           const float* sink, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || heads > 65535 || r <= 0 || p < 0 || r + p > 32 * kMaxPerLane) return YALIS_ERR_SHAPE;
  const size_t smem = ((size_t)kWarps * r + 2 * kWarps) * sizeof(float);
  const dim3 grid(n_tokens, heads);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(latent_attention_exact_kernel<T>, grid, dim3(kWarps * 32), smem, stream, qc, out,
                                           (const T*)pool, positions, req_of_token, block_table, table_width, page_size,
                                           num_pages, heads, r, p, scale, window, sink));
  return YALIS_OK;
}

// Whether the tensor-core form takes these sizes: r one of 64, 96, 128, 256, 384, 512 and p a multiple of 16 with
// (32 + 128) rows of r + p + 8 bfloat16 within an SM's shared memory.
YALIS_API int yalis_latent_attention_mma_supports(int r, int p) {
  if (!(r == 64 || r == 96 || r == 128 || r == 256 || r == 384 || r == 512) || p < 0 || p % 16) return 0;
  return (size_t)(32 + 2 * kKeyTile) * (r + p + 8) * 2 + 10240 <= 227 * 1024 ? 1 : 0;
}

// max_q_len: the longest portion of the step (bounds the grid); q_lat / out: float32 or bfloat16 by their flags.
// n_splits > 1 (steps of single tokens): part_o float32 [n_splits, n_tokens * heads, r], part_ml [.., 2].
YALIS_API int yalis_latent_attention_mma(const void* q_lat, int q_lat_bf16, long ql_n, long ql_h, const float* q_rot, long qr_n,
                                         long qr_h, void* out, int out_bf16, long o_n, long o_h, const void* pool,
                                         const int32_t* positions, const int32_t* q_start, const int32_t* req_of_token,
                                         const int32_t* block_table, int table_width, int page_size, int num_pages,
                                         int n_requests, int n_tokens, int max_q_len, int heads, int r, int p, float scale,
                                         int window, const float* sink, int n_splits, float* part_o, float* part_ml,
                                         cudaStream_t stream) {
  if (n_requests <= 0 || max_q_len <= 0) return YALIS_OK;
  if (!yalis_latent_attention_mma_supports(r, p) || heads <= 0 || n_requests > 65535 || n_splits < 1 || n_splits > 32)
    return YALIS_ERR_SHAPE;
  if (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return YALIS_ERR_SHAPE;
  if ((uintptr_t)pool & 15) return YALIS_ERR_ALIGN;
  LatentMma a;
  a.q_lat = q_lat; a.q_lat_bf16 = q_lat_bf16; a.ql_n = ql_n; a.ql_h = ql_h; a.q_rot = q_rot; a.qr_n = qr_n; a.qr_h = qr_h;
  a.out = out; a.out_bf16 = out_bf16; a.o_n = o_n; a.o_h = o_h; a.pool = (const __nv_bfloat16*)pool; a.positions = positions;
  a.q_start = q_start; a.block_table = block_table; a.table_width = table_width; a.page_size = page_size;
  a.num_pages = num_pages; a.heads = heads; a.p = p; a.scale = scale; a.window = window; a.sink = sink;
  a.n_splits = n_splits; a.part_o = part_o; a.part_ml = part_ml; a.n_tokens = n_tokens;
  const int max_rows = max_q_len * heads;
  int status = YALIS_ERR_SHAPE;
  switch (r) {
    case 64: status = launch_latent_mma_any<64>(a, max_rows, n_requests, stream); break;
    case 96: status = launch_latent_mma_any<96>(a, max_rows, n_requests, stream); break;
    case 128: status = launch_latent_mma_any<128>(a, max_rows, n_requests, stream); break;
    case 256: status = launch_latent_mma_any<256>(a, max_rows, n_requests, stream); break;
    case 384: status = launch_latent_mma_any<384>(a, max_rows, n_requests, stream); break;
    case 512: status = launch_latent_mma_any<512>(a, max_rows, n_requests, stream); break;
  }
  if (status != YALIS_OK || n_splits == 1) return status;
  const int rows = n_tokens * heads, warps = 4;
  return yalis_launch(latent_merge_kernel, dim3((rows + warps - 1) / warps), dim3(32 * warps), 0, stream, (const float*)part_o,
                      (const float*)part_ml, n_splits, n_tokens, heads, r, req_of_token, out, out_bf16, o_n, o_h, sink);
}
