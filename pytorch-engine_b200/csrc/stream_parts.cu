// Small parts around the residual stream and the mixers' inputs and outputs, all in float32 arithmetic:
//
//   norm_token_shift   h[t] = x[t] / rms(x[t]) * w ;  out[t] = h[t] + (h[t-1] - h[t]) * mix, where a sequence's first token
//                      of the step takes the row that the sequence kept (zeros at its start), and the sequence's last
//                      h of the step is kept for the next one
//   depth_average      out = sum_j coeff[j] * results[j]  over the results of the embedding and of every block so far
//   polynorm           a N(z) + b N(z^2) + c N(z^3) + e,  N(u) = u / sqrt(mean(u^2) + eps) over a token's row
//   sigmoid_gate       x[t, h, :] *= sigmoid(g[t, h])  (one gate a head)  or  x[t, c] *= sigmoid(g[t, c])
//   diff_combine       o = a1 - lambda * a2 ;  out = o / sqrt(mean(o^2) + eps) * post  per (token, head)
//   rows_to_pages      rows of a step's tokens copied into the pages of their sequences (keys, values or latent rows)
//   latent_prepare     a latent-attention layer's cached row and the rotated part of its queries (see the kernel)
#include "api.h"
#include "common.cuh"

namespace pe {

// grid: tokens; block: threads over the width.
template <typename T>
__global__ void __launch_bounds__(256) norm_token_shift_kernel(const float* x, const float* __restrict__ w, float eps,
                                                               const float* __restrict__ mix, float* state,
                                                               const int* token_seq, const int* seq_slot,
                                                               const int* seq_qstart, T* __restrict__ out, int n_tokens,
                                                               int width, int n_slots, int* status) {
  __shared__ float red[32];
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const bool first = t == seq_qstart[b];
  const int slot = seq_slot[b];
  if (first && (slot < 0 || slot >= n_slots)) {
    if (threadIdx.x == 0) report(status, kStatusSlotOutOfRange, t, slot, n_slots);
    return;
  }
  const float* cur = x + (size_t)t * width;
  // the other row this block needs: the previous token's, or (first token) the sequence's last row of the step
  const float* other = first ? x + (size_t)(seq_qstart[b + 1] - 1) * width : cur - width;
  float s0 = 0.f, s1 = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float a = cur[c], o = other[c];
    s0 = fmaf(a, a, s0);
    s1 = fmaf(o, o, s1);
  }
  s0 = block_sum(s0, red);
  s1 = block_sum(s1, red);
  const float inv0 = rsqrtf(s0 / (float)width + eps), inv1 = rsqrtf(s1 / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float h = cur[c] * inv0 * w[c];
    const float ho = other[c] * inv1 * w[c];
    float hp = ho;
    if (first) {
      // this thread alone reads and writes the element: the kept row is read before it is replaced
      hp = state[(size_t)slot * width + c];
      state[(size_t)slot * width + c] = ho;
    }
    out[(size_t)t * width + c] = from_f32<T>(fmaf(hp - h, mix[c], h));
  }
}

__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// The same for rows that a block holds in registers (width a multiple of 4, at most 4 * VPT * 256): every global read
// is issued before the first reduction, and each row is read once.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) norm_token_shift_rows_kernel(const float* x, const float* __restrict__ w, float eps,
                                                                    const float* __restrict__ mix, float* state,
                                                                    const int* token_seq, const int* seq_slot,
                                                                    const int* seq_qstart, T* __restrict__ out, int n_tokens,
                                                                    int width, int n_slots, int* status) {
  __shared__ float red[32];
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const bool first = t == seq_qstart[b];
  const int slot = seq_slot[b];
  if (first && (slot < 0 || slot >= n_slots)) {
    if (threadIdx.x == 0) report(status, kStatusSlotOutOfRange, t, slot, n_slots);
    return;
  }
  const int nv = width >> 2;
  const float4* cur = reinterpret_cast<const float4*>(x + (size_t)t * width);
  const float4* other = first ? reinterpret_cast<const float4*>(x + (size_t)(seq_qstart[b + 1] - 1) * width) : cur - nv;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const float4* m4 = reinterpret_cast<const float4*>(mix);
  float4* kept4 = reinterpret_cast<float4*>(state + (size_t)(first ? slot : 0) * width);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 a[VPT], o[VPT], wv[VPT], mv[VPT], kp[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * 256;
    const bool in = c < nv;
    a[k] = in ? cur[c] : zero;
    o[k] = in ? other[c] : zero;
    wv[k] = in ? w4[c] : zero;
    mv[k] = in ? m4[c] : zero;
    kp[k] = (in && first) ? kept4[c] : zero;
  }
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    s0 = fmaf(a[k].x, a[k].x, fmaf(a[k].y, a[k].y, fmaf(a[k].z, a[k].z, fmaf(a[k].w, a[k].w, s0))));
    s1 = fmaf(o[k].x, o[k].x, fmaf(o[k].y, o[k].y, fmaf(o[k].z, o[k].z, fmaf(o[k].w, o[k].w, s1))));
  }
  s0 = block_sum(s0, red);
  s1 = block_sum(s1, red);
  const float inv0 = rsqrtf(s0 / (float)width + eps), inv1 = rsqrtf(s1 / (float)width + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * 256;
    if (c >= nv) continue;
    const float4 h = make_float4(a[k].x * inv0 * wv[k].x, a[k].y * inv0 * wv[k].y, a[k].z * inv0 * wv[k].z, a[k].w * inv0 * wv[k].w);
    const float4 ho = make_float4(o[k].x * inv1 * wv[k].x, o[k].y * inv1 * wv[k].y, o[k].z * inv1 * wv[k].z, o[k].w * inv1 * wv[k].w);
    float4 hp = ho;
    if (first) {
      hp = kp[k];       // read above, before this thread (alone) replaces it
      kept4[c] = ho;
    }
    store4(out + (size_t)t * width + 4 * c, fmaf(hp.x - h.x, mv[k].x, h.x), fmaf(hp.y - h.y, mv[k].y, h.y),
           fmaf(hp.z - h.z, mv[k].z, h.z), fmaf(hp.w - h.w, mv[k].w, h.w));
  }
}

__global__ void depth_average_kernel(const float* results, long long layer_stride, const float* __restrict__ coeff,
                                     int n_terms, float* __restrict__ out, float* __restrict__ copy, long long n) {
  pdl_wait_block();
  pdl_launch_dependents();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < n_terms; ++j) acc = fmaf(coeff[j], results[(size_t)j * layer_stride + i], acc);
    out[i] = acc;
    if (copy) copy[i] = acc;
  }
}

// grid: rows; the row is read twice (sums, then values).
template <typename T>
__global__ void __launch_bounds__(256) polynorm_kernel(const T* z, const float* __restrict__ coeff, float eps,
                                                       T* __restrict__ out, int width) {
  __shared__ float red[32];
  pdl_wait_block();
  pdl_launch_dependents();
  const T* row = z + (size_t)blockIdx.x * width;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_f32<T>(row[c]), v2 = v * v, v3 = v2 * v;
    s1 = fmaf(v, v, s1);
    s2 = fmaf(v2, v2, s2);
    s3 = fmaf(v3, v3, s3);
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  s3 = block_sum(s3, red);
  const float n = (float)width;
  const float f1 = coeff[0] * rsqrtf(s1 / n + eps), f2 = coeff[1] * rsqrtf(s2 / n + eps), f3 = coeff[2] * rsqrtf(s3 / n + eps);
  const float e = coeff[3];
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_f32<T>(row[c]), v2 = v * v;
    out[(size_t)blockIdx.x * width + c] = from_f32<T>(fmaf(f1, v, fmaf(f2, v2, fmaf(f3, v2 * v, e))));
  }
}

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 q;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = q;
  }
};

// The same for rows that a block holds in registers (rows of whole 16-byte vectors, at most VPT a thread): the row is
// read once.  grid: rows; block: any multiple of 32 threads.
template <typename T, int VPT>
__global__ void __launch_bounds__(1024) polynorm_rows_kernel(const T* z, const float* __restrict__ coeff, float eps,
                                                             T* __restrict__ out, int width) {
  __shared__ float red[32];
  pdl_wait_block();
  pdl_launch_dependents();
  constexpr int N = Vec16<T>::N;
  const int nv = width / N;
  const T* row = z + (size_t)blockIdx.x * width;
  float v[VPT][N];
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < nv) {
      Vec16<T>::load(row + (size_t)c * N, v[k]);
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) v[k][i] = 0.f;
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const float u = v[k][i], u2 = u * u, u3 = u2 * u;
      s1 = fmaf(u, u, s1);
      s2 = fmaf(u2, u2, s2);
      s3 = fmaf(u3, u3, s3);
    }
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  s3 = block_sum(s3, red);
  const float n = (float)width;
  const float f1 = coeff[0] * rsqrtf(s1 / n + eps), f2 = coeff[1] * rsqrtf(s2 / n + eps), f3 = coeff[2] * rsqrtf(s3 / n + eps);
  const float e = coeff[3];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c >= nv) continue;
    float r[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const float u = v[k][i], u2 = u * u;
      r[i] = fmaf(f1, u, fmaf(f2, u2, fmaf(f3, u2 * u, e)));
    }
    Vec16<T>::store(out + (size_t)blockIdx.x * width + (size_t)c * N, r);
  }
}

// x: feature c of head h of token t at x + h * x_head_stride + t * x_token_stride + c (heads side by side in a row, or
// one matrix a head as a product over heads leaves them); out: packed rows [n, heads * dv].
template <typename T>
__global__ void sigmoid_gate_kernel(const T* x, long long x_head_stride, long long x_token_stride, const T* g, long long g_ld,
                                    T* __restrict__ out, long long out_ld, int n_tokens, int heads, int dv, int per_head) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int row = heads * dv;
  const size_t total = (size_t)n_tokens * row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / row), c = (int)(i - (size_t)t * row);
    const int h = c / dv;
    const float z = to_f32<T>(g[(size_t)t * g_ld + (per_head ? h : c)]);
    const float v = to_f32<T>(x[(size_t)h * x_head_stride + (size_t)t * x_token_stride + (c - h * dv)]);
    out[(size_t)t * out_ld + c] = from_f32<T>(v / (1.f + expf(-z)));
  }
}

// One warp per (token, head).  a: float32 [n, 2 * heads, dv] with the first map's heads first.
template <typename T>
__global__ void diff_combine_kernel(const float* a, T* __restrict__ out, int n_tokens, int heads, int dv, float lambda,
                                    float eps, float post) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  const float* a1 = a + ((size_t)t * 2 * heads + h) * dv;
  const float* a2 = a1 + (size_t)heads * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float o = fmaf(-lambda, a2[c], a1[c]);
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  const float f = rsqrtf(ss / (float)dv + eps) * post;
  T* o_row = out + ((size_t)t * heads + h) * dv;
  for (int c = lane; c < dv; c += 32)
    o_row[c] = from_f32<T>(fmaf(-lambda, a2[c], a1[c]) * f);
}

// Where a token's row lies in the pages of its sequence; -1 (and a status report) if the page table has none.
__device__ __forceinline__ long long page_row(int t, const int* token_seq, const int* token_pos, const int* seq_slot,
                                              const int* page_table, int table_stride, int num_pages, int* status) {
  const int pos = token_pos[t];
  const int slot = seq_slot[token_seq[t]];
  const int logical = pos / kPageTokens;
  int page = -1;
  if (pos >= 0 && logical < table_stride) page = page_table[(size_t)slot * table_stride + logical];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) report(status, kStatusPageOutOfRange, slot, page, pos);
    return -1;
  }
  return (long long)page * kPageTokens + (pos % kPageTokens);
}

// pages: [num_pages, heads, 64, dim]; src row t holds heads * dim features from column col0.  A second set (col0_b,
// heads_b, dim_b, pages_b; pages_b null: none) goes to the same page numbers of its own pool.  grid: tokens.
template <typename T>
__global__ void rows_to_pages_kernel(const T* src, long long src_ld, int col0, int heads, int dim, int col0_b, int heads_b,
                                     int dim_b, const int* token_seq, const int* token_pos, const int* seq_slot,
                                     const int* page_table, int table_stride, int num_pages, T* __restrict__ pages,
                                     T* __restrict__ pages_b, int* status) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const long long pr = page_row(t, token_seq, token_pos, seq_slot, page_table, table_stride, num_pages, status);
  if (pr < 0) return;
  const long long page = pr / kPageTokens, r = pr % kPageTokens;
  const T* row = src + (size_t)t * src_ld + col0;
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
    const int h = i / dim, c = i - h * dim;
    pages[(((size_t)page * heads + h) * kPageTokens + r) * dim + c] = row[i];
  }
  if (pages_b == nullptr) return;
  const T* row_b = src + (size_t)t * src_ld + col0_b;
  for (int i = threadIdx.x; i < heads_b * dim_b; i += blockDim.x) {
    const int h = i / dim_b, c = i - h * dim_b;
    pages_b[(((size_t)page * heads_b + h) * kPageTokens + r) * dim_b + c] = row_b[i];
  }
}

// A latent-attention layer's step, per token (grid: tokens).  x row: [.. q: heads x (d + dr) at q_col0 ..
// low: rank + dr at low_col0 ..].
//   cached row  = [ low[:rank] / rms(low[:rank]) * norm_w | turn(low[rank:]) ]        -> pages [num_pages, 1, 64, rank + dr]
//   qfull[t, h] = [ absorbed[h, t] (a product over heads left it as [heads, n, rank]; null: left as it is) | turn(q[h, d:]) ]
// turn: adjacent pairs (2i, 2i+1) of the first `rot` features by the angle tables' row of the token's position.
template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const T* x, long long x_ld, int q_col0, int low_col0, int heads,
                                                             int d, int dr, int rank, const float* __restrict__ norm_w,
                                                             float eps, const float* __restrict__ cos_t,
                                                             const float* __restrict__ sin_t, int rot, int table_rows,
                                                             const int* token_seq, const int* token_pos, const int* seq_slot,
                                                             const int* page_table, int table_stride, int num_pages,
                                                             T* __restrict__ pages, T* __restrict__ qfull,
                                                             const T* absorbed, int n_tokens, int write_cache, int* status) {
  __shared__ float red[32];
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = token_pos[t];
  const T* row = x + (size_t)t * x_ld;
  const int half = rot / 2;
  if (rot > 0 && (pos < 0 || pos >= table_rows)) {
    if (threadIdx.x == 0) report(status, kStatusPositionOutOfRange, t, pos, table_rows);
    return;
  }
  const float* cs = cos_t + (size_t)pos * half;
  const float* sn = sin_t + (size_t)pos * half;
  // the rotated part of every head's query
  const int wide = rank + dr;
  for (int i = threadIdx.x; i < heads * dr; i += blockDim.x) {
    const int h = i / dr, c = i - h * dr;
    const T* q = row + q_col0 + (size_t)h * (d + dr) + d;
    float v = to_f32<T>(q[c]);
    if (c < rot) {
      const int m = c >> 1;
      const float o = to_f32<T>(q[c ^ 1]);
      v = (c & 1) ? fmaf(v, cs[m], o * sn[m]) : fmaf(v, cs[m], -o * sn[m]);
    }
    qfull[((size_t)t * heads + h) * wide + rank + c] = from_f32<T>(v);
  }
  if (absorbed) {
    for (int i = threadIdx.x; i < heads * rank; i += blockDim.x) {
      const int h = i / rank, c = i - h * rank;
      qfull[((size_t)t * heads + h) * wide + c] = absorbed[((size_t)h * n_tokens + t) * rank + c];
    }
  }
  if (!write_cache) return;
  const T* low = row + low_col0;
  float ss = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    const float v = to_f32<T>(low[c]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)rank + eps);
  const long long pr = page_row(t, token_seq, token_pos, seq_slot, page_table, table_stride, num_pages, status);
  if (pr < 0) return;
  T* dst = pages + (size_t)pr * wide;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f32<T>(to_f32<T>(low[c]) * inv * norm_w[c]);
  for (int c = threadIdx.x; c < dr; c += blockDim.x) {
    float v = to_f32<T>(low[rank + c]);
    if (c < rot) {
      const int m = c >> 1;
      const float o = to_f32<T>(low[rank + (c ^ 1)]);
      v = (c & 1) ? fmaf(v, cs[m], o * sn[m]) : fmaf(v, cs[m], -o * sn[m]);
    }
    dst[rank + c] = from_f32<T>(v);
  }
}

static int flat_blocks(size_t total, int threads) {
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > (size_t)kSMs * 16) blocks = (size_t)kSMs * 16;
  return (int)(blocks ? blocks : 1);
}

}  // namespace pe

#define PE_BY_DTYPE(dtype, CALL)                       \
  if ((dtype) == PE_F32) { using T = float; CALL; }    \
  else if ((dtype) == PE_BF16) { using T = __nv_bfloat16; CALL; } \
  else return PE_ERR_UNSUPPORTED_DTYPE;

extern "C" int pe_norm_token_shift(int out_dtype, const float* x, const float* w, float eps, const float* mix, float* state,
                                   const int* token_seq, const int* seq_slot, const int* seq_qstart, void* out, int n_tokens,
                                   int width, int n_slots, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (width <= 0 || n_slots <= 0) return PE_ERR_BAD_ARGUMENT;
  const bool vec = width % 4 == 0 && width <= 8192 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
                   ((uintptr_t)mix % 16) == 0 && ((uintptr_t)state % 16) == 0 && ((uintptr_t)out % 16) == 0;
#define PE_NTS(KERNEL)                                                                                                     \
  PE_BY_DTYPE(out_dtype, pe::launch(KERNEL, n_tokens, 256, 0, stream, x, w, eps, mix, state, token_seq, seq_slot, seq_qstart, \
                                    (T*)out, n_tokens, width, n_slots, status))
  if (!vec) { PE_NTS(pe::norm_token_shift_kernel<T>); }
  else if (width <= 1024) { PE_NTS((pe::norm_token_shift_rows_kernel<T, 1>)); }
  else if (width <= 2048) { PE_NTS((pe::norm_token_shift_rows_kernel<T, 2>)); }
  else if (width <= 4096) { PE_NTS((pe::norm_token_shift_rows_kernel<T, 4>)); }
  else { PE_NTS((pe::norm_token_shift_rows_kernel<T, 8>)); }
#undef PE_NTS
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_depth_average(const float* results, long long layer_stride, const float* coeff, int n_terms, float* out,
                                float* copy, long long n, cudaStream_t stream) {
  if (n <= 0) return PE_OK;
  if (n_terms <= 0 || layer_stride < n) return PE_ERR_BAD_ARGUMENT;
  pe::launch(pe::depth_average_kernel, pe::flat_blocks((size_t)n, 256), 256, 0, stream, results, layer_stride, coeff, n_terms,
             out, copy, n);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_polynorm(int dtype, const void* z, const float* coeff, float eps, void* out, int n_rows, int width,
                           cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (width <= 0) return PE_ERR_BAD_ARGUMENT;
  const int per_vec = dtype == PE_F32 ? 4 : 8;
  const int nv = width / per_vec;
  // few rows: as many threads a row as it has vectors (one pass of loads in flight); many rows: 256 threads
  int threads = n_rows <= 2 * pe::kSMs ? (nv + 31) / 32 * 32 : 256;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  const int vpt = (nv + threads - 1) / threads;
  const bool vec = width % per_vec == 0 && vpt <= 4 && ((uintptr_t)z % 16) == 0 && ((uintptr_t)out % 16) == 0;
#define PE_PN(KERNEL, THREADS) \
  PE_BY_DTYPE(dtype, pe::launch(KERNEL, n_rows, THREADS, 0, stream, (const T*)z, coeff, eps, (T*)out, width))
  if (!vec) { PE_PN(pe::polynorm_kernel<T>, 256); }
  else if (vpt <= 1) { PE_PN((pe::polynorm_rows_kernel<T, 1>), threads); }
  else if (vpt <= 2) { PE_PN((pe::polynorm_rows_kernel<T, 2>), threads); }
  else { PE_PN((pe::polynorm_rows_kernel<T, 4>), threads); }
#undef PE_PN
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_sigmoid_gate(int dtype, const void* x, long long x_head_stride, long long x_token_stride, const void* g,
                               long long g_ld, void* out, long long out_ld, int n_tokens, int heads, int dv, int per_head,
                               cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (heads <= 0 || dv <= 0) return PE_ERR_BAD_ARGUMENT;
  const int blocks = pe::flat_blocks((size_t)n_tokens * heads * dv, 256);
  PE_BY_DTYPE(dtype, pe::launch(pe::sigmoid_gate_kernel<T>, blocks, 256, 0, stream, (const T*)x, x_head_stride, x_token_stride,
                                (const T*)g, g_ld, (T*)out, out_ld, n_tokens, heads, dv, per_head));
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_diff_combine(int dtype, const float* a, void* out, int n_tokens, int heads, int dv, float lambda, float eps,
                               float post, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (heads <= 0 || dv <= 0) return PE_ERR_BAD_ARGUMENT;
  const long long items = (long long)n_tokens * heads;
  const int blocks = (int)((items + 7) / 8);
  PE_BY_DTYPE(dtype, pe::launch(pe::diff_combine_kernel<T>, blocks, 256, 0, stream, a, (T*)out, n_tokens, heads, dv,
                                lambda, eps, post));
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_rows_to_pages(int dtype, const void* src, long long src_ld, int col0, int heads, int dim, int n_tokens,
                                const int* token_seq, const int* token_pos, const int* seq_slot, const int* page_table,
                                int table_stride, int num_pages, void* pages, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (heads <= 0 || dim <= 0 || col0 < 0) return PE_ERR_BAD_ARGUMENT;
  return pe_rows_to_pages_pair(dtype, src, src_ld, col0, heads, dim, 0, 0, 0, n_tokens, token_seq, token_pos, seq_slot,
                               page_table, table_stride, num_pages, pages, nullptr, status, stream);
}

// Two column ranges of the same rows into two pools that share their page numbers (keys and values) in one launch;
// pages_b null: only the first.
extern "C" int pe_rows_to_pages_pair(int dtype, const void* src, long long src_ld, int col0, int heads, int dim, int col0_b,
                                     int heads_b, int dim_b, int n_tokens, const int* token_seq, const int* token_pos,
                                     const int* seq_slot, const int* page_table, int table_stride, int num_pages,
                                     void* pages, void* pages_b, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (heads <= 0 || dim <= 0 || col0 < 0) return PE_ERR_BAD_ARGUMENT;
  if (pages_b && (heads_b <= 0 || dim_b <= 0 || col0_b < 0)) return PE_ERR_BAD_ARGUMENT;
  PE_BY_DTYPE(dtype, pe::launch(pe::rows_to_pages_kernel<T>, n_tokens, 128, 0, stream, (const T*)src, src_ld, col0, heads, dim,
                                col0_b, heads_b, dim_b, token_seq, token_pos, seq_slot, page_table, table_stride, num_pages,
                                (T*)pages, (T*)pages_b, status));
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_latent_prepare(int dtype, const void* x, long long x_ld, int q_col0, int low_col0, int heads, int d, int dr,
                                 int rank, const float* norm_w, float eps, const float* cos_t, const float* sin_t, int rot,
                                 int table_rows, int n_tokens, const int* token_seq, const int* token_pos,
                                 const int* seq_slot, const int* page_table, int table_stride, int num_pages, void* pages,
                                 void* qfull, const void* absorbed, int write_cache, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (heads <= 0 || d <= 0 || dr < 0 || rank <= 0 || rot < 0 || rot > dr || (rot & 1)) return PE_ERR_BAD_ARGUMENT;
  if (rot > 0 && (!cos_t || !sin_t)) return PE_ERR_BAD_ARGUMENT;
  PE_BY_DTYPE(dtype, pe::launch(pe::latent_prepare_kernel<T>, n_tokens, 256, 0, stream, (const T*)x, x_ld, q_col0, low_col0,
                                heads, d, dr, rank, norm_w, eps, cos_t, sin_t, rot, table_rows, token_seq, token_pos, seq_slot,
                                page_table, table_stride, num_pages, (T*)pages, (T*)qfull, (const T*)absorbed, n_tokens,
                                write_cache, status));
  PE_LAUNCH_CHECK();
  return PE_OK;
}
