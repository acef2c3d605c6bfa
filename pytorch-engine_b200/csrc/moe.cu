// Routed experts: the router's choice, the grouping of (token, choice) pairs by expert, a product whose weight matrix
// is chosen row by row, and the weighted sum of what the chosen experts return.
//
//   route     s = softmax(z) over all router outputs; the `top` largest of s + correction are chosen (ties: the
//             lower index), each weighted with its own s (not renormalised); all in float32
//   route by logits   the `top` largest of z + bias are chosen, weighted by a softmax over the chosen ones alone
//   route by groups   s = sigmoid(z); only the best groups of neighbouring experts may be chosen from; weights s
//   group     pairs whose choice is a real expert (index < n_real) are ordered by expert: offsets[e] .. offsets[e+1]
//             are expert e's rows, row_token[r] the token of row r, pair_row[t, j] the row of a pair (-1: the
//             choice is an identity expert, which returns its input)
//   product   out[r] = W[e(r)] x[row_token[r]]  (optionally act(gate rows, up rows) of a [gate | up] matrix)
//   combine   y[t] = sum_j weight[t, j] * (out[pair_row[t, j]] or x[t]) (+ shared[t])
//
// Which row a pair gets inside its expert's range depends on the order in which blocks arrive; the values do not:
// every row is computed by itself, and a token's sum runs over its choices in their own order.
#include "api.h"
#include "common.cuh"

namespace pe {

// One warp per token.
__global__ void moe_route_kernel(const float* logits, const float* __restrict__ correction, int n_tokens, int n_all, int top,
                                 int* __restrict__ chosen, float* __restrict__ weight, int* __restrict__ dense_rows, int n_real) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * n_all;
  float mx = -INFINITY;
  for (int e = lane; e < n_all; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < n_all; e += 32) sum += expf(z[e] - mx);
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  unsigned long long taken_lo = 0ull;   // this lane's entries e = lane + 32 * i, bit i set once chosen (n_all <= 2048)
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane, i = 0; e < n_all; e += 32, ++i) {
      if ((taken_lo >> i) & 1ull) continue;
      const float c = expf(z[e] - mx) * inv + correction[e];
      if (c > best) { best = c; best_e = e; }
    }
    // the warp's best: larger value, then lower index
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (best_e != 0x7fffffff && (best_e & 31) == lane) taken_lo |= 1ull << (best_e >> 5);
    if (lane == 0) {
      const bool any = best_e != 0x7fffffff;
      chosen[(size_t)t * top + j] = any ? best_e : -1;
      weight[(size_t)t * top + j] = any ? expf(z[best_e] - mx) * inv : 0.f;
      // where every expert runs on every token, the pair's row is known here
      if (dense_rows) dense_rows[(size_t)t * top + j] = (any && best_e < n_real) ? t * n_real + best_e : -1;
    }
  }
}

// The choice by the logits themselves: z' = z + bias, the `top` largest z' (ties: the lower index), weighted by a
// softmax over the chosen z' alone.  One warp per token.
__global__ void moe_route_logits_kernel(const float* logits, const float* __restrict__ bias, int n_tokens, int n_all, int top,
                                        int* __restrict__ chosen, float* __restrict__ weight, int* __restrict__ dense_rows,
                                        int n_real) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * n_all;
  unsigned long long taken_lo = 0ull;   // this lane's entries e = lane + 32 * i, bit i set once chosen (n_all <= 2048)
  float first = 0.f, sum = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane, i = 0; e < n_all; e += 32, ++i) {
      if ((taken_lo >> i) & 1ull) continue;
      const float c = z[e] + (bias ? bias[e] : 0.f);
      if (c > best || best_e == 0x7fffffff) { best = c; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) { best = ob; best_e = oe; }
    }
    if (best_e != 0x7fffffff && (best_e & 31) == lane) taken_lo |= 1ull << (best_e >> 5);
    if (j == 0) first = best;            // the largest chosen logit: the softmax's reference
    const float w = expf(best - first);
    sum += w;
    if (lane == 0) {
      chosen[(size_t)t * top + j] = best_e;
      weight[(size_t)t * top + j] = w;
      if (dense_rows) dense_rows[(size_t)t * top + j] = best_e < n_real ? t * n_real + best_e : -1;
    }
  }
  if (lane == 0) {
    const float inv = 1.f / sum;
    for (int j = 0; j < top; ++j) weight[(size_t)t * top + j] *= inv;
  }
}

// The choice among groups of neighbours: s = sigmoid(z); the outputs form `n_groups` equal groups, a group's score is the sum
// of its two largest s (its one s for groups of one), only the `keep` best groups (ties: the lower group) may be chosen from;
// the `top` largest s among those (ties: the lower index), weighted with s itself.  n_groups <= 1: no groups.  One warp per token.
__global__ void moe_route_sigmoid_groups_kernel(const float* logits, int n_tokens, int n_all, int top, int n_groups, int keep,
                                                int* __restrict__ chosen, float* __restrict__ weight, int* __restrict__ dense_rows,
                                                int n_real) {
  extern __shared__ float gs_all[];    // [warps][n_groups]: group scores, -inf once a group is kept... then 1 / 0 flags
  pdl_wait_block();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * n_all;
  float* gs = gs_all + (size_t)warp * (n_groups > 0 ? n_groups : 1);
  const int per = n_groups > 1 ? n_all / n_groups : n_all;
  if (n_groups > 1) {
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;   // the two largest
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float sc = 1.f / (1.f + expf(-z[e]));
        if (sc > a) { b = a; a = sc; } else if (sc > b) { b = sc; }
      }
      gs[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // pick the `keep` best groups one at a time; a picked group's entry becomes +inf (allowed), at the end the others -inf
    for (int j = 0; j < keep; ++j) {
      float best = -INFINITY;
      int best_g = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (v > best || best_g == 0x7fffffff)) { best = v; best_g = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (og != 0x7fffffff && (best_g == 0x7fffffff || ob > best || (ob == best && og < best_g))) { best = ob; best_g = og; }
      }
      if (lane == 0 && best_g != 0x7fffffff) gs[best_g] = INFINITY;
      __syncwarp();
    }
  }
  unsigned long long taken_lo = 0ull;   // this lane's entries e = lane + 32 * i, bit i set once chosen (n_all <= 2048)
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane, i = 0; e < n_all; e += 32, ++i) {
      if ((taken_lo >> i) & 1ull) continue;
      if (n_groups > 1 && gs[e / per] != INFINITY) continue;
      const float c = 1.f / (1.f + expf(-z[e]));
      if (c > best || best_e == 0x7fffffff) { best = c; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) { best = ob; best_e = oe; }
    }
    if (best_e != 0x7fffffff && (best_e & 31) == lane) taken_lo |= 1ull << (best_e >> 5);
    if (lane == 0) {
      const bool any = best_e != 0x7fffffff;
      chosen[(size_t)t * top + j] = any ? best_e : -1;
      weight[(size_t)t * top + j] = any ? best : 0.f;
      if (dense_rows) dense_rows[(size_t)t * top + j] = (any && best_e < n_real) ? t * n_real + best_e : -1;
    }
  }
}

// One block: counts, offsets, then places.  `offsets` has n_real + 1 entries.
__global__ void moe_group_kernel(const int* chosen, int n_pairs, int top, int n_real, int* __restrict__ offsets,
                                 int* __restrict__ row_token, int* __restrict__ pair_row) {
  extern __shared__ int cnt[];   // n_real counters, then n_real + 1 offsets
  int* off = cnt + n_real;
  pdl_wait_block();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < n_real; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < n_real) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < n_real; ++e) {
      off[e] = run;
      offsets[e] = run;
      run += cnt[e];
      cnt[e] = 0;
    }
    off[n_real] = run;
    offsets[n_real] = run;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < n_real) {
      const int r = off[e] + atomicAdd(&cnt[e], 1);
      row_token[r] = p / top;
      pair_row[p] = r;
    } else {
      pair_row[p] = -1;
    }
  }
}

// The product with a weight matrix per row group.  A block takes up to ROWS rows of one expert and COLS outputs;
// a warp takes an output at a time, its lanes split k (16-byte weight loads when k allows).  x rows sit in shared
// memory as float32.  GLU != 0: W is [gate rows | up rows] (n_out of each) and out = act(gate, up):
//   1: silu(g) u    2: relu(g) u    3: g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)
constexpr int kMoeRows = 8;
constexpr int kMoeCols = 32;

__device__ __forceinline__ float glu_value(int kind, float g, float u, float limit, float alpha) {
  if (kind == 1) return g / (1.f + expf(-g)) * u;
  if (kind == 2) return fmaxf(g, 0.f) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

template <typename T> struct WVec;
template <> struct WVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
};
template <> struct WVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(h[e]);
      f[2 * e] = v.x; f[2 * e + 1] = v.y;
    }
  }
};

template <typename T, typename TOut>
__global__ void __launch_bounds__(256) moe_rows_gemm_kernel(const T* x, long long x_ld, const int* row_map, const int* offsets,
                                                            int n_groups, const T* __restrict__ w, long long w_group_stride,
                                                            TOut* __restrict__ out, long long out_ld, int n_out, int k_dim,
                                                            int glu, float limit, float alpha, int vec_ok) {
  extern __shared__ float xs[];   // [kMoeRows][k_dim]
  __shared__ int tile_info[3];    // group, first row, rows
  pdl_wait_block();
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    int left = blockIdx.x, g = 0, found = -1, first = 0, rows = 0;
    for (; g < n_groups; ++g) {
      const int cnt = offsets[g + 1] - offsets[g];
      const int tiles = (cnt + kMoeRows - 1) / kMoeRows;
      if (left < tiles) {
        found = g;
        first = offsets[g] + left * kMoeRows;
        rows = min(kMoeRows, offsets[g + 1] - first);
        break;
      }
      left -= tiles;
    }
    tile_info[0] = found; tile_info[1] = first; tile_info[2] = rows;
  }
  __syncthreads();
  const int group = tile_info[0], first = tile_info[1], rows = tile_info[2];
  if (group < 0) return;
  for (int i = threadIdx.x; i < kMoeRows * k_dim; i += blockDim.x) {
    const int r = i / k_dim, c = i - r * k_dim;
    float v = 0.f;
    if (r < rows) {
      const int src = row_map ? row_map[first + r] : first + r;
      v = to_f32<T>(x[(size_t)src * x_ld + c]);
    }
    xs[i] = v;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const T* wg = w + (size_t)group * w_group_stride;
  const int col_end = min(n_out, (int)(blockIdx.y + 1) * kMoeCols);
  for (int n = blockIdx.y * kMoeCols + warp; n < col_end; n += n_warps) {
    float acc[kMoeRows], acc2[kMoeRows];
#pragma unroll
    for (int r = 0; r < kMoeRows; ++r) acc[r] = acc2[r] = 0.f;
    const T* w_row = wg + (size_t)n * k_dim;
    const T* w_row2 = wg + ((size_t)n_out + n) * k_dim;
    if (vec_ok) {
      constexpr int V = WVec<T>::N;
      for (int c = lane * V; c < k_dim; c += 32 * V) {
        float wv[V], wv2[V];
        WVec<T>::load(w_row + c, wv);
        if (glu) WVec<T>::load(w_row2 + c, wv2);
#pragma unroll
        for (int r = 0; r < kMoeRows; ++r) {
          const float* xr = xs + (size_t)r * k_dim + c;
#pragma unroll
          for (int e = 0; e < V; ++e) {
            acc[r] = fmaf(wv[e], xr[e], acc[r]);
            if (glu) acc2[r] = fmaf(wv2[e], xr[e], acc2[r]);
          }
        }
      }
    } else {
      for (int c = lane; c < k_dim; c += 32) {
        const float wv = to_f32<T>(w_row[c]);
        const float wv2 = glu ? to_f32<T>(w_row2[c]) : 0.f;
#pragma unroll
        for (int r = 0; r < kMoeRows; ++r) {
          acc[r] = fmaf(wv, xs[(size_t)r * k_dim + c], acc[r]);
          if (glu) acc2[r] = fmaf(wv2, xs[(size_t)r * k_dim + c], acc2[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kMoeRows; ++r) {
      acc[r] = warp_sum(acc[r]);
      if (glu) acc2[r] = warp_sum(acc2[r]);
    }
    if (lane == 0) {
      for (int r = 0; r < rows; ++r) {
        float y = acc[r];
        if (glu) {
          // the two products are rounded as a kernel that writes them would round them
          const float g = to_f32<T>(from_f32<T>(acc[r])), u = to_f32<T>(from_f32<T>(acc2[r]));
          y = glu_value(glu, g, u, limit, alpha);
        }
        out[(size_t)(first + r) * out_ld + n] = from_f32<TOut>(y);
      }
    }
  }
}

// xs[r] = x[row_token[r]] for the rows that some expert owns (r < offsets[n_groups]): the grouped rows laid out for a
// library product over row groups.
template <typename T>
__global__ void moe_gather_kernel(const T* x, const int* row_token, const int* offsets, int n_groups, T* __restrict__ xs,
                                  int max_rows, int width) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  if (r >= max_rows || r >= offsets[n_groups]) return;
  const T* src = x + (size_t)row_token[r] * width;
  T* dst = xs + (size_t)r * width;
  if (sizeof(T) == 2 && width % 8 == 0) {
    for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8)
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
  }
}

// y[t][c] = sum_j weight[t][j] * (rows[pair_row[t][j]][c] or x[t][c]) (+ shared[t][c])
template <typename T>
__global__ void moe_combine_kernel(const T* rows, const T* x, const T* shared, const int* pair_row, const float* weight,
                                   int top, T* __restrict__ out, int n_tokens, int width) {
  constexpr int kKeep = 32;            // a token's rows and weights, read once (more choices than this: the rest from global memory)
  __shared__ int s_row[kKeep];
  __shared__ float s_w[kKeep];
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  if (threadIdx.x < top && threadIdx.x < kKeep) {
    s_row[threadIdx.x] = pair_row[(size_t)t * top + threadIdx.x];
    s_w[threadIdx.x] = weight[(size_t)t * top + threadIdx.x];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const int r = j < kKeep ? s_row[j] : pair_row[(size_t)t * top + j];
      const float wj = j < kKeep ? s_w[j] : weight[(size_t)t * top + j];
      const float v = r >= 0 ? to_f32<T>(rows[(size_t)r * width + c]) : to_f32<T>(x[(size_t)t * width + c]);
      acc = fmaf(wj, v, acc);
    }
    if (shared) acc += to_f32<T>(shared[(size_t)t * width + c]);
    out[(size_t)t * width + c] = from_f32<T>(acc);
  }
}

// The same for bfloat16 rows whose width is a multiple of 8 and that start on 16-byte boundaries: a thread takes eight
// channels of a token, 16-byte loads and stores (a token's rows and weights are read once per eight channels).
__global__ void moe_combine_vec8_kernel(const __nv_bfloat16* rows, const __nv_bfloat16* x, const __nv_bfloat16* shared,
                                        const int* pair_row, const float* weight, int top, __nv_bfloat16* __restrict__ out,
                                        int n_tokens, int width) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int per_row = width / 8;
  const size_t total = (size_t)n_tokens * per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / per_row), c = (int)(idx - (size_t)t * per_row) * 8;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    auto add = [&](const __nv_bfloat16* p, float w) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
        acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
      }
    };
    for (int j = 0; j < top; ++j) {
      const int r = pair_row[(size_t)t * top + j];
      add(r >= 0 ? rows + (size_t)r * width + c : x + (size_t)t * width + c, weight[(size_t)t * top + j]);
    }
    if (shared) add(shared + (size_t)t * width + c, 1.f);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)t * width + c) = o;
  }
}

// act(gate, up) over the two halves of a row of a [gate | up] product (kinds as above)
template <typename T>
__global__ void glu_act_kernel(const T* gate_up, T* __restrict__ out, int n_rows, int inter, int kind, float limit, float alpha) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t total = (size_t)n_rows * inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / inter, c = i - r * inter;
    const float g = to_f32<T>(gate_up[r * 2 * inter + c]);
    const float u = to_f32<T>(gate_up[r * 2 * inter + inter + c]);
    out[i] = from_f32<T>(glu_value(kind, g, u, limit, alpha));
  }
}

}  // namespace pe

extern "C" int pe_moe_route(const float* logits, const float* correction, int n_tokens, int n_all, int top, int* chosen,
                            float* weight, int* dense_rows, int n_real, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (n_all <= 0 || top <= 0 || top > n_all) return PE_ERR_BAD_ARGUMENT;
  if (n_all > 2048) return PE_ERR_UNSUPPORTED_SIZE;
  const int warps = 4;
  pe::launch(pe::moe_route_kernel, (n_tokens + warps - 1) / warps, warps * 32, 0, stream, logits, correction, n_tokens, n_all,
             top, chosen, weight, dense_rows, n_real);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_moe_route_logits(const float* logits, const float* bias, int n_tokens, int n_all, int top, int* chosen,
                                   float* weight, int* dense_rows, int n_real, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (n_all <= 0 || top <= 0 || top > n_all) return PE_ERR_BAD_ARGUMENT;
  if (n_all > 2048) return PE_ERR_UNSUPPORTED_SIZE;
  const int warps = 4;
  pe::launch(pe::moe_route_logits_kernel, (n_tokens + warps - 1) / warps, warps * 32, 0, stream, logits, bias, n_tokens, n_all,
             top, chosen, weight, dense_rows, n_real);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_moe_route_sigmoid_groups(const float* logits, int n_tokens, int n_all, int top, int n_groups, int keep,
                                           int* chosen, float* weight, int* dense_rows, int n_real, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (n_all <= 0 || top <= 0 || top > n_all) return PE_ERR_BAD_ARGUMENT;
  if (n_groups > 1 && (n_all % n_groups || keep <= 0 || keep > n_groups || top > keep * (n_all / n_groups))) return PE_ERR_BAD_ARGUMENT;
  if (n_all > 2048) return PE_ERR_UNSUPPORTED_SIZE;
  const int warps = 4;
  const size_t smem = (size_t)warps * (n_groups > 0 ? n_groups : 1) * sizeof(float);
  pe::launch(pe::moe_route_sigmoid_groups_kernel, (n_tokens + warps - 1) / warps, warps * 32, smem, stream, logits, n_tokens, n_all,
             top, n_groups, keep, chosen, weight, dense_rows, n_real);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_moe_group(const int* chosen, int n_tokens, int top, int n_real, int* offsets, int* row_token, int* pair_row,
                            cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (top <= 0 || n_real < 0 || n_real > 4096) return PE_ERR_BAD_ARGUMENT;
  const int n_pairs = n_tokens * top;
  const int threads = n_pairs >= 1024 ? 1024 : (n_pairs + 31) / 32 * 32;
  pe::launch(pe::moe_group_kernel, 1, threads, (size_t)(2 * n_real + 1) * sizeof(int), stream, chosen, n_pairs, top, n_real,
             offsets, row_token, pair_row);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_moe_rows_gemm(int dtype, int out_dtype, const void* x, long long x_ld, const int* row_map, const int* offsets,
                                int n_groups, int max_rows, const void* w, long long w_group_stride, void* out, long long out_ld,
                                int n_out, int k_dim, int glu, float limit, float alpha, cudaStream_t stream) {
  if (max_rows <= 0 || n_groups <= 0) return PE_OK;
  if (n_out <= 0 || k_dim <= 0 || glu < 0 || glu > 3) return PE_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)pe::kMoeRows * k_dim * sizeof(float);
  if (smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  const int elem = dtype == PE_F32 ? 4 : 2;
  const int vec = 16 / elem;
  const int vec_ok = (k_dim % vec == 0) && (((uintptr_t)w) % 16 == 0) && ((w_group_stride * elem) % 16 == 0);
  // every group may leave one tile partly filled
  const int tiles = (max_rows + pe::kMoeRows - 1) / pe::kMoeRows + n_groups;
  const dim3 grid(tiles, (n_out + pe::kMoeCols - 1) / pe::kMoeCols);
#define PE_MOE_LAUNCH(T, TOut)                                                                                          \
  do {                                                                                                                  \
    auto kernel = pe::moe_rows_gemm_kernel<T, TOut>;                                                                     \
    if (smem > 48 * 1024) {                                                                                             \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
      if (e != cudaSuccess) return (int)e;                                                                              \
    }                                                                                                                   \
    pe::launch(kernel, grid, dim3(256), smem, stream, (const T*)x, x_ld, row_map, offsets, n_groups, (const T*)w,       \
               w_group_stride, (TOut*)out, out_ld, n_out, k_dim, glu, limit, alpha, vec_ok);                            \
  } while (0)
  if (dtype == PE_F32 && out_dtype == PE_F32) PE_MOE_LAUNCH(float, float);
  else if (dtype == PE_BF16 && out_dtype == PE_BF16) PE_MOE_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == PE_BF16 && out_dtype == PE_F32) PE_MOE_LAUNCH(__nv_bfloat16, float);
  else return PE_ERR_UNSUPPORTED_DTYPE;
#undef PE_MOE_LAUNCH
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_moe_gather_rows(int dtype, const void* x, const int* row_token, const int* offsets, int n_groups, void* xs,
                                  int max_rows, int width, cudaStream_t stream) {
  if (max_rows <= 0) return PE_OK;
  if (width <= 0 || n_groups <= 0) return PE_ERR_BAD_ARGUMENT;
  if (((uintptr_t)x % 16) || ((uintptr_t)xs % 16)) return PE_ERR_BAD_ARGUMENT;
  const int threads = width >= 2048 ? 256 : 128;
  if (dtype == PE_F32)
    pe::launch(pe::moe_gather_kernel<float>, max_rows, threads, 0, stream, (const float*)x, row_token, offsets, n_groups, (float*)xs,
               max_rows, width);
  else if (dtype == PE_BF16)
    pe::launch(pe::moe_gather_kernel<__nv_bfloat16>, max_rows, threads, 0, stream, (const __nv_bfloat16*)x, row_token, offsets,
               n_groups, (__nv_bfloat16*)xs, max_rows, width);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_moe_combine(int dtype, const void* rows, const void* x, const void* shared, const int* pair_row,
                              const float* weight, int top, void* out, int n_tokens, int width, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (top <= 0 || width <= 0) return PE_ERR_BAD_ARGUMENT;
  const int threads = width >= 1024 ? 256 : 128;
  const bool vec8 = dtype == PE_BF16 && width % 8 == 0 && (uintptr_t)rows % 16 == 0 && (uintptr_t)x % 16 == 0 &&
                    (uintptr_t)shared % 16 == 0 && (uintptr_t)out % 16 == 0;
  if (vec8) {
    const size_t total = (size_t)n_tokens * (width / 8);
    size_t blocks = (total + 127) / 128;
    if (blocks > (size_t)pe::kSMs * 32) blocks = (size_t)pe::kSMs * 32;
    pe::launch(pe::moe_combine_vec8_kernel, (int)blocks, 128, 0, stream, (const __nv_bfloat16*)rows, (const __nv_bfloat16*)x,
               (const __nv_bfloat16*)shared, pair_row, weight, top, (__nv_bfloat16*)out, n_tokens, width);
  } else if (dtype == PE_F32)
    pe::launch(pe::moe_combine_kernel<float>, n_tokens, threads, 0, stream, (const float*)rows, (const float*)x, (const float*)shared,
               pair_row, weight, top, (float*)out, n_tokens, width);
  else if (dtype == PE_BF16)
    pe::launch(pe::moe_combine_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)rows,
               (const __nv_bfloat16*)x, (const __nv_bfloat16*)shared, pair_row, weight, top, (__nv_bfloat16*)out, n_tokens, width);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_glu_act(int dtype, const void* gate_up, void* out, int n_rows, int inter, int kind, float limit, float alpha,
                          cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (inter <= 0 || kind < 1 || kind > 3) return PE_ERR_BAD_ARGUMENT;
  const size_t total = (size_t)n_rows * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > pe::kSMs * 16) blocks = pe::kSMs * 16;
  if (dtype == PE_F32)
    pe::launch(pe::glu_act_kernel<float>, (int)blocks, threads, 0, stream, (const float*)gate_up, (float*)out, n_rows, inter, kind, limit, alpha);
  else if (dtype == PE_BF16)
    pe::launch(pe::glu_act_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out,
               n_rows, inter, kind, limit, alpha);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
