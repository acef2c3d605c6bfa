// Dynamic Tanh, a norm without statistics:  y = tanh(alpha * x) * w + b  (alpha one number, w and b per feature), in
// float32 arithmetic; and the two things a block with a norm on either side of each sublayer does around it.
//
//   pe_dyt        out = dyt(x)                                     the norm in front of a sublayer (optionally of gathered rows)
//   pe_dyt_add    stream += dyt_1(delta) ;  out = dyt_2(stream)    the norm behind a sublayer, its add, and (optionally) the
//                                                                  norm in front of the next sublayer, in one pass
//   pe_rmsnorm_pair_mix   out = sa * unit(a) * wa + sb * unit(b) * wb   two outputs side by side, each divided by its own
//                                                                  root mean square over the row
//   pe_concat_split       rows [a | b] of two float32 matrices in the run dtype, as two terms whose sum has 16 significant bits
#include "api.h"
#include "common.cuh"

namespace pe {

// four consecutive elements at once (the pointer is aligned to four elements)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a);
  raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float4 dyt4(float4 x, float alpha, float4 w, float4 b) {
  return make_float4(fmaf(tanhf(alpha * x.x), w.x, b.x), fmaf(tanhf(alpha * x.y), w.y, b.y), fmaf(tanhf(alpha * x.z), w.z, b.z),
                     fmaf(tanhf(alpha * x.w), w.w, b.w));
}

// dim % 4 == 0 and every pointer aligned to four elements: a thread takes four features at a time
template <typename TIn, typename TOut>
__global__ void dyt_vec4_kernel(const TIn* x, const int* rows, const float* __restrict__ w, const float* __restrict__ b, float alpha,
                                TOut* __restrict__ out, int n_rows, int dim) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int per_row = dim / 4;
  const size_t total = (size_t)n_rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / per_row), c = (int)(i - (size_t)r * per_row) * 4;
    const size_t src = (rows ? (size_t)rows[r] : (size_t)r) * dim + c;
    store4(out + (size_t)r * dim + c, dyt4(load4(x + src), alpha, load4(w + c), load4(b + c)));
  }
}

template <typename T>
__global__ void dyt_add_vec4_kernel(float* stream, const T* delta, const float* __restrict__ w1, const float* __restrict__ b1,
                                    float alpha1, const float* __restrict__ w2, const float* __restrict__ b2, float alpha2,
                                    T* __restrict__ out, int n_rows, int dim) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int per_row = dim / 4;
  const size_t total = (size_t)n_rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % per_row) * 4;
    const size_t at = i * 4;
    const float4 d = dyt4(load4(delta + at), alpha1, load4(w1 + c), load4(b1 + c));
    float4 v = load4(stream + at);
    v = make_float4(v.x + d.x, v.y + d.y, v.z + d.z, v.w + d.w);
    store4(stream + at, v);
    if (out) store4(out + at, dyt4(v, alpha2, load4(w2 + c), load4(b2 + c)));
  }
}

template <typename TIn, typename TOut>
__global__ void dyt_kernel(const TIn* x, const int* rows, const float* __restrict__ w, const float* __restrict__ b, float alpha,
                           TOut* __restrict__ out, int n_rows, int dim) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t total = (size_t)n_rows * dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / dim), c = (int)(i - (size_t)r * dim);
    const size_t src = rows ? (size_t)rows[r] * dim + c : i;
    out[i] = from_f32<TOut>(fmaf(tanhf(alpha * to_f32<TIn>(x[src])), w[c], b[c]));
  }
}

template <typename T>
__global__ void dyt_add_kernel(float* stream, const T* delta, const float* __restrict__ w1, const float* __restrict__ b1,
                               float alpha1, const float* __restrict__ w2, const float* __restrict__ b2, float alpha2,
                               T* __restrict__ out, int n_rows, int dim) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t total = (size_t)n_rows * dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % dim);
    const float s = stream[i] + fmaf(tanhf(alpha1 * to_f32<T>(delta[i])), w1[c], b1[c]);
    stream[i] = s;
    if (out) out[i] = from_f32<T>(fmaf(tanhf(alpha2 * s), w2[c], b2[c]));
  }
}

// One block per row; a thread keeps up to kMixItems groups of four features of both inputs in registers, so a row is read
// once.  stream == null: out = mix.  stream != null: stream += dyt_1(mix), and out (if given) = dyt_2(stream).
constexpr int kMixItems = 4;

template <typename T>
__global__ void __launch_bounds__(1024) rmsnorm_pair_mix_kernel(const T* a, const T* b, const float* __restrict__ wa,
                                                                const float* __restrict__ wb, float eps, float sa, float sb,
                                                                T* __restrict__ out, int n_rows, int dim, int vec4, float* stream,
                                                                const float* __restrict__ w1, const float* __restrict__ b1,
                                                                float alpha1, const float* __restrict__ w2,
                                                                const float* __restrict__ b2, float alpha2) {
  __shared__ float red[32];
  pdl_wait_block();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const T* ar = a + (size_t)r * dim;
  const T* br = b + (size_t)r * dim;
  float ssa = 0.f, ssb = 0.f;
  float4 xa[kMixItems], xb[kMixItems];
  if (vec4) {
    int it = 0;
    for (int c = threadIdx.x * 4; c < dim; c += blockDim.x * 4, ++it) {
      const float4 x = load4(ar + c), y = load4(br + c);
      if (it < kMixItems) { xa[it] = x; xb[it] = y; }
      ssa += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
      ssb += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
    }
  } else {
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float x = to_f32<T>(ar[c]), y = to_f32<T>(br[c]);
      ssa = fmaf(x, x, ssa);
      ssb = fmaf(y, y, ssb);
    }
  }
  ssa = block_sum(ssa, red);
  ssb = block_sum(ssb, red);
  const float ia = rsqrtf(ssa / (float)dim + eps) * sa, ib = rsqrtf(ssb / (float)dim + eps) * sb;
  float* srow = stream ? stream + (size_t)r * dim : nullptr;
  if (vec4) {
    int it = 0;
    for (int c = threadIdx.x * 4; c < dim; c += blockDim.x * 4, ++it) {
      const float4 x = it < kMixItems ? xa[it] : load4(ar + c), y = it < kMixItems ? xb[it] : load4(br + c);
      const float4 u = load4(wa + c), v = load4(wb + c);
      const float4 m = make_float4(x.x * ia * u.x + y.x * ib * v.x, x.y * ia * u.y + y.y * ib * v.y,
                                   x.z * ia * u.z + y.z * ib * v.z, x.w * ia * u.w + y.w * ib * v.w);
      if (!srow) {
        store4(out + (size_t)r * dim + c, m);
        continue;
      }
      const float4 d = dyt4(m, alpha1, load4(w1 + c), load4(b1 + c));
      float4 sv = load4(srow + c);
      sv = make_float4(sv.x + d.x, sv.y + d.y, sv.z + d.z, sv.w + d.w);
      store4(srow + c, sv);
      if (out) store4(out + (size_t)r * dim + c, dyt4(sv, alpha2, load4(w2 + c), load4(b2 + c)));
    }
    return;
  }
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    const float m = to_f32<T>(ar[c]) * ia * wa[c] + to_f32<T>(br[c]) * ib * wb[c];
    if (!srow) {
      out[(size_t)r * dim + c] = from_f32<T>(m);
      continue;
    }
    const float sv = srow[c] + fmaf(tanhf(alpha1 * m), w1[c], b1[c]);
    srow[c] = sv;
    if (out) out[(size_t)r * dim + c] = from_f32<T>(fmaf(tanhf(alpha2 * sv), w2[c], b2[c]));
  }
}

// rows [a | b] of two float32 matrices side by side, as the run dtype's rounding `hi` and (bfloat16) what that left over `lo`
template <typename T>
__global__ void concat_split_kernel(const float* a, const float* b, T* __restrict__ hi, T* __restrict__ lo, int n_rows, int dim) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t total = (size_t)n_rows * 2 * dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / (2 * dim);
    const int c = (int)(i - r * 2 * dim);
    const float v = c < dim ? a[r * dim + c] : b[r * dim + (c - dim)];
    const T h = from_f32<T>(v);
    hi[i] = h;
    if (lo) lo[i] = from_f32<T>(v - to_f32<T>(h));
  }
}

static int grid_for(size_t total, int threads) {
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > (size_t)kSMs * 16) blocks = (size_t)kSMs * 16;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace pe

// in_f32 != 0: x is float32 (the stream) whatever `dtype`; `dtype` is the type of out (and of x otherwise).
extern "C" int pe_dyt(int dtype, int in_f32, const void* x, const int* rows, const float* w, const float* b, float alpha,
                      void* out, int n_rows, int dim, cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (dim <= 0) return PE_ERR_BAD_ARGUMENT;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  auto al16 = [](const void* p) { return (uintptr_t)p % 16 == 0; };
  if (dim % 4 == 0 && al16(x) && al16(w) && al16(b) && al16(out)) {
    const int threads = 256, grid = pe::grid_for((size_t)n_rows * (dim / 4), threads);
    if (dtype == PE_F32)
      pe::launch(pe::dyt_vec4_kernel<float, float>, grid, threads, 0, stream, (const float*)x, rows, w, b, alpha, (float*)out, n_rows, dim);
    else if (in_f32)
      pe::launch(pe::dyt_vec4_kernel<float, __nv_bfloat16>, grid, threads, 0, stream, (const float*)x, rows, w, b, alpha,
                 (__nv_bfloat16*)out, n_rows, dim);
    else
      pe::launch(pe::dyt_vec4_kernel<__nv_bfloat16, __nv_bfloat16>, grid, threads, 0, stream, (const __nv_bfloat16*)x, rows, w, b,
                 alpha, (__nv_bfloat16*)out, n_rows, dim);
    PE_LAUNCH_CHECK();
    return PE_OK;
  }
  const int threads = 256, grid = pe::grid_for((size_t)n_rows * dim, threads);
  if (dtype == PE_F32)
    pe::launch(pe::dyt_kernel<float, float>, grid, threads, 0, stream, (const float*)x, rows, w, b, alpha, (float*)out, n_rows, dim);
  else if (in_f32)
    pe::launch(pe::dyt_kernel<float, __nv_bfloat16>, grid, threads, 0, stream, (const float*)x, rows, w, b, alpha,
               (__nv_bfloat16*)out, n_rows, dim);
  else
    pe::launch(pe::dyt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, threads, 0, stream, (const __nv_bfloat16*)x, rows, w, b, alpha,
               (__nv_bfloat16*)out, n_rows, dim);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

// out == null: only the add.
extern "C" int pe_dyt_add(int dtype, float* stream_rows, const void* delta, const float* w1, const float* b1, float alpha1,
                          const float* w2, const float* b2, float alpha2, void* out, int n_rows, int dim, cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (dim <= 0 || (out && (!w2 || !b2))) return PE_ERR_BAD_ARGUMENT;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  auto al16 = [](const void* p) { return (uintptr_t)p % 16 == 0; };
  if (dim % 4 == 0 && al16(stream_rows) && al16(delta) && al16(w1) && al16(b1) && al16(w2) && al16(b2) && al16(out)) {
    const int threads = 256, grid = pe::grid_for((size_t)n_rows * (dim / 4), threads);
    if (dtype == PE_F32)
      pe::launch(pe::dyt_add_vec4_kernel<float>, grid, threads, 0, stream, stream_rows, (const float*)delta, w1, b1, alpha1, w2, b2,
                 alpha2, (float*)out, n_rows, dim);
    else
      pe::launch(pe::dyt_add_vec4_kernel<__nv_bfloat16>, grid, threads, 0, stream, stream_rows, (const __nv_bfloat16*)delta, w1, b1,
                 alpha1, w2, b2, alpha2, (__nv_bfloat16*)out, n_rows, dim);
    PE_LAUNCH_CHECK();
    return PE_OK;
  }
  const int threads = 256, grid = pe::grid_for((size_t)n_rows * dim, threads);
  if (dtype == PE_F32)
    pe::launch(pe::dyt_add_kernel<float>, grid, threads, 0, stream, stream_rows, (const float*)delta, w1, b1, alpha1, w2, b2, alpha2,
               (float*)out, n_rows, dim);
  else if (dtype == PE_BF16)
    pe::launch(pe::dyt_add_kernel<__nv_bfloat16>, grid, threads, 0, stream, stream_rows, (const __nv_bfloat16*)delta, w1, b1, alpha1,
               w2, b2, alpha2, (__nv_bfloat16*)out, n_rows, dim);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_rmsnorm_pair_mix(int dtype, const void* a, const void* b, const float* wa, const float* wb, float eps, float sa,
                                   float sb, void* out, int n_rows, int dim, cudaStream_t stream) {
  return pe_rmsnorm_pair_mix_dyt_add(dtype, a, b, wa, wb, eps, sa, sb, nullptr, nullptr, nullptr, 0.f, nullptr, nullptr, 0.f, out,
                                     n_rows, dim, stream);
}

// The mix, then (stream_rows != null) stream += dyt_1(mix) and, with out, out = dyt_2(stream): what a block with two mixers
// side by side does between them and its feed-forward, in one pass over the rows.
extern "C" int pe_rmsnorm_pair_mix_dyt_add(int dtype, const void* a, const void* b, const float* wa, const float* wb, float eps,
                                           float sa, float sb, float* stream_rows, const float* w1, const float* b1, float alpha1,
                                           const float* w2, const float* b2, float alpha2, void* out, int n_rows, int dim,
                                           cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (dim <= 0 || (!stream_rows && !out) || (stream_rows && (!w1 || !b1)) || (stream_rows && out && (!w2 || !b2)))
    return PE_ERR_BAD_ARGUMENT;
  auto al16 = [](const void* p) { return (uintptr_t)p % 16 == 0; };
  const int vec4 = (dim % 4 == 0 && al16(a) && al16(b) && al16(wa) && al16(wb) && al16(out) && al16(stream_rows) && al16(w1) &&
                    al16(b1) && al16(w2) && al16(b2)) ? 1 : 0;
  const int work = vec4 ? dim / 4 : dim;
  const int threads = work > 1024 ? 512 : (work > 512 ? 256 : 128);   // up to four groups of four features a thread
  if (dtype == PE_F32)
    pe::launch(pe::rmsnorm_pair_mix_kernel<float>, n_rows, threads, 0, stream, (const float*)a, (const float*)b, wa, wb, eps, sa, sb,
               (float*)out, n_rows, dim, vec4, stream_rows, w1, b1, alpha1, w2, b2, alpha2);
  else if (dtype == PE_BF16)
    pe::launch(pe::rmsnorm_pair_mix_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, (const __nv_bfloat16*)a,
               (const __nv_bfloat16*)b, wa, wb, eps, sa, sb, (__nv_bfloat16*)out, n_rows, dim, vec4, stream_rows, w1, b1, alpha1, w2,
               b2, alpha2);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}

// hi = [a | b] in the run dtype; lo (may be null) = the part of [a | b] that the rounding to hi left over, rounded likewise.
extern "C" int pe_concat_split(int dtype, const float* a, const float* b, void* hi, void* lo, int n_rows, int dim,
                               cudaStream_t stream) {
  if (n_rows <= 0) return PE_OK;
  if (dim <= 0) return PE_ERR_BAD_ARGUMENT;
  const int threads = 256, grid = pe::grid_for((size_t)n_rows * 2 * dim, threads);
  if (dtype == PE_F32)
    pe::launch(pe::concat_split_kernel<float>, grid, threads, 0, stream, a, b, (float*)hi, (float*)lo, n_rows, dim);
  else if (dtype == PE_BF16)
    pe::launch(pe::concat_split_kernel<__nv_bfloat16>, grid, threads, 0, stream, a, b, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, n_rows, dim);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
