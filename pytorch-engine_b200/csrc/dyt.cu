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

// One block per row.
template <typename T>
__global__ void rmsnorm_pair_mix_kernel(const T* a, const T* b, const float* __restrict__ wa, const float* __restrict__ wb,
                                        float eps, float sa, float sb, T* __restrict__ out, int n_rows, int dim) {
  __shared__ float red[32];
  pdl_wait_block();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const T* ar = a + (size_t)r * dim;
  const T* br = b + (size_t)r * dim;
  float ssa = 0.f, ssb = 0.f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    const float x = to_f32<T>(ar[c]), y = to_f32<T>(br[c]);
    ssa = fmaf(x, x, ssa);
    ssb = fmaf(y, y, ssb);
  }
  ssa = block_sum(ssa, red);
  ssb = block_sum(ssb, red);
  const float ia = rsqrtf(ssa / (float)dim + eps) * sa, ib = rsqrtf(ssb / (float)dim + eps) * sb;
  for (int c = threadIdx.x; c < dim; c += blockDim.x)
    out[(size_t)r * dim + c] = from_f32<T>(to_f32<T>(ar[c]) * ia * wa[c] + to_f32<T>(br[c]) * ib * wb[c]);
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
  if (n_rows <= 0) return PE_OK;
  if (dim <= 0) return PE_ERR_BAD_ARGUMENT;
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  if (dtype == PE_F32)
    pe::launch(pe::rmsnorm_pair_mix_kernel<float>, n_rows, threads, 0, stream, (const float*)a, (const float*)b, wa, wb, eps, sa, sb,
               (float*)out, n_rows, dim);
  else if (dtype == PE_BF16)
    pe::launch(pe::rmsnorm_pair_mix_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, (const __nv_bfloat16*)a,
               (const __nv_bfloat16*)b, wa, wb, eps, sa, sb, (__nv_bfloat16*)out, n_rows, dim);
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
