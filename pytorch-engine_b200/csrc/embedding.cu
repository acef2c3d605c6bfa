// Token embedding: residual stream (float32) <- table[ids].
// Reference formula: pygguf_engine/quant_kernels.py:1846-1847 (row gather, cast to float32).
#include "api.h"
#include "common.cuh"

namespace pe {

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* ids,
                                    float* __restrict__ out, int n_tokens, int hidden, int vocab, int* status, float scale,
                                    float* __restrict__ copy) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  if (row >= n_tokens) return;
  int id = ids[row];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) report(status, kStatusTokenOutOfRange, row, id, vocab);
    // the row is still defined: zeros
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      out[(size_t)row * hidden + c] = 0.f;
      if (copy) copy[(size_t)row * hidden + c] = 0.f;
    }
    return;
  }
  const T* src = table + (size_t)id * hidden;
  float* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = to_f32<T>(src[c]) * scale;
    dst[c] = v;
    if (copy) copy[(size_t)row * hidden + c] = v;
  }
}

// Token embedding plus an embedding of the pair (previous token, token):
//   out[t] = table[tok[t]] + pairs[(tok[t-1] * mul_prev + tok[t] * mul_cur) mod buckets],   row `buckets` at position 0.
// The token before a step's first one is kept per sequence (`last[slot]`); the block of a sequence's first token
// of the step reads it and then stores the step's last token there.
template <typename T>
__global__ void embed_pair_kernel(const T* __restrict__ table, const T* __restrict__ pairs, const int* ids, const int* token_seq,
                                  const int* token_pos, const int* seq_slot, const int* seq_qstart, int* last,
                                  float* __restrict__ out, int n_tokens, int hidden, int vocab, int buckets, int mul_prev,
                                  int mul_cur, int n_slots, int* status) {
  __shared__ int prev_s;
  pdl_wait_block();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  if (row >= n_tokens) return;
  const int id = ids[row];
  const int b = token_seq[row];
  const int first = seq_qstart[b];
  const int slot = seq_slot[b];
  if (threadIdx.x == 0) {
    int prev = 0;
    if (row > first) {
      prev = ids[row - 1];
    } else if (slot >= 0 && slot < n_slots) {
      prev = last[slot];
      last[slot] = ids[seq_qstart[b + 1] - 1];
    } else {
      report(status, kStatusSlotOutOfRange, row, slot, n_slots);
    }
    prev_s = prev;
  }
  __syncthreads();
  const int prev = prev_s;
  float* dst = out + (size_t)row * hidden;
  if (id < 0 || id >= vocab || prev < 0 || prev >= vocab) {
    if (threadIdx.x == 0) report(status, kStatusTokenOutOfRange, row, id, vocab);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = 0.f;
    return;
  }
  const long long pair = token_pos[row] == 0 ? (long long)buckets
                                             : ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
  const T* src = table + (size_t)id * hidden;
  const T* src2 = pairs + (size_t)pair * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32<T>(src[c]) + to_f32<T>(src2[c]);
}

}  // namespace pe

extern "C" int pe_embed_gather(int dtype, const void* table, const int* ids, float* out, int n_tokens, int hidden,
                               int vocab, int* status, cudaStream_t stream) {
  return pe_embed_gather_scaled(dtype, table, ids, out, n_tokens, hidden, vocab, 1.f, nullptr, status, stream);
}

// The same with a factor on every row, and optionally a second copy of the rows (what a later part reads again after the
// first has become the residual stream).
extern "C" int pe_embed_gather_scaled(int dtype, const void* table, const int* ids, float* out, int n_tokens, int hidden,
                                      int vocab, float scale, float* copy, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (hidden <= 0 || vocab <= 0) return PE_ERR_BAD_ARGUMENT;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == PE_F32)
    pe::launch(pe::embed_gather_kernel<float>, n_tokens, threads, 0, stream, (const float*)table, ids, out, n_tokens, hidden, vocab, status, scale, copy);
  else if (dtype == PE_BF16)
    pe::launch(pe::embed_gather_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, n_tokens, hidden, vocab, status, scale, copy);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_embed_pair_gather(int dtype, const void* table, const void* pairs, const int* ids, const int* token_seq,
                                    const int* token_pos, const int* seq_slot, const int* seq_qstart, int* last, float* out,
                                    int n_tokens, int hidden, int vocab, int buckets, int mul_prev, int mul_cur, int n_slots,
                                    int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (hidden <= 0 || vocab <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0) return PE_ERR_BAD_ARGUMENT;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == PE_F32)
    pe::launch(pe::embed_pair_kernel<float>, n_tokens, threads, 0, stream, (const float*)table, (const float*)pairs, ids, token_seq,
               token_pos, seq_slot, seq_qstart, last, out, n_tokens, hidden, vocab, buckets, mul_prev, mul_cur, n_slots, status);
  else if (dtype == PE_BF16)
    pe::launch(pe::embed_pair_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)table,
               (const __nv_bfloat16*)pairs, ids, token_seq, token_pos, seq_slot, seq_qstart, last, out, n_tokens, hidden, vocab,
               buckets, mul_prev, mul_cur, n_slots, status);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
