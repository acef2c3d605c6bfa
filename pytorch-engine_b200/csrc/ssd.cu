// The selective state-space recurrence with a scalar decay per head (the "state-space duality" form), and the gated
// norm over equal parts of a row that follows it.
//
//   step   dt = softplus(dt_raw + dt_bias) ;  a = exp(-exp(A) dt)                      per token and head
//          S <- a S + dt B x^T   (S: [n, dv]) ;  y = S^T C + D x                         head h reads group h / (heads / groups)
//   norm   v = y * silu(z) ;  out = v / sqrt(mean_part(v^2) + eps) * w                   each of `parts` equal parts of a row
//
// A block owns one head's S of one sequence and walks the sequence's tokens of this step in order; one, two or four threads
// own a column of S (in registers up to 256 rows, in shared memory beyond).  State, dt, the decay and y are float32 whatever the
// run dtype.  For long prompts the tokens are cut into chunks that run side by side: the update is linear in S with a
// scalar factor, so a chunk is first folded from an empty state (MODE 1, which also leaves the sum of its log decays),
// a small kernel chains the chunks' true start states  S_start[c+1] = exp(sum_c) S_start[c] + S_chunk[c],  and the
// chunks then run from those and write their outputs (MODE 3).
#include "api.h"
#include "common.cuh"

namespace pe {

struct SsdArgs {
  const void* xbc; long long xbc_ld;   // [n_tokens, *]: x (heads * dv) | B (groups * n) | C (groups * n), after the convolution
  const void* dt; long long dt_ld;     // [n_tokens, *]: heads columns, before the bias and the softplus (run dtype)
  const float* dt_bias; const float* A_log; const float* D;   // [heads] each
  float* y;                            // [n_tokens, heads * dv] float32
  float* S;                            // [slots, heads, n, dv]
  const int* seq_slot; const int* seq_qstart;
  int n_seqs, heads, groups, n, dv, n_slots;
  int chunk, max_chunks;               // tokens per chunk (0: the whole step in one go)
  float* scratch;                      // [n_seqs, heads, max_chunks, n * dv] then [n_seqs, heads, max_chunks] log decays
  int* status;
};

constexpr int kSsdBatch = 32;

// A staged B or C row with SPLIT threads a column: part p's rows [p * NP, (p + 1) * NP) start 4 floats further on for every
// part before them, so the four parts' 16-byte reads of one step (one address a quarter-warp) fall into different banks.
__host__ __device__ inline int ssd_row_floats(int np, int split) { return split == 1 ? np : split * (np + 4); }

// dst[r][col(c)] = float(src[r][c]) with col(c) = c + 4 * (c / np) (np == 0: col(c) = c)
template <typename T>
__device__ __forceinline__ void ssd_stage_rows(float* dst, int dst_ld, int np, const T* src, long long src_ld, int n_rows, int width,
                                               bool vec) {
  if (vec) {
    constexpr int N = StageVec<T>::N;
    const int per_row = width / N;
    for (int e = threadIdx.x; e < n_rows * per_row; e += blockDim.x) {
      const int r = e / per_row, c = (e - r * per_row) * N;
      const uint4 raw = *reinterpret_cast<const uint4*>(src + (size_t)r * src_ld + c);
      float* o = dst + (size_t)r * dst_ld + (np > 0 ? c + 4 * (c / np) : c);
      if (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(o) = *reinterpret_cast<const float4*>(&raw);
      } else {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c2 = __bfloat1622float2(h[2]), d2 = __bfloat1622float2(h[3]);
        *reinterpret_cast<float4*>(o) = make_float4(a.x, a.y, b.x, b.y);
        *reinterpret_cast<float4*>(o + 4) = make_float4(c2.x, c2.y, d2.x, d2.y);
      }
    }
  } else {
    for (int e = threadIdx.x; e < n_rows * width; e += blockDim.x) {
      const int r = e / width, c = e - r * width;
      dst[(size_t)r * dst_ld + (np > 0 ? c + 4 * (c / np) : c)] = to_f32<T>(src[(size_t)r * src_ld + c]);
    }
  }
}

// MODE 0: the whole step from the slot's state; MODE 1: chunk blockIdx.z from an empty state, no outputs; MODE 3: chunk
// blockIdx.z from its true start, outputs, and the sequence's last chunk writes the state back.
// NR > 0: a thread keeps NR rows of its column in registers and SPLIT threads share a column (lanes l, l ^ 16 for two,
// l, l ^ 8, l ^ 16, l ^ 24 for four: a quarter of a warp reads one address of the staged B and C rows, and the partial
// outputs meet in shuffles); more threads a column hide the walk's latencies and fill the state's loads.  NR == 0: the state
// lives in shared memory, one thread a column.
template <typename T, int MODE, int NR, int SPLIT>
__global__ void __launch_bounds__(NR == 0 ? 1024 : 512) ssd_kernel(SsdArgs a) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float s_dt[kSsdBatch], s_a[kSsdBatch], s_log[kSsdBatch];
  const int n = a.n, dv = a.dv, head = blockIdx.x, b = blockIdx.y, c = blockIdx.z;
  const int g = head / (a.heads / a.groups);
  constexpr int NP = NR > 0 ? NR : 1;
  const int npad = NR > 0 ? NR * SPLIT : n;                    // rows with the padding up to what the threads hold
  const int ldb = NR > 0 ? ssd_row_floats(NR, SPLIT) : n;      // floats of a staged B or C row
  const int part_np = (NR > 0 && SPLIT > 1) ? NR : 0;          // rows a part (0: the row is not cut into parts)
  float* Ssm = sm;                                             // [n][dv] (NR == 0 only)
  float* Bb = Ssm + (NR > 0 ? 0 : (size_t)n * dv);             // [batch][ldb]
  float* Cb = Bb + (size_t)kSsdBatch * ldb;                    // [batch][ldb]
  float* xb = Cb + (size_t)kSsdBatch * ldb;                    // [batch][dv]
  pdl_wait_block();
  pdl_launch_dependents();
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) {
    if (threadIdx.x == 0 && head == 0 && c == 0) report(a.status, kStatusSlotOutOfRange, b, slot, a.n_slots);
    return;
  }
  const int q0 = a.seq_qstart[b], q1 = a.seq_qstart[b + 1];
  int t0 = q0, t1 = q1;
  if (MODE != 0) {
    t0 = q0 + c * a.chunk;
    t1 = min(q1, t0 + a.chunk);
    if (t0 >= q1) return;
    if (MODE == 1 && t1 == q1) return;             // nothing follows the sequence's last chunk
  }
  const size_t unit = (size_t)n * dv;
  const size_t cidx = ((size_t)b * a.heads + head) * a.max_chunks + c;      // a head's chunks lie side by side
  float* cs = MODE != 0 ? a.scratch + cidx * unit : nullptr;
  float* gS = a.S + ((size_t)slot * a.heads + head) * unit;
  const float* src = MODE == 0 ? gS : cs;
  const int lane = threadIdx.x & 31;
  // the thread's column and the first of its rows
  const int j = SPLIT == 1 ? (int)threadIdx.x : (int)(threadIdx.x >> 5) * (32 / SPLIT) + (lane & (32 / SPLIT - 1));
  const int part = SPLIT == 1 ? 0 : lane / (32 / SPLIT);
  const int i0 = part * NP;
  const int s0 = SPLIT == 1 ? 0 : part * (NP + 4);             // where the part's rows start in a staged row
  float Sr[NP];
  if (NR > 0) {
#pragma unroll
    for (int i = 0; i < NP; ++i) Sr[i] = (MODE != 1 && i0 + i < n && j < dv) ? src[(size_t)(i0 + i) * dv + j] : 0.f;
  } else {
    for (int i = threadIdx.x; i < n * dv; i += blockDim.x) Ssm[i] = MODE == 1 ? 0.f : src[i];
  }
  if (npad > n)
    for (int e = threadIdx.x; e < kSsdBatch * (npad - n); e += blockDim.x) {
      const int tt = e / (npad - n), i = n + e % (npad - n);
      const int at = part_np > 0 ? i + 4 * (i / part_np) : i;
      Bb[(size_t)tt * ldb + at] = 0.f;
      Cb[(size_t)tt * ldb + at] = 0.f;
    }
  const T* x = (const T*)a.xbc;
  const int b_col = a.heads * dv + g * n, c_col = a.heads * dv + a.groups * n + g * n, x_col = head * dv;
  const float rate = expf(a.A_log[head]), bias = a.dt_bias[head], Dh = a.D[head];
  const bool sm_ok = NR > 0 || (n * dv) % 4 == 0;   // the staged rows start on 16-byte boundaries
  const bool vec_b = sm_ok && ldb % 4 == 0 && stage_vec_ok<T>(x + (size_t)t0 * a.xbc_ld + b_col, a.xbc_ld, n);
  const bool vec_c = sm_ok && ldb % 4 == 0 && stage_vec_ok<T>(x + (size_t)t0 * a.xbc_ld + c_col, a.xbc_ld, n);
  const bool vec_x = sm_ok && dv % 4 == 0 && stage_vec_ok<T>(x + (size_t)t0 * a.xbc_ld + x_col, a.xbc_ld, dv);
  float log_sum = 0.f;
  for (int tb = t0; tb < t1; tb += kSsdBatch) {
    const int nb = min(kSsdBatch, t1 - tb);
    __syncthreads();                               // the batch before this one has been read
    ssd_stage_rows<T>(Bb, ldb, part_np, x + (size_t)tb * a.xbc_ld + b_col, a.xbc_ld, nb, n, vec_b);
    if (MODE != 1) ssd_stage_rows<T>(Cb, ldb, part_np, x + (size_t)tb * a.xbc_ld + c_col, a.xbc_ld, nb, n, vec_c);
    stage_rows_f32<T>(xb, dv, x + (size_t)tb * a.xbc_ld + x_col, a.xbc_ld, nb, dv, 1.f, vec_x);
    if (threadIdx.x < nb) {
      const float z = to_f32<T>(((const T*)a.dt)[(size_t)(tb + threadIdx.x) * a.dt_ld + head]) + bias;
      const float dt = z > 20.f ? z : log1pf(expf(z));
      s_dt[threadIdx.x] = dt;
      s_log[threadIdx.x] = -rate * dt;
      s_a[threadIdx.x] = expf(-rate * dt);
    }
    __syncthreads();
    if (MODE == 1)
      for (int tt = 0; tt < nb; ++tt) log_sum += s_log[tt];
    if (NR > 0) {
      // whole warps walk together (the parts of a column meet in shuffles); a column beyond the matrix carries zeros
      for (int tt = 0; tt < nb; ++tt) {
        const float decay = s_a[tt];
        const float xj = j < dv ? xb[(size_t)tt * dv + j] : 0.f;
        const float dx = s_dt[tt] * xj;
        const float* Bs = Bb + (size_t)tt * ldb + s0;
        const float* Cs = Cb + (size_t)tt * ldb + s0;
        float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
        for (int i = 0; i < NP; i += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(Bs + i);
          Sr[i] = fmaf(decay, Sr[i], dx * b4.x);
          Sr[i + 1] = fmaf(decay, Sr[i + 1], dx * b4.y);
          Sr[i + 2] = fmaf(decay, Sr[i + 2], dx * b4.z);
          Sr[i + 3] = fmaf(decay, Sr[i + 3], dx * b4.w);
          if (MODE != 1) {
            const float4 c4 = *reinterpret_cast<const float4*>(Cs + i);
            y0 = fmaf(Sr[i], c4.x, y0);
            y1 = fmaf(Sr[i + 1], c4.y, y1);
            y2 = fmaf(Sr[i + 2], c4.z, y2);
            y3 = fmaf(Sr[i + 3], c4.w, y3);
          }
        }
        if (MODE != 1) {
          float y = (y0 + y1) + (y2 + y3);
          if (SPLIT >= 2) y += __shfl_xor_sync(0xffffffffu, y, 16);
          if (SPLIT == 4) y += __shfl_xor_sync(0xffffffffu, y, 8);
          if (i0 == 0 && j < dv) a.y[(size_t)(tb + tt) * a.heads * dv + head * dv + j] = fmaf(Dh, xj, y);
        }
      }
    } else if (j < dv) {
      for (int tt = 0; tt < nb; ++tt) {
        const float decay = s_a[tt];
        const float xj = xb[(size_t)tt * dv + j];
        const float dx = s_dt[tt] * xj;
        const float* Bs = Bb + (size_t)tt * ldb;
        const float* Cs = Cb + (size_t)tt * ldb;
        float y0 = 0.f;
        for (int i = 0; i < n; ++i) {
          const float s = fmaf(decay, Ssm[(size_t)i * dv + j], dx * Bs[i]);
          Ssm[(size_t)i * dv + j] = s;
          if (MODE != 1) y0 = fmaf(s, Cs[i], y0);
        }
        if (MODE != 1) a.y[(size_t)(tb + tt) * a.heads * dv + head * dv + j] = fmaf(Dh, xj, y0);
      }
    }
  }
  __syncthreads();
  if (MODE == 3 && t1 != q1) return;               // only the sequence's last chunk leaves the state
  float* dst = MODE == 1 ? cs : gS;
  if (NR > 0) {
    if (j < dv) {
#pragma unroll
      for (int i = 0; i < NP; ++i)
        if (i0 + i < n) dst[(size_t)(i0 + i) * dv + j] = Sr[i];
    }
  } else {
    for (int i = threadIdx.x; i < n * dv; i += blockDim.x) dst[i] = Ssm[i];
  }
  if (MODE == 1 && threadIdx.x == 0) a.scratch[(size_t)a.n_seqs * a.max_chunks * a.heads * unit + cidx] = log_sum;
}

// Chain the chunks: on entry scratch[c] holds chunk c's end state from zero and the sum of its log decays (every chunk
// but the sequence's last); on exit it holds chunk c's true start state, chunk 0's being the slot's state.
__global__ void ssd_chain_kernel(SsdArgs a) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int head = blockIdx.x, b = blockIdx.y;
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) return;
  const int q_len = a.seq_qstart[b + 1] - a.seq_qstart[b];
  const int n_chunks = (q_len + a.chunk - 1) / a.chunk;
  const size_t unit = (size_t)a.n * a.dv;
  const size_t first = ((size_t)b * a.heads + head) * a.max_chunks;          // the head's first chunk
  const float* logs = a.scratch + (size_t)a.n_seqs * a.max_chunks * a.heads * unit + first;
  const float* gS = a.S + ((size_t)slot * a.heads + head) * unit;
  // a thread follows one element through the chunks, eight chunks' loads in flight at a time (a chunk's slot is read
  // before it is overwritten with that chunk's true start)
  constexpr int G = 8;
  const size_t e = (size_t)blockIdx.z * blockDim.x + threadIdx.x;
  if (e >= unit) return;
  float* u = a.scratch + first * unit + e;
  float val = gS[e];
  for (int c0 = 0; c0 < n_chunks; c0 += G) {
    float loc[G], lg[G];
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const bool has = c0 + i + 1 < n_chunks;
      loc[i] = has ? u[(size_t)(c0 + i) * unit] : 0.f;
      lg[i] = has ? logs[c0 + i] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < G; ++i) {
      if (c0 + i >= n_chunks) break;
      u[(size_t)(c0 + i) * unit] = val;
      if (c0 + i + 1 < n_chunks) val = fmaf(expf(lg[i]), val, loc[i]);
    }
  }
}

// v = y * silu(z); each of `parts` equal parts of a row is divided by its root mean square and multiplied by w.
// One block per (token, part).
template <typename T>
__global__ void gated_part_norm_kernel(const float* y, const T* z, long long z_ld, const float* __restrict__ w, float eps,
                                       T* __restrict__ out, int n_tokens, int width, int parts) {
  __shared__ float red[32];
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x, p = blockIdx.y;
  const int part = width / parts, c0 = p * part;
  float ss = 0.f;
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    const float zz = to_f32<T>(z[(size_t)t * z_ld + c0 + c]);
    const float v = y[(size_t)t * width + c0 + c] * (zz / (1.f + expf(-zz)));
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)part + eps);
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    const float zz = to_f32<T>(z[(size_t)t * z_ld + c0 + c]);
    const float v = y[(size_t)t * width + c0 + c] * (zz / (1.f + expf(-zz)));
    out[(size_t)t * width + c0 + c] = from_f32<T>(v * inv * w[c0 + c]);
  }
}

template <typename T, int NR, int SPLIT>
static int ssd_run(const SsdArgs& a, cudaStream_t stream) {
  const int n = a.n, dv = a.dv;
  const int ldb = NR > 0 ? ssd_row_floats(NR, SPLIT) : n;
  const size_t smem = ((NR > 0 ? 0 : (size_t)n * dv) + 2 * (size_t)kSsdBatch * ldb + (size_t)kSsdBatch * dv) * sizeof(float);
  if (smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  const int cols_per_warp = 32 / SPLIT;
  int threads = (dv + cols_per_warp - 1) / cols_per_warp * 32;
  if (threads < 32) threads = 32;
  if (threads > (NR == 0 ? 1024 : 512)) return PE_ERR_UNSUPPORTED_SIZE;
  auto k0 = ssd_kernel<T, 0, NR, SPLIT>;
  auto k1 = ssd_kernel<T, 1, NR, SPLIT>;
  auto k3 = ssd_kernel<T, 3, NR, SPLIT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (a.chunk > 0) {
    launch(k1, dim3(a.heads, a.n_seqs, a.max_chunks), dim3(threads), smem, stream, a);
    const size_t unit = (size_t)n * dv;
    const size_t zb = (unit + 255) / 256;
    if (zb > 65535) return PE_ERR_UNSUPPORTED_SIZE;
    launch(ssd_chain_kernel, dim3(a.heads, a.n_seqs, (unsigned)zb), dim3(256), 0, stream, a);
    launch(k3, dim3(a.heads, a.n_seqs, a.max_chunks), dim3(threads), smem, stream, a);
  } else {
    launch(k0, dim3(a.heads, a.n_seqs, 1), dim3(threads), smem, stream, a);
  }
  return PE_OK;
}

// Threads a column and rows a thread for a state of n rows and dv columns: as many threads a column as the rows are worth
// (four from 65 rows on, two from 33) and a block of at most 512 threads allows; 0 rows: the shared-memory form.
static void ssd_shape(int n, int dv, int* rows, int* split) {
  int s = n > 64 ? 4 : (n > 32 ? 2 : 1);
  while (s > 1 && (dv + 32 / s - 1) / (32 / s) * 32 > 512) s /= 2;
  const int per = (n + s - 1) / s;
  int r = per <= 16 ? 16 : (per <= 32 ? 32 : (per <= 64 ? 64 : (per <= 128 ? 128 : 0)));
  if (s == 1 && dv > 512) r = 0;
  if (s == 2 && r == 16) r = 32;
  if (s == 4 && r == 16) r = 32;
  if (s > 1 && r == 128) { r = 0; s = 1; }
  *rows = r; *split = r == 0 ? 1 : s;
}

}  // namespace pe

// Floats of scratch that the chunked form needs for `max_chunks` chunks per sequence.
extern "C" long long pe_ssd_scratch_floats(int n_seqs, int heads, int n, int dv, int max_chunks) {
  return (long long)n_seqs * max_chunks * heads * ((long long)n * dv + 1);
}

// chunk > 0: prompts cut into chunks of that many tokens (scratch from pe_ssd_scratch_floats, max_chunks >=
// ceil(max_q / chunk)); chunk == 0: each sequence's tokens in one go (single tokens, short prompts).
extern "C" int pe_ssd_recurrence(int dtype, const void* xbc, long long xbc_ld, const void* dt, long long dt_ld,
                                 const float* dt_bias, const float* A_log, const float* D, float* y, float* S,
                                 const int* seq_slot, const int* seq_qstart, int n_seqs, int max_q, int heads, int groups,
                                 int n, int dv, int n_slots, int chunk, int max_chunks, float* scratch, int* status,
                                 cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (heads <= 0 || groups <= 0 || heads % groups || n <= 0 || dv <= 0) return PE_ERR_BAD_ARGUMENT;
  if (dv > 1024 || n > 4096) return PE_ERR_UNSUPPORTED_SIZE;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  pe::SsdArgs args{xbc, xbc_ld, dt, dt_ld, dt_bias, A_log, D, y, S, seq_slot, seq_qstart, n_seqs, heads, groups, n, dv,
                   n_slots, 0, 1, nullptr, status};
  if (chunk > 0) {
    if (!scratch || max_chunks <= 0 || (long long)max_chunks * chunk < max_q || max_chunks > 65535) return PE_ERR_BAD_ARGUMENT;
    args.chunk = chunk; args.max_chunks = max_chunks; args.scratch = scratch;
  }
  int rows = 0, split = 1;
  pe::ssd_shape(n, dv, &rows, &split);
  int rc;
#define PE_SSD(T)                                                                                                   \
  (split == 4 ? (rows == 32 ? pe::ssd_run<T, 32, 4>(args, stream) : pe::ssd_run<T, 64, 4>(args, stream))            \
   : split == 2 ? (rows == 32 ? pe::ssd_run<T, 32, 2>(args, stream) : pe::ssd_run<T, 64, 2>(args, stream))          \
   : rows == 16 ? pe::ssd_run<T, 16, 1>(args, stream) : rows == 32 ? pe::ssd_run<T, 32, 1>(args, stream)            \
   : rows == 64 ? pe::ssd_run<T, 64, 1>(args, stream) : rows == 128 ? pe::ssd_run<T, 128, 1>(args, stream)          \
   : pe::ssd_run<T, 0, 1>(args, stream))
  rc = dtype == PE_F32 ? PE_SSD(float) : PE_SSD(__nv_bfloat16);
#undef PE_SSD
  if (rc != PE_OK) return rc;
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_gated_part_norm(int dtype, const float* y, const void* z, long long z_ld, const float* w, float eps,
                                  void* out, int n_tokens, int width, int parts, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (width <= 0 || parts <= 0 || width % parts) return PE_ERR_BAD_ARGUMENT;
  if (parts > 65535) return PE_ERR_UNSUPPORTED_SIZE;
  const int part = width / parts;
  const int threads = part >= 1024 ? 256 : (part >= 256 ? 128 : 64);
  const dim3 grid(n_tokens, parts);
  if (dtype == PE_F32)
    pe::launch(pe::gated_part_norm_kernel<float>, grid, dim3(threads), 0, stream, y, (const float*)z, z_ld, w, eps, (float*)out,
               n_tokens, width, parts);
  else if (dtype == PE_BF16)
    pe::launch(pe::gated_part_norm_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, y, (const __nv_bfloat16*)z, z_ld, w,
               eps, (__nv_bfloat16*)out, n_tokens, width, parts);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
