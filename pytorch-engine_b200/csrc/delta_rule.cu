// The gated delta rule: a linear recurrence whose matrix state forgets per key channel and is corrected, not just
// added to, by every token; with the short causal convolutions that precede it.
//
//   convolution  y[t][c] = silu(sum_j w[c][j] x[t - taps + 1 + j][c])       inputs before a sequence's start are zero,
//                                                                           before this step's start they come from the state
//   unit vectors q = q / sqrt(sum q^2 + 1e-6) * q_scale ;  k = k / sqrt(sum k^2 + 1e-6)          per head
//   decay        g[i] = exp(-exp(A) softplus(a[i] + dt[i]))                 per head and key channel, or one per head
//   step         S <- diag(g) S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q            beta = sigmoid(b)
//   out          = o / rms(o) * w * sigmoid(gate)  (or * silu(gate))        per head, eps inside the root, w of size dv
//
// A block owns one head's S [d, dv] of one sequence (in registers or in shared memory) and walks the sequence's tokens
// of this step in order; thread j owns column j.  State, decay, beta, the unit vectors and the head norm are float32 whatever
// the run dtype.
#include "api.h"
#include "common.cuh"

namespace pe {

// ---- short convolution + silu -----------------------------------------------------------------------------------
// x: [n_tokens, ld] (channels at columns col0 .. col0 + channels), w: [channels, taps] float32,
// tail: [slots, taps - 1, channels] float32 (the last inputs of every sequence, oldest first).
template <typename T>
__global__ void short_conv_kernel(const T* x, long long ld, int col0, const float* __restrict__ w, const float* __restrict__ bias, int taps,
                                  const float* tail, const int* token_seq, const int* seq_slot, const int* seq_qstart,
                                  T* __restrict__ out, int n_tokens, int channels, int n_slots, int* status) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int b = token_seq[t];
  const int first = seq_qstart[b];
  const int slot = seq_slot[b];
  if (slot < 0 || slot >= n_slots) {
    if (threadIdx.x == 0) report(status, kStatusSlotOutOfRange, t, slot, n_slots);
    return;
  }
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = t - (taps - 1) + j;          // row of the step, if it belongs to this sequence
      float v;
      if (src >= first) v = to_f32<T>(x[(size_t)src * ld + col0 + c]);
      else v = tail[((size_t)slot * (taps - 1) + (taps - 1) - (first - src)) * channels + c];
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[(size_t)t * channels + c] = from_f32<T>(acc / (1.f + expf(-acc)));
  }
}

// The same for bfloat16 rows whose channels are a multiple of 8 and start on 16-byte boundaries: a thread takes eight
// channels of a strip of eight tokens with its 8 x TAPS weights in registers (loaded once per strip: a weight load of
// a warp touches 32 cache lines), 16-byte loads and stores.  A step of few tokens takes strips of one.

template <int TAPS>
__global__ void short_conv_vec8_kernel(const __nv_bfloat16* x, long long ld, int col0, const float* __restrict__ w,
                                       const float* __restrict__ bias, const float* tail, const int* token_seq, const int* seq_slot, const int* seq_qstart,
                                       __nv_bfloat16* __restrict__ out, int n_tokens, int channels, int n_slots, int* status,
                                       int kConvStrip) {
  const int per_row = channels / 8;
  const int strips = (n_tokens + kConvStrip - 1) / kConvStrip;
  const size_t total = (size_t)strips * per_row;
  const size_t idx0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  float wr[8][TAPS], br[8];
  int c_have = -1;
  pdl_wait_block();
  pdl_launch_dependents();
  for (size_t idx = idx0; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int strip = (int)(idx / per_row), c = (int)(idx - (size_t)strip * per_row) * 8;
    if (c != c_have) {
#pragma unroll
      for (int e = 0; e < 8; ++e)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wr[e][j] = w[(size_t)(c + e) * TAPS + j];
#pragma unroll
      for (int e = 0; e < 8; ++e) br[e] = bias ? bias[c + e] : 0.f;
      c_have = c;
    }
    const int t_end = min(n_tokens, (strip + 1) * kConvStrip);
    for (int t = strip * kConvStrip; t < t_end; ++t) {
      const int b = token_seq[t];
      const int first = seq_qstart[b];
      const int slot = seq_slot[b];
      if (slot < 0 || slot >= n_slots) {
        if (c == 0) report(status, kStatusSlotOutOfRange, t, slot, n_slots);
        continue;
      }
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = br[e];
#pragma unroll
      for (int j = 0; j < TAPS; ++j) {
        const int src = t - (TAPS - 1) + j;
        float v[8];
        if (src >= first) {
          const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)src * ld + col0 + c);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            v[2 * e] = f.x; v[2 * e + 1] = f.y;
          }
        } else {
          const float* tp = tail + ((size_t)slot * (TAPS - 1) + (TAPS - 1) - (first - src)) * channels + c;
          const float4 a0 = *reinterpret_cast<const float4*>(tp), a1 = *reinterpret_cast<const float4*>(tp + 4);
          v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w; v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wr[e][j], v[e], acc[e]);
      }
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        o2[e] = __floats2bfloat162_rn(acc[2 * e] / (1.f + expf(-acc[2 * e])), acc[2 * e + 1] / (1.f + expf(-acc[2 * e + 1])));
      *reinterpret_cast<uint4*>(out + (size_t)t * channels + c) = o;
    }
  }
}

// The new tail of every sequence: the last taps - 1 rows of (old tail, this step's inputs).  One thread per
// (sequence, channel) walks the rows oldest first, so a row is read before it is overwritten.
template <typename T>
__global__ void conv_tail_kernel(const T* x, long long ld, int col0, float* tail, int taps, const int* seq_slot,
                                 const int* seq_qstart, int n_seqs, int channels, int n_slots) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int slot = seq_slot[b];
  if (slot < 0 || slot >= n_slots) return;
  const int first = seq_qstart[b], len = seq_qstart[b + 1] - first, keep = taps - 1;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x) {
    float* mine = tail + (size_t)slot * keep * channels + c;
    for (int r = 0; r < keep; ++r) {
      const int at = len + r;                      // index into (old tail, inputs)
      mine[(size_t)r * channels] = at < keep ? mine[(size_t)at * channels]
                                             : to_f32<T>(x[(size_t)(first + at - keep) * ld + col0 + c]);
    }
  }
}

// ---- the recurrence -----------------------------------------------------------------------------------------------
struct DeltaArgs {
  const void* qkv;          // [n_tokens, channels] after the convolution: q (kv_heads * d) | k (kv_heads * d) | v (heads * dv)
  const float* a;           // [n_tokens, heads * d]: the decay projection before its offset ([n_tokens, heads] with head_decay)
  const float* dt_bias;     // [heads * d] ([heads] with head_decay)
  const float* A_log;       // [heads]
  const float* b;           // [n_tokens, heads]: beta before the sigmoid
  const void* gate; long long gate_ld;   // [n_tokens, heads * dv] in the run dtype, before the sigmoid
  const float* norm_w;      // [dv]
  float eps, q_scale;
  void* out;                // [n_tokens, heads * dv]
  float* S;                 // [slots, heads, d, dv]
  const int* seq_slot; const int* seq_qstart;
  int n_seqs, heads, kv_heads, d, dv, n_slots;
  int chunk;                // tokens per chunk (modes 1 and 3), 0: the whole step in one go
  int max_chunks;
  float* scratch;           // [n_seqs, max_chunks, heads, d * dv + d * d]: a chunk's S, then its transition matrix
  int* status;
  int head_decay;           // != 0: one decay per head and token instead of one per key channel
  int gate_silu;            // != 0: the output gate is silu(gate) instead of sigmoid(gate)
  long long a_ld, b_ld;     // floats between two tokens' rows of a and of b
};

__host__ __device__ inline size_t delta_unit(int d, int dv) { return (size_t)d * dv + (size_t)d * d; }

// MODE 0: the whole step: start from the slot's state, write outputs, write the state back.
// MODE 1: chunk c = blockIdx.z % max_chunks from an empty state, no outputs.  A token's step is linear in S,
//         S <- (I - beta k k^T) diag(g) S + beta k v^T, and every column of S goes its own way; so the chunk's end
//         state from zero (blockIdx.z < max_chunks: the columns of S) and the product of its tokens' transition
//         matrices (blockIdx.z >= max_chunks: the same step on the columns of a d x d matrix that starts as the
//         identity and is fed v = 0) are both left for the chain kernel: S_start[c+1] = T_c S_start[c] + S_chunk[c].
// MODE 3: chunk blockIdx.z from its true start (as the chain kernel left it): writes outputs; the sequence's last chunk
//         writes the state back.
// DREG > 0: d <= DREG and thread j keeps its column in registers; DREG == 0: the matrix lives in shared memory.
//
// Tokens are taken `batch` at a time: their q, k, v and gate rows are staged in shared memory with all loads in flight
// at once, the decays, the vectors' lengths and beta are computed side by side; the walk over the batch's tokens then
// reads shared memory only, and where no output is written (MODE 1) it needs no barrier at all.
constexpr int kDeltaBatch = 32;

template <typename T>
__host__ __device__ inline size_t delta_smem_bytes(int d, int dv, int dreg, int batch) {
  const size_t dpad = dreg > 0 ? dreg : d;
  const size_t widest = dv > d ? dv : d;
  return ((dreg > 0 ? 0 : (size_t)d * widest) + 3 * (size_t)batch * dpad) * sizeof(float) + 2 * (size_t)batch * dv * sizeof(T);
}

// SPLIT == 2: two threads share a column, each with 64 of its rows in registers; they are lanes l and l ^ 16 of one warp
// and add their partial sums with one shuffle.  Half the registers a thread, so more warps an SM holds: the walk waits
// on shared-memory and arithmetic latencies, which more warps hide.
template <typename T, int MODE, int DREG, int SPLIT>
__global__ void __launch_bounds__(DREG == 0 ? 1024 : 512) delta_rule_kernel(DeltaArgs a, int batch) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float red[32];
  __shared__ float s_kn[kDeltaBatch], s_qn[kDeltaBatch], s_beta[kDeltaBatch];
  const int d = a.d, head = blockIdx.x, b = blockIdx.y;
  const int c = MODE == 1 ? blockIdx.z % a.max_chunks : blockIdx.z;
  const bool transition = MODE == 1 && (int)blockIdx.z >= a.max_chunks;
  const int dv = a.dv;
  const int cols = transition ? d : dv;            // columns of the matrix this block carries
  const int kvh = head / (a.heads / a.kv_heads);
  constexpr int DP = DREG > 0 ? DREG : 1;          // rows of a column that a thread keeps
  const int dpad = DREG > 0 ? DREG * SPLIT : d;
  float* S = sm;                                   // [d][cols] (DREG == 0 only)
  float* qb = S + (DREG > 0 ? 0 : (size_t)d * (dv > d ? dv : d));   // [batch][dpad]
  float* kb = qb + (size_t)batch * dpad;           // [batch][dpad]
  float* db = kb + (size_t)batch * dpad;           // [batch][dpad]: the decays
  T* vb = reinterpret_cast<T*>(db + (size_t)batch * dpad);   // [batch][dv]
  T* gb = vb + (size_t)batch * dv;                 // [batch][dv]: the output gates before their sigmoid
  pdl_wait_block();
  pdl_launch_dependents();
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) {
    if (threadIdx.x == 0 && head == 0 && blockIdx.z == 0) report(a.status, kStatusSlotOutOfRange, b, slot, a.n_slots);
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
  const size_t unit = delta_unit(d, dv);
  float* cs = MODE != 0 ? a.scratch + (((size_t)b * a.max_chunks + c) * a.heads + head) * unit : nullptr;
  float* gS = a.S + ((size_t)slot * a.heads + head) * d * dv;
  const float* src = MODE == 0 ? gS : cs;
  // the thread's column and, with two threads a column, the first of its rows
  const int j = SPLIT == 2 ? (threadIdx.x >> 5) * 16 + (threadIdx.x & 15) : threadIdx.x;
  const int i0 = SPLIT == 2 ? ((threadIdx.x >> 4) & 1) * DP : 0;
  float Sr[DP];
  if (MODE == 1) {
    if (DREG > 0) {
#pragma unroll
      for (int i = 0; i < DP; ++i) Sr[i] = (transition && i0 + i == j) ? 1.f : 0.f;
    } else {
      for (int i = threadIdx.x; i < d * cols; i += blockDim.x) S[i] = (transition && i / cols == i % cols) ? 1.f : 0.f;
    }
  } else {
    if (DREG > 0) {
#pragma unroll
      for (int i = 0; i < DP; ++i) Sr[i] = (i0 + i < d && j < dv) ? src[(size_t)(i0 + i) * dv + j] : 0.f;
    } else {
      for (int i = threadIdx.x; i < d * dv; i += blockDim.x) S[i] = src[i];
    }
  }
  if (dpad > d)
    for (int e = threadIdx.x; e < batch * (dpad - d); e += blockDim.x) {
      const int tt = e / (dpad - d), i = d + e % (dpad - d);
      qb[(size_t)tt * dpad + i] = 0.f;
      kb[(size_t)tt * dpad + i] = 0.f;
      db[(size_t)tt * dpad + i] = 0.f;
    }
  const int channels = 2 * a.kv_heads * d + a.heads * dv;
  const int k_col = a.kv_heads * d, v_col = 2 * a.kv_heads * d;
  const T* x = (const T*)a.qkv;
  const float rate = expf(a.A_log[head]);
  const float nw = (MODE != 1 && j < dv) ? a.norm_w[j] : 0.f;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  // 16-byte staging where the rows allow it (a token's rows keep their alignment from token to token)
  const bool smem_ok = dpad % 4 == 0 && (DREG > 0 || (d * (dv > d ? dv : d)) % 4 == 0);
  const bool vec_k = smem_ok && stage_vec_ok<T>(x + (size_t)t0 * channels + k_col + kvh * d, channels, d);
  const bool vec_q = smem_ok && stage_vec_ok<T>(x + (size_t)t0 * channels + kvh * d, channels, d);
  const bool vec_v = smem_ok && stage_vec_ok<T>(x + (size_t)t0 * channels + v_col + head * dv, channels, dv);
  const bool vec_g = smem_ok && stage_vec_ok<T>((const T*)a.gate + (size_t)t0 * a.gate_ld + head * dv, a.gate_ld, dv);
  for (int tb = t0; tb < t1; tb += batch) {
    const int nb = min(batch, t1 - tb);
    __syncthreads();                               // the batch before this one has been read
    stage_rows_f32<T>(kb, dpad, x + (size_t)tb * channels + k_col + kvh * d, channels, nb, d, 1.f, vec_k);
    if (MODE != 1) stage_rows_f32<T>(qb, dpad, x + (size_t)tb * channels + kvh * d, channels, nb, d, 1.f, vec_q);
    // the decays: exp(-exp(A) softplus(a + dt)) per token and key channel
    for (int e = threadIdx.x; e < nb * d; e += blockDim.x) {
      const int tt = e / d, i = e - tt * d;
      const float z = a.head_decay ? a.a[(size_t)(tb + tt) * a.a_ld + head] + a.dt_bias[head]
                                   : a.a[(size_t)(tb + tt) * a.a_ld + head * d + i] + a.dt_bias[head * d + i];
      const float softplus = z > 20.f ? z : log1pf(expf(z));
      db[(size_t)tt * dpad + i] = expf(-rate * softplus);
    }
    if (!transition) {
      stage_rows_raw<T>(vb, x + (size_t)tb * channels + v_col + head * dv, channels, nb, dv, vec_v);
      if (MODE != 1) stage_rows_raw<T>(gb, (const T*)a.gate + (size_t)tb * a.gate_ld + head * dv, a.gate_ld, nb, dv, vec_g);
    }
    if (threadIdx.x < nb) s_beta[threadIdx.x] = 1.f / (1.f + expf(-a.b[(size_t)(tb + threadIdx.x) * a.b_ld + head]));
    __syncthreads();
    for (int tt = warp; tt < nb; tt += n_warps) {  // a warp per token: the lengths of k and q
      float k2 = 0.f, q2 = 0.f;
      for (int i = lane; i < d; i += 32) {
        const float kk = kb[(size_t)tt * dpad + i];
        k2 = fmaf(kk, kk, k2);
        if (MODE != 1) {
          const float qq = qb[(size_t)tt * dpad + i];
          q2 = fmaf(qq, qq, q2);
        }
      }
      k2 = warp_sum(k2);
      q2 = warp_sum(q2);
      if (lane == 0) {
        s_kn[tt] = rsqrtf(k2 + 1e-6f);
        s_qn[tt] = rsqrtf(q2 + 1e-6f) * a.q_scale;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nb; ++tt) {
      const float kn = s_kn[tt], qn = s_qn[tt], beta = s_beta[tt];
      const float* ks = kb + (size_t)tt * dpad;
      const float* qs = qb + (size_t)tt * dpad;
      const float* gs = db + (size_t)tt * dpad;
      float o = 0.f;
      if (DREG > 0 && SPLIT == 2) {
        // whole warps walk together (the two halves of a column meet in a shuffle); a column beyond the matrix
        // carries zeros and is never stored
        float acc = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        const float vj = (transition || j >= dv) ? 0.f : to_f32<T>(vb[(size_t)tt * dv + j]);
#pragma unroll
        for (int i = 0; i < DP; i += 4) {
          const float4 g4 = *reinterpret_cast<const float4*>(gs + i0 + i);
          const float4 k4 = *reinterpret_cast<const float4*>(ks + i0 + i);
          Sr[i] *= g4.x; Sr[i + 1] *= g4.y; Sr[i + 2] *= g4.z; Sr[i + 3] *= g4.w;
          acc = fmaf(Sr[i], k4.x, acc);            // four sums side by side: a chain of dependent adds is what
          acc1 = fmaf(Sr[i + 1], k4.y, acc1);      // the walk would otherwise wait for
          acc2 = fmaf(Sr[i + 2], k4.z, acc2);
          acc3 = fmaf(Sr[i + 3], k4.w, acc3);
        }
        acc = (acc + acc1) + (acc2 + acc3);
        acc += __shfl_xor_sync(0xffffffffu, acc, 16);
        const float uk = beta * (vj - acc * kn) * kn;
#pragma unroll
        for (int i = 0; i < DP; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(ks + i0 + i);
          Sr[i] = fmaf(k4.x, uk, Sr[i]);
          Sr[i + 1] = fmaf(k4.y, uk, Sr[i + 1]);
          Sr[i + 2] = fmaf(k4.z, uk, Sr[i + 2]);
          Sr[i + 3] = fmaf(k4.w, uk, Sr[i + 3]);
          if (MODE != 1) {
            const float4 q4 = *reinterpret_cast<const float4*>(qs + i0 + i);
            o = fmaf(Sr[i], q4.x, o);
            o1 = fmaf(Sr[i + 1], q4.y, o1);
            o2 = fmaf(Sr[i + 2], q4.z, o2);
            o3 = fmaf(Sr[i + 3], q4.w, o3);
          }
        }
        o = (o + o1) + (o2 + o3);
        if (MODE != 1) o = (o + __shfl_xor_sync(0xffffffffu, o, 16)) * qn;
      } else if (j < cols) {
        float acc = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        const float vj = transition ? 0.f : to_f32<T>(vb[(size_t)tt * dv + j]);
        if (DREG > 0) {
#pragma unroll
          for (int i = 0; i < DP; i += 4) {
            const float4 g4 = *reinterpret_cast<const float4*>(gs + i);
            const float4 k4 = *reinterpret_cast<const float4*>(ks + i);
            Sr[i] *= g4.x; Sr[i + 1] *= g4.y; Sr[i + 2] *= g4.z; Sr[i + 3] *= g4.w;
            acc = fmaf(Sr[i], k4.x, acc);
            acc1 = fmaf(Sr[i + 1], k4.y, acc1);
            acc2 = fmaf(Sr[i + 2], k4.z, acc2);
            acc3 = fmaf(Sr[i + 3], k4.w, acc3);
          }
          acc = (acc + acc1) + (acc2 + acc3);
          const float uk = beta * (vj - acc * kn) * kn;
#pragma unroll
          for (int i = 0; i < DP; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(ks + i);
            Sr[i] = fmaf(k4.x, uk, Sr[i]);
            Sr[i + 1] = fmaf(k4.y, uk, Sr[i + 1]);
            Sr[i + 2] = fmaf(k4.z, uk, Sr[i + 2]);
            Sr[i + 3] = fmaf(k4.w, uk, Sr[i + 3]);
            if (MODE != 1) {
              const float4 q4 = *reinterpret_cast<const float4*>(qs + i);
              o = fmaf(Sr[i], q4.x, o);
              o1 = fmaf(Sr[i + 1], q4.y, o1);
              o2 = fmaf(Sr[i + 2], q4.z, o2);
              o3 = fmaf(Sr[i + 3], q4.w, o3);
            }
          }
          o = (o + o1) + (o2 + o3);
        } else {
          for (int i = 0; i < d; ++i) {
            const float s = gs[i] * S[(size_t)i * cols + j];
            S[(size_t)i * cols + j] = s;
            acc = fmaf(s, ks[i], acc);
          }
          const float uk = beta * (vj - acc * kn) * kn;
          for (int i = 0; i < d; ++i) {
            const float s = fmaf(ks[i], uk, S[(size_t)i * cols + j]);
            S[(size_t)i * cols + j] = s;
            if (MODE != 1) o = fmaf(s, qs[i], o);
          }
        }
        o *= qn;
      }
      if (MODE == 1) continue;                     // a column is its own thread's, the staged rows are only read
      const float ss = block_sum((i0 == 0 && j < dv) ? o * o : 0.f, red);
      if (j < dv && i0 == 0) {
        const float gate = to_f32<T>(gb[(size_t)tt * dv + j]);
        const float y = o * rsqrtf(ss / (float)dv + a.eps) * nw * (a.gate_silu ? gate : 1.f) / (1.f + expf(-gate));
        ((T*)a.out)[(size_t)(tb + tt) * a.heads * dv + head * dv + j] = from_f32<T>(y);
      }
    }
  }
  __syncthreads();
  if (MODE == 3 && t1 != q1) return;               // only the sequence's last chunk leaves the state
  float* dst = MODE == 1 ? (transition ? cs + (size_t)d * dv : cs) : gS;
  if (DREG > 0) {
    if (j < cols) {
#pragma unroll
      for (int i = 0; i < DP; ++i)
        if (i0 + i < d) dst[(size_t)(i0 + i) * cols + j] = Sr[i];
    }
  } else {
    for (int i = threadIdx.x; i < d * cols; i += blockDim.x) dst[i] = S[i];
  }
}

// Chain the chunks: on entry scratch[c] holds chunk c's end state from zero and its transition matrix (every chunk
// but the sequence's last); on exit its S part holds chunk c's true start state, chunk 0's being the slot's state.
// A block takes a few columns of one head's state: thread (i, col) keeps element i of its column, the chunk's
// transition matrix passes through shared memory (rows padded by one float, so that a read across i has no conflicts).
// The next chunk's matrix is on its way into registers while this chunk's product runs.  (What a chunk costs here is
// the arrival of its matrix, 4 d^2 bytes for every block: forms with fewer threads a block and four columns a thread,
// which halve the shared-memory reads of the product, took two to four times as long.)
constexpr int kChainLoads = 16;                    // floats of the matrix a thread carries ahead (d * d <= 16 * threads)

__global__ void __launch_bounds__(1024) delta_chain_kernel(DeltaArgs a, int col_tile) {
  extern __shared__ float sm[];
  const int d = a.d, dv = a.dv, head = blockIdx.x, b = blockIdx.y;
  float* Ts = sm;                                  // [d][d + 1]
  float* cur = Ts + (size_t)d * (d + 1);           // [col_tile][d]
  pdl_wait_block();
  pdl_launch_dependents();
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) return;
  const int q_len = a.seq_qstart[b + 1] - a.seq_qstart[b];
  const int n_chunks = (q_len + a.chunk - 1) / a.chunk;
  const int i = threadIdx.x % d, cj = threadIdx.x / d;
  const int j = blockIdx.z * col_tile + cj;
  const bool live = cj < col_tile && j < dv;
  const size_t unit = delta_unit(d, dv);
  float* cs = a.scratch + ((size_t)b * a.max_chunks * a.heads + head) * unit;
  const size_t per = (size_t)a.heads * unit;
  float val = live ? a.S[((size_t)slot * a.heads + head) * d * dv + (size_t)i * dv + j] : 0.f;
  // this thread's share of a matrix: elements threadIdx.x + r * blockDim.x, at row tr + r * tstep of shared memory
  const int tr = threadIdx.x / d, tc = threadIdx.x % d, tstep = blockDim.x / d;
  const bool by_rows = blockDim.x % d == 0;        // else the share is addressed element by element
  const bool ahead = d * d <= kChainLoads * (int)blockDim.x;   // else a chunk's matrix is loaded when its turn comes
  float tn[kChainLoads];
  auto fetch = [&](int c) {
    const float* Tg = cs + (size_t)c * per + (size_t)d * dv;
#pragma unroll
    for (int r = 0; r < kChainLoads; ++r) {
      const int e = threadIdx.x + r * blockDim.x;
      tn[r] = e < d * d ? Tg[e] : 0.f;
    }
  };
  if (ahead && n_chunks > 1) fetch(0);
  for (int c = 0; c < n_chunks; ++c) {
    float* u = cs + (size_t)c * per;
    const bool has = c + 1 < n_chunks;
    const float loc = (has && live) ? u[(size_t)i * dv + j] : 0.f;
    if (live) u[(size_t)i * dv + j] = val;
    if (!has) break;
    if (ahead) {
#pragma unroll
      for (int r = 0; r < kChainLoads; ++r) {
        const int e = threadIdx.x + r * blockDim.x;
        if (e < d * d) {
          if (by_rows) Ts[(size_t)(tr + r * tstep) * (d + 1) + tc] = tn[r];
          else Ts[(size_t)(e / d) * (d + 1) + e % d] = tn[r];
        }
      }
    } else {
      const float* Tg = u + (size_t)d * dv;
      for (int e = threadIdx.x; e < d * d; e += blockDim.x) Ts[(size_t)(e / d) * (d + 1) + e % d] = Tg[e];
    }
    if (cj < col_tile) cur[(size_t)cj * d + i] = val;
    __syncthreads();
    if (ahead && c + 2 < n_chunks) fetch(c + 1);   // in flight during the product below
    float acc0 = loc, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    if (live) {
      const float* trow = Ts + (size_t)i * (d + 1);
      const float* col = cur + (size_t)cj * d;
      int k = 0;
      for (; k + 4 <= d; k += 4) {
        acc0 = fmaf(trow[k], col[k], acc0);
        acc1 = fmaf(trow[k + 1], col[k + 1], acc1);
        acc2 = fmaf(trow[k + 2], col[k + 2], acc2);
        acc3 = fmaf(trow[k + 3], col[k + 3], acc3);
      }
      for (; k < d; ++k) acc0 = fmaf(trow[k], col[k], acc0);
    }
    val = (acc0 + acc1) + (acc2 + acc3);
    __syncthreads();
  }
}

template <typename T, int DREG, int SPLIT>
static int delta_run(const DeltaArgs& a, cudaStream_t stream) {
  const int d = a.d, dv = a.dv;
  const int widest = dv > d ? dv : d;
  int batch = kDeltaBatch;                       // as many tokens staged at a time as shared memory takes
  while (batch > 1 && delta_smem_bytes<T>(d, dv, DREG * SPLIT, batch) > 200 * 1024) batch /= 2;
  const size_t smem = delta_smem_bytes<T>(d, dv, DREG * SPLIT, batch);
  if (smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  int threads = (SPLIT * widest + 31) / 32 * 32;
  const int cap_threads = DREG == 0 ? 1024 : 512;
  if (threads > cap_threads) threads = cap_threads;
  if (SPLIT * widest > threads) return PE_ERR_UNSUPPORTED_SIZE;
  auto k0 = delta_rule_kernel<T, 0, DREG, SPLIT>;
  auto k1 = delta_rule_kernel<T, 1, DREG, SPLIT>;
  auto k3 = delta_rule_kernel<T, 3, DREG, SPLIT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (a.chunk > 0) {
    launch(k1, dim3(a.heads, a.n_seqs, 2 * a.max_chunks), dim3(threads), smem, stream, a, batch);
    int col_tile = 1024 / d;
    if (col_tile > 8) col_tile = 8;
    if (col_tile < 1) return PE_ERR_UNSUPPORTED_SIZE;
    const size_t chain_smem = ((size_t)d * (d + 1) + (size_t)col_tile * d) * sizeof(float);
    if (chain_smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
    if (chain_smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(delta_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)chain_smem);
      if (e != cudaSuccess) return (int)e;
    }
    launch(delta_chain_kernel, dim3(a.heads, a.n_seqs, (dv + col_tile - 1) / col_tile), dim3(col_tile * d), chain_smem, stream, a,
           col_tile);
    launch(k3, dim3(a.heads, a.n_seqs, a.max_chunks), dim3(threads), smem, stream, a, batch);
  } else {
    launch(k0, dim3(a.heads, a.n_seqs, 1), dim3(threads), smem, stream, a, batch);
  }
  return PE_OK;
}

}  // namespace pe

extern "C" int pe_short_conv_silu(int dtype, const void* x, long long ld, int col0, const float* w, const float* bias, int taps, float* tail,
                                  const int* token_seq, const int* seq_slot, const int* seq_qstart, void* out,
                                  int n_tokens, int n_seqs, int channels, int n_slots, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (channels <= 0 || taps <= 0 || taps > 64 || col0 < 0 || col0 + channels > ld) return PE_ERR_BAD_ARGUMENT;
  const int threads = channels >= 1024 ? 256 : 128;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  const bool vec8 = dtype == PE_BF16 && taps >= 2 && taps <= 4 && channels % 8 == 0 && ld % 8 == 0 && col0 % 8 == 0 &&
                    (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)tail % 16 == 0;   // (taps == 1: no tail is read)
  if (vec8) {
    const int strip = n_tokens >= 512 ? 8 : 1;
    const size_t total = (size_t)((n_tokens + strip - 1) / strip) * (channels / 8);
    size_t blocks = (total + 127) / 128;
    if (blocks > (size_t)pe::kSMs * 32) blocks = (size_t)pe::kSMs * 32;
    auto kernel = taps == 2 ? pe::short_conv_vec8_kernel<2> : (taps == 3 ? pe::short_conv_vec8_kernel<3> : pe::short_conv_vec8_kernel<4>);
    pe::launch(kernel, (int)blocks, 128, 0, stream, (const __nv_bfloat16*)x, ld, col0, w, bias, (const float*)tail, token_seq, seq_slot,
               seq_qstart, (__nv_bfloat16*)out, n_tokens, channels, n_slots, status, strip);
  } else if (dtype == PE_F32)
    pe::launch(pe::short_conv_kernel<float>, n_tokens, threads, 0, stream, (const float*)x, ld, col0, w, bias, taps, (const float*)tail,
               token_seq, seq_slot, seq_qstart, (float*)out, n_tokens, channels, n_slots, status);
  else
    pe::launch(pe::short_conv_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)x, ld, col0, w, bias, taps,
               (const float*)tail, token_seq, seq_slot, seq_qstart, (__nv_bfloat16*)out, n_tokens, channels, n_slots, status);
  PE_LAUNCH_CHECK();
  if (taps > 1) {
    const dim3 grid((channels + 127) / 128, n_seqs);
    if (dtype == PE_F32)
      pe::launch(pe::conv_tail_kernel<float>, grid, dim3(128), 0, stream, (const float*)x, ld, col0, tail, taps, seq_slot,
                 seq_qstart, n_seqs, channels, n_slots);
    else
      pe::launch(pe::conv_tail_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)x, ld, col0, tail, taps,
                 seq_slot, seq_qstart, n_seqs, channels, n_slots);
    PE_LAUNCH_CHECK();
  }
  return PE_OK;
}

// Floats of scratch that the chunked form needs for `max_chunks` chunks per sequence.
extern "C" long long pe_delta_rule_scratch_floats(int n_seqs, int heads, int d, int dv, int max_chunks) {
  return (long long)n_seqs * max_chunks * heads * (long long)pe::delta_unit(d, dv);
}

// chunk > 0: prompts cut into chunks of that many tokens (scratch from pe_delta_rule_scratch_floats, max_chunks >=
// ceil(max_q / chunk)); chunk == 0: each sequence's tokens in one go (single tokens, short prompts).
extern "C" int pe_delta_rule_recurrence(int dtype, const void* qkv, const float* a, const float* dt_bias, const float* A_log,
                                        const float* b, const void* gate, long long gate_ld, const float* norm_w, float eps,
                                        float q_scale, void* out, float* S, const int* seq_slot, const int* seq_qstart,
                                        int n_seqs, int max_q, int heads, int kv_heads, int d, int dv, int n_slots, int chunk,
                                        int max_chunks, float* scratch, int head_decay, int gate_silu, long long a_ld,
                                        long long b_ld, int* status, cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || d <= 0 || dv <= 0) return PE_ERR_BAD_ARGUMENT;
  if (dv > 1024 || d > 1024) return PE_ERR_UNSUPPORTED_SIZE;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  pe::DeltaArgs args{qkv, a, dt_bias, A_log, b, gate, gate_ld, norm_w, eps, q_scale, out, S, seq_slot, seq_qstart,
                     n_seqs, heads, kv_heads, d, dv, n_slots, 0, 1, nullptr, status, head_decay, gate_silu,
                     a_ld > 0 ? a_ld : (long long)(head_decay ? heads : heads * d), b_ld > 0 ? b_ld : (long long)heads};
  if (chunk > 0) {
    if (!scratch || max_chunks <= 0 || (long long)max_chunks * chunk < max_q || max_chunks > 32767) return PE_ERR_BAD_ARGUMENT;
    args.chunk = chunk; args.max_chunks = max_chunks; args.scratch = scratch;
  }
  const int widest = dv > d ? dv : d;
  // 128: two threads a column with 64 rows each (the columns then fill whole half-warps)
  const int reg = (d <= 32 && widest <= 512) ? 32
                  : (d <= 64 && widest <= 512 ? 64 : (d <= 128 && widest <= 256 && dv % 16 == 0 && d % 16 == 0 ? 128 : 0));
  if (reg == 0 && ((size_t)d * widest + 3 * (size_t)d + 2 * (size_t)dv) * sizeof(float) > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  int rc;
#define PE_DELTA(T)                                                       \
  (reg == 32 ? pe::delta_run<T, 32, 1>(args, stream)                      \
   : reg == 64 ? pe::delta_run<T, 64, 1>(args, stream)                    \
   : reg == 128 ? pe::delta_run<T, 64, 2>(args, stream) : pe::delta_run<T, 0, 1>(args, stream))
  rc = dtype == PE_F32 ? PE_DELTA(float) : PE_DELTA(__nv_bfloat16);
#undef PE_DELTA
  if (rc != PE_OK) return rc;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
