// Causal attention of many query heads over ONE cached row per position whose leading features are also
// the values (a latent cache: the row is [latent | rotated key part], the value is the latent), on the
// tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 accumulation).  Rows of up to 576 features
// in steps of 64; values of 128, 256 or 512 features.  Other shapes and the float32 mode use
// attention_generic.cu (same arguments: one kv head, v_ld = row).
//
// Scores, the softmax state (m, l) and the output accumulator are float32.  The tensor cores take bfloat16
// operands, so each probability enters the P.V product as the sum of two bfloat16 terms (its rounding and
// the rounding of what that left over: 16 significant bits instead of 8), in two products.
//
// Rows.  A "row" is a (query token, head) pair of one sequence: row r is token r / n_heads, head
// r % n_heads.  All rows share the cached rows, so heads ride along in the M dimension.  A block owns
// M = 16 * MB rows and walks the 64-key pages; the page (64 x row bfloat16, up to 72 KB) arrives by TMA
// into one of two stages, split into 64-feature sub-tiles with the 128-byte swizzle.  The accumulator
// of a 512-feature value does not fit one warp's registers beside the scores, so the block's MB * KS
// warps split the work twice: for Q.K^T warp (rb, ks) takes row block rb and keys [ks * 64/KS, ..) of
// the page; the row maxima are exchanged through shared memory, P (both terms) goes to shared memory, and
// for P.V the same warp takes row block rb and value features [ks * RANK/KS, ..) over all 64 keys.
//   prefill: MB = 4, KS = 2 (256 threads, 64 rows), or MB = 3 (192 threads, 48 rows) where the 64 query
//            rows no longer fit shared memory beside the stages (rows of 576); grid (row tiles, sequences).
//   decode:  MB = 1, KS = 4 (128 threads, 16 heads of the sequence's one token); grid (key ranges, head
//            blocks, sequences); a second kernel merges the ranges by their log-sum-exp weights.  Which
//            keys a partial result covers depends only on the sequence's own length.
// Rows of a page beyond the sequence's length are not read as zeros: the cache never holds a non-finite
// value there, and their probabilities are exactly zero.
#include "api.h"
#include "common.cuh"
#include "tma.cuh"

namespace pe {
namespace la {

constexpr int BN = 64;  // keys per tile = one cache page

struct Args {
  const __nv_bfloat16* q; long long q_ld;   // token t, head h: q + t * q_ld + h * row
  __nv_bfloat16* out;     long long out_ld; // token t, head h: out + t * out_ld + h * RANK
  int n_heads, row;
  float scale_log2;                         // softmax scale * log2(e)
  const int* seq_qstart; const int* seq_past; const int* seq_slot;
  const int* page_table; int table_stride; int num_pages;
  int* status;
  float* part_acc; float* part_lse; int split_keys, max_splits, min_range_keys;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware approximation (exp2(-inf) = 0): the result is rounded to bfloat16 or summed into a
// float32 denominator, so this is within the path's precision.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `r` in a [rows][features] bfloat16 tile kept as sub-tiles of
// [rows][64] with the 128-byte swizzle (the layout TMA writes): the chunks of a row are XOR-ed with r & 7.
__device__ __forceinline__ uint32_t tile_off(int r, int chunk, int rows) {
  return (uint32_t)((chunk >> 3) * (rows * 128) + r * 128 + (((chunk & 7) ^ (r & 7)) << 4));
}

// The page table's entry for the page that holds position k0 (-1 beyond the table).  The value is looked at only by
// issue_page, one round later, so that the elected thread does not wait for the table while the others compute.
__device__ __forceinline__ int lookup_page(const Args& a, int slot, int k0) {
  const int logical = k0 / BN;
  return logical < a.table_stride ? a.page_table[(size_t)slot * a.table_stride + logical] : -1;
}

// One elected thread starts the copy of `page` (it holds position k0) into a stage; `bar` counts the bytes.
__device__ __forceinline__ void issue_page(const Args& a, const CUtensorMap* map, int slot, int k0, int page, char* stage,
                                           uint64_t* bar) {
  if (page < 0 || page >= a.num_pages) {
    report(a.status, kStatusPageOutOfRange, slot, page, k0);
    page = 0;
  }
  tma::mbar_expect_tx(bar, BN * a.row * 2);
  for (int sub = 0; sub < a.row / 64; ++sub) tma::load_2d(stage + sub * (BN * 128), map, sub * 64, page * BN, bar);
}

// A wait ran out: record it, give copies still in flight a last bounded chance to land, and leave.
__device__ __forceinline__ void give_up(const Args& a, uint64_t* bars, int where) {
  if (threadIdx.x == 0) report(a.status, kStatusWaitTimedOut, where, blockIdx.x, blockIdx.z);
  for (int s = 0; s < 2; ++s)
    for (int i = 0; i < 1000; ++i)
      if (tma::mbar_try_wait(&bars[s], 0) || tma::mbar_try_wait(&bars[s], 1)) break;
}

__device__ __forceinline__ char* align_1024(char* p) {
  return reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}

// Keys per range of a sequence of `len` keys (decode): the fixed split_keys, or (split_keys == 0) the sequence's
// own length shared out evenly over max_splits ranges, in whole pages, but no fewer than min_range_keys.
__device__ __forceinline__ int range_keys(const Args& a, int len) {
  if (a.split_keys > 0) return a.split_keys;
  const int per = (len + a.max_splits - 1) / a.max_splits;
  return max(max(BN, a.min_range_keys), (per + BN - 1) / BN * BN);
}

template <int MB, int KS>
constexpr size_t smem_bytes(int row) {
  // two stages, the queries, both terms of P, and the exchanged row maxima and denominators
  return (size_t)2 * BN * row * 2 + (size_t)MB * 16 * row * 2 + (size_t)2 * MB * 16 * 128 + (size_t)2 * KS * MB * 16 * 4 + 1024;
}

// grid prefill: (row tiles of 16 * MB, n_seqs); decode: (max_splits, blocks of 16 heads, n_seqs).
template <int RANK, int MB, int KS, bool DECODE>
__global__ void __launch_bounds__(MB * KS * 32, 1) latent_kernel(Args a, const __grid_constant__ CUtensorMap map) {
  extern __shared__ char smem_raw[];
  __shared__ uint64_t bars[2];
  pdl_wait_block();
  pdl_launch_dependents();
  constexpr int M = MB * 16;          // rows of the block
  constexpr int KW = BN / KS;         // keys of a page that one warp scores
  constexpr int NT = KW / 8;          // their n-tiles
  constexpr int DW = RANK / KS;       // value features that one warp accumulates
  constexpr int NO = DW / 8;          // their n-tiles
  constexpr int THREADS = MB * KS * 32;
  static_assert(NT >= 2 && NT % 2 == 0 && NO % 2 == 0, "warps take pairs of n-tiles");
  const int row = a.row;
  const int stage_bytes = BN * row * 2;
  char* smem = align_1024(smem_raw);
  char* q_s = smem + 2 * stage_bytes;                         // [M][row] swizzled
  char* p_s = q_s + M * row * 2;                              // [2][M][64] swizzled: P's leading and trailing terms
  float* mx_s = reinterpret_cast<float*>(p_s + 2 * M * 128);  // [KS][M] row maxima of the page
  float* l_s = mx_s + KS * M;                                 // [KS][M] denominators at the end
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rb = warp % MB, ks = warp / MB;
  const int b = DECODE ? blockIdx.z : blockIdx.y;
  const int nh = a.n_heads;
  const int q0 = a.seq_qstart[b], past = a.seq_past[b];
  const int q_len = DECODE ? 1 : a.seq_qstart[b + 1] - q0;
  const int n_rows = q_len * nh;
  // prefill: late rows see the most keys and go first, so that the longest blocks do not form the tail
  const int row0 = DECODE ? (int)blockIdx.y * M : ((int)gridDim.x - 1 - (int)blockIdx.x) * M;
  if (row0 >= n_rows) return;
  int k_lo = 0, k_hi;
  if (DECODE) {
    const int len = past + 1;
    const int per_range = range_keys(a, len);
    k_lo = (int)blockIdx.x * per_range;
    k_hi = min(len, k_lo + per_range);
    if (k_lo >= len) return;
  } else {
    k_hi = past + (min(n_rows, row0 + M) - 1) / nh + 1;       // the block's last row sees keys up to its own position
  }
  const int slot = a.seq_slot[b];
  const int n_tiles = (k_hi - k_lo + BN - 1) / BN;

  int page_next = -1;   // the elected thread's: the table's entry for the page after the one in flight
  if (tid == 0) {
    tma::mbar_init(&bars[0], 1);
    tma::mbar_init(&bars[1], 1);
    tma::fence_barrier_init();
    issue_page(a, &map, slot, k_lo, lookup_page(a, slot, k_lo), smem, &bars[0]);
    if (n_tiles > 1) page_next = lookup_page(a, slot, k_lo + BN);
  }
  const int cpr = row / 8;   // 16-byte chunks of a query row
  for (int i = tid; i < M * cpr; i += THREADS) {
    const int r = i / cpr, chunk = i - r * cpr;
    const int rr = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rr < n_rows) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(q0 + rr / nh) * a.q_ld + (size_t)(rr % nh) * row + chunk * 8);
    *reinterpret_cast<uint4*>(q_s + tile_off(r, chunk, M)) = v;
  }
  __syncthreads();
  // this thread's two rows and their positions (rows beyond n_rows are never stored)
  const int r_lo = row0 + rb * 16 + g, r_hi = r_lo + 8;
  const int pos_lo = past + r_lo / nh, pos_hi = past + r_hi / nh;
  float o[NO][4];
#pragma unroll
  for (int n = 0; n < NO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;   // l: over this warp's keys only
  const uint32_t q_base = smem_u32(q_s), p_base = smem_u32(p_s);
  const int a_row = rb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;     // this lane's row of an A operand (Q or P)

  for (int it = 0; it < n_tiles; ++it) {
    const int k0 = k_lo + it * BN;
    // next page into the other stage (everyone left it at the end of the last round)
    if (tid == 0 && it + 1 < n_tiles) {
      issue_page(a, &map, slot, k0 + BN, page_next, smem + ((it + 1) & 1) * stage_bytes, &bars[(it + 1) & 1]);
      if (it + 2 < n_tiles) page_next = lookup_page(a, slot, k0 + 2 * BN);
    }
    if (!tma::mbar_wait(&bars[it & 1], (it >> 1) & 1)) {
      give_up(a, bars, 3);
      return;
    }
    const uint32_t k_base = smem_u32(smem + (it & 1) * stage_bytes);
    // ---- scores of this warp's rows and keys
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll 4   // rows come in steps of 64 features: the loads of four steps can be in flight ahead of their products
    for (int kk = 0; kk < row / 16; ++kk) {
      uint32_t qf[4];
      ldmatrix_x4(qf, q_base + tile_off(a_row, kk * 2 + (lane >> 4), M));
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t kb[4];
        const int key = ks * KW + np * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(kb, k_base + tile_off(key, kk * 2 + ((lane >> 3) & 1), BN));
        mma_bf16(s[np * 2], qf, kb[0], kb[1]);
        mma_bf16(s[np * 2 + 1], qf, kb[2], kb[3]);
      }
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kpos = k0 + ks * KW + n * 8 + 2 * t + (e & 1);
        const bool vis = DECODE ? (kpos < k_hi) : (kpos <= ((e < 2) ? pos_lo : pos_hi));
        const float v = vis ? s[n][e] * a.scale_log2 : -INFINITY;
        s[n][e] = v;
        if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    if (t == 0) {
      mx_s[ks * M + rb * 16 + g] = mx_lo;
      mx_s[ks * M + rb * 16 + g + 8] = mx_hi;
    }
    __syncthreads();
    // ---- the page's row maxima over all keys: every warp of a row block keeps the same running maximum
    float mn_lo = m_lo, mn_hi = m_hi;
#pragma unroll
    for (int w = 0; w < KS; ++w) {
      mn_lo = fmaxf(mn_lo, mx_s[w * M + rb * 16 + g]);
      mn_hi = fmaxf(mn_hi, mx_s[w * M + rb * 16 + g + 8]);
    }
    const float al_lo = (m_lo == -INFINITY) ? 0.f : fast_exp2(m_lo - mn_lo);
    const float al_hi = (m_hi == -INFINITY) ? 0.f : fast_exp2(m_hi - mn_hi);
    const float base_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, base_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const float p0 = fast_exp2(s[n][0] - base_lo), p1 = fast_exp2(s[n][1] - base_lo);
      const float p2 = fast_exp2(s[n][2] - base_hi), p3 = fast_exp2(s[n][3] - base_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      const int chunk = ks * NT + n;   // keys chunk * 8 .. + 7 of the page
      const uint32_t off_lo = tile_off(rb * 16 + g, chunk, M) + 4 * t, off_hi = tile_off(rb * 16 + g + 8, chunk, M) + 4 * t;
      const __nv_bfloat162 lead_lo = __floats2bfloat162_rn(p0, p1), lead_hi = __floats2bfloat162_rn(p2, p3);
      *reinterpret_cast<__nv_bfloat162*>(p_s + off_lo) = lead_lo;
      *reinterpret_cast<__nv_bfloat162*>(p_s + off_hi) = lead_hi;
      *reinterpret_cast<uint32_t*>(p_s + M * 128 + off_lo) =
          pack_bf16(p0 - __bfloat162float(lead_lo.x), p1 - __bfloat162float(lead_lo.y));
      *reinterpret_cast<uint32_t*>(p_s + M * 128 + off_hi) =
          pack_bf16(p2 - __bfloat162float(lead_hi.x), p3 - __bfloat162float(lead_hi.y));
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * al_lo + sum_lo;
    l_hi = l_hi * al_hi + sum_hi;
    m_lo = mn_lo;
    m_hi = mn_hi;
#pragma unroll
    for (int n = 0; n < NO; ++n) {
      o[n][0] *= al_lo; o[n][1] *= al_lo; o[n][2] *= al_hi; o[n][3] *= al_hi;
    }
    __syncthreads();
    // ---- P.V over all 64 keys for this warp's value features (the leading RANK features of the cached rows)
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t pf[4], pr[4];
      ldmatrix_x4(pf, p_base + tile_off(a_row, kk * 2 + (lane >> 4), M));
      ldmatrix_x4(pr, p_base + M * 128 + tile_off(a_row, kk * 2 + (lane >> 4), M));
      const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int np = 0; np < NO / 2; ++np) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, k_base + tile_off(key, ks * (DW / 8) + np * 2 + (lane >> 4), BN));
        mma_bf16(o[np * 2], pf, vb[0], vb[1]);
        mma_bf16(o[np * 2 + 1], pf, vb[2], vb[3]);
        mma_bf16(o[np * 2], pr, vb[0], vb[1]);
        mma_bf16(o[np * 2 + 1], pr, vb[2], vb[3]);
      }
    }
    __syncthreads();  // the stage, P and the maxima may be overwritten in the next round
  }
  // ---- the denominators of all key slices
  if (t == 0) {
    l_s[ks * M + rb * 16 + g] = l_lo;
    l_s[ks * M + rb * 16 + g + 8] = l_hi;
  }
  __syncthreads();
  float lt_lo = 0.f, lt_hi = 0.f;
#pragma unroll
  for (int w = 0; w < KS; ++w) {
    lt_lo += l_s[w * M + rb * 16 + g];
    lt_hi += l_s[w * M + rb * 16 + g + 8];
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int rr = half ? r_hi : r_lo;
    if (rr >= n_rows) continue;
    const int tok = rr / nh, head = rr % nh;
    const float lt = half ? lt_hi : lt_lo, mm = half ? m_hi : m_lo;
    const float inv = (lt > 0.f) ? 1.f / lt : 0.f;
    if (DECODE) {
      const size_t pidx = ((size_t)b * nh + head) * a.max_splits + blockIdx.x;
      float* dst = a.part_acc + pidx * RANK + ks * DW;
#pragma unroll
      for (int n = 0; n < NO; ++n)
        *reinterpret_cast<float2*>(dst + n * 8 + 2 * t) = make_float2(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
      // log-sum-exp in natural units, as the merge expects: (m + log2 l) * ln 2
      if (ks == 0 && t == 0) a.part_lse[pidx] = (lt > 0.f) ? (mm + log2f(lt)) * 0.6931471805599453f : -INFINITY;
    } else {
      __nv_bfloat16* dst = a.out + (size_t)(q0 + tok) * a.out_ld + (size_t)head * RANK + ks * DW;
#pragma unroll
      for (int n = 0; n < NO; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
    }
  }
}

// grid: (n_heads, n_seqs): merge the key ranges of one (sequence, head) by their log-sum-exp weights, in range order.
template <int RANK>
__global__ void latent_merge_kernel(Args a) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.y, h = blockIdx.x;
  const int tq = a.seq_qstart[b];
  const int len = a.seq_past[b] + 1;
  const int per_range = range_keys(a, len);
  int n_splits = (len + per_range - 1) / per_range;
  if (n_splits > a.max_splits) {
    // only with a fixed split_keys: the sequence is longer than split_keys * max_splits keys, for which the split grid
    // has no blocks and the scratch no room; say so and merge what was computed
    if (threadIdx.x == 0) report(a.status, kStatusPositionOutOfRange, b, len - 1, per_range * a.max_splits);
    n_splits = a.max_splits;
  }
  const size_t base = ((size_t)b * a.n_heads + h) * a.max_splits;
  __nv_bfloat16* o = a.out + (size_t)tq * a.out_ld + (size_t)h * RANK;
  float mx = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, a.part_lse[base + s]);
  float denom = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float e = a.part_lse[base + s];
    denom += (e == -INFINITY) ? 0.f : expf(e - mx);
  }
  const float inv = 1.f / fmaxf(denom, 1e-20f);
  for (int c = threadIdx.x; c < RANK; c += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float e = a.part_lse[base + s];
      const float w = (e == -INFINITY) ? 0.f : expf(e - mx) * inv;
      v = fmaf(w, a.part_acc[(base + s) * RANK + c], v);
    }
    o[c] = __float2bfloat16_rn(v);
  }
}

constexpr size_t kSmemLimit = 227 * 1024;

template <typename K>
static int opt_in(K kernel, size_t bytes) {
  if (bytes > kSmemLimit) return PE_ERR_UNSUPPORTED_SIZE;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

constexpr int kPrefillMB = 4, kPrefillMBSmall = 3, kPrefillKS = 2, kDecodeMB = 1, kDecodeKS = 4;

template <int RANK, int MB>
static int launch_prefill(const Args& a, const CUtensorMap& map, int n_seqs, int max_q, cudaStream_t stream) {
  auto k = latent_kernel<RANK, MB, kPrefillKS, false>;
  const size_t smem = smem_bytes<MB, kPrefillKS>(a.row);
  int e = opt_in(k, smem);
  if (e) return e;
  const long long tiles = ((long long)max_q * a.n_heads + MB * 16 - 1) / (MB * 16);
  if (tiles > 0x7fffffffLL || n_seqs > 65535) return PE_ERR_UNSUPPORTED_SIZE;
  pe::launch(k, dim3((unsigned)tiles, n_seqs), MB * kPrefillKS * 32, smem, stream, a, map);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

template <int RANK>
static int launch(const Args& a, const void* pages, bool decode, int n_seqs, int max_q, cudaStream_t stream) {
  CUtensorMap map;
  const int me = tma::make_map_2d_bf16(&map, pages, a.row, (uint64_t)a.num_pages * BN, a.row, 64, BN);
  if (me != 0) return me < 0 ? me : PE_ERR_BAD_ARGUMENT;
  if (!decode) {
    if (smem_bytes<kPrefillMB, kPrefillKS>(a.row) <= kSmemLimit) return launch_prefill<RANK, kPrefillMB>(a, map, n_seqs, max_q, stream);
    return launch_prefill<RANK, kPrefillMBSmall>(a, map, n_seqs, max_q, stream);
  }
  auto k = latent_kernel<RANK, kDecodeMB, kDecodeKS, true>;
  const size_t smem = smem_bytes<kDecodeMB, kDecodeKS>(a.row);
  int e = opt_in(k, smem);
  if (e) return e;
  const int head_blocks = (a.n_heads + 15) / 16;
  if (head_blocks > 65535 || n_seqs > 65535) return PE_ERR_UNSUPPORTED_SIZE;
  pe::launch(k, dim3(a.max_splits, head_blocks, n_seqs), kDecodeMB * kDecodeKS * 32, smem, stream, a, map);
  PE_LAUNCH_CHECK();
  pe::launch_after(latent_merge_kernel<RANK>, dim3(a.n_heads, n_seqs), 128, 0, stream, a);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

}  // namespace la
}  // namespace pe

// Whether these kernels take a cached row of `row` features whose leading `rank` are the values.
extern "C" int pe_attention_latent_supported(int row, int rank) {
  if (row <= 0 || row % 64 || rank > row) return 0;
  if (rank != 128 && rank != 256 && rank != 512) return 0;
  return pe::la::smem_bytes<pe::la::kPrefillMBSmall, pe::la::kPrefillKS>(row) <= pe::la::kSmemLimit ? 1 : 0;
}

// q: [n_tokens, n_heads * row] (row stride q_ld); out: [n_tokens, n_heads * rank] (row stride out_ld); pages:
// [num_pages, 64, row].  `decode` != 0: every sequence brings one token; scratch holds n_seqs * n_heads * max_splits *
// (rank + 1) floats; with split_keys 0 a sequence's keys are shared out evenly over max_splits ranges of whole pages,
// each of at least min_range_keys keys.
extern "C" int pe_attention_latent(int decode, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs, int max_q,
                                   int n_heads, int row, int rank, float scale, const int* seq_qstart, const int* seq_past,
                                   const int* seq_slot, const int* page_table, int table_stride, int num_pages,
                                   const void* pages, float* scratch, int split_keys, int max_splits, int min_range_keys,
                                   int* status, cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (n_heads <= 0 || !pe_attention_latent_supported(row, rank)) return PE_ERR_UNSUPPORTED_SIZE;
  // 16-byte vector loads of q rows, 4-byte stores of output pairs
  if ((q_ld * 2) % 16 || ((uintptr_t)q % 16) || (out_ld * 2) % 4 || ((uintptr_t)out % 4) || ((uintptr_t)pages % 16))
    return PE_ERR_BAD_ARGUMENT;
  pe::la::Args a;
  a.q = (const __nv_bfloat16*)q; a.q_ld = q_ld; a.out = (__nv_bfloat16*)out; a.out_ld = out_ld;
  a.n_heads = n_heads; a.row = row; a.scale_log2 = scale * 1.4426950408889634f;
  a.seq_qstart = seq_qstart; a.seq_past = seq_past; a.seq_slot = seq_slot;
  a.page_table = page_table; a.table_stride = table_stride; a.num_pages = num_pages; a.status = status;
  a.part_acc = nullptr; a.part_lse = nullptr; a.split_keys = 0; a.max_splits = 0; a.min_range_keys = 0;
  if (decode) {
    if (!scratch || ((uintptr_t)scratch % 8) || split_keys < 0 || split_keys % pe::la::BN || max_splits <= 0) return PE_ERR_BAD_ARGUMENT;
    if (min_range_keys < 0 || min_range_keys % pe::la::BN) return PE_ERR_BAD_ARGUMENT;
    a.split_keys = split_keys; a.max_splits = max_splits; a.min_range_keys = min_range_keys;
    a.part_acc = scratch;
    a.part_lse = scratch + (size_t)n_seqs * n_heads * max_splits * rank;
  }
  if (rank == 128) return pe::la::launch<128>(a, pages, decode != 0, n_seqs, max_q, stream);
  if (rank == 256) return pe::la::launch<256>(a, pages, decode != 0, n_seqs, max_q, stream);
  return pe::la::launch<512>(a, pages, decode != 0, n_seqs, max_q, stream);
}
