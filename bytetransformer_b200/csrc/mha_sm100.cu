// Fused variable-length multi-head attention for sm_100a (head size 64, fp16 in/out).
//
// Stands in for the reference's packed attention kernels
// (bytetransformer/src/attention_fused.cu:295-414 for short sequences,
// bytetransformer/src/attention_fused_long.cu:171-312 and the grouped-GEMM path
// of bytetransformer/src/cutlass_attention.cu:150-210 for long ones).  Two kernels:
//   mha_fwd_kernel         one CTA per (128 query rows, head, sequence), 192 threads, two CTAs per SM.
//                          Used while the longest sequence fits two key tiles' worth of work per item
//                          (max_len <= 192) and for the general-mask variant.
//   mha_persistent_kernel  persistent CTAs walking a static list of (sequence, query tile, head) items,
//                          256 threads, two CTAs per SM; everything longer.
// Both run an online softmax over 128-key tiles, so no S x S logits ever reach HBM and any length
// works.
//
// Input is the packed QKV activation [rows, 3H] with bias already added by the
// QKV GEMM epilogue; head h of Q/K/V is the 64-column slice at h*64 / H+h*64 /
// 2H+h*64, fetched straight from that buffer by TMA (the reference's separate
// bias-add + head-split transpose kernel, attention_nofused_utils.cu:142-184, has
// no counterpart here).  Only `batch_idx` tells where sequences start and end;
// as in the reference's packed kernels the mask tensor is not consulted again.
//
// Common to both kernels: one warp issues TMA loads, one thread issues the tcgen05 MMAs (and its warp
// owns the tensor-memory allocation), four softmax warps own one query row per thread.
//   S = Q K^T      128x128x64, both operands from shared memory -> tensor memory, 128 fp32 columns
//   P = 2^(c*S-m)  fp16 pairs written to tensor memory with tcgen05.st
//   O += P V       128x64x128 with the A operand (P) read from tensor memory and V
//                  consumed MN-major from shared memory exactly as it lies in the QKV
//                  buffer -> 64 fp32 columns
// P never touches shared memory.  O stays in tensor memory across key tiles.  The
// exponent reference m only moves when the running maximum grows by more than a
// threshold (then the O row is rescaled in tensor memory); otherwise P simply grows
// up to 2^threshold, which fp16 holds, and the final division by the row sum makes
// the result exact.
// Keys beyond the sequence end are masked by selection (never by arithmetic on
// the fetched values) and their V rows are zeroed in shared memory, so rows of
// neighbouring sequences or never-written workspace cannot leak in.
// Offsets that do not describe rows inside the allocation (negative, decreasing, longer than max_len,
// past the last row) make the sequence a no-op and set kStatusBadOffsets: nothing outside the
// buffers is read or written.
//
// What the measurements on B200 say about the softmax (it, not the tensor core, bounds both kernels:
// the MMAs of a 128x128 tile take ~540 clocks when two CTAs interleave them, a tile takes ~1900):
// the special-function unit delivers one warp-wide ex2 per 4 clocks and scheduler, but a single warp
// only reaches one per ~10 clocks (two warps 6.9, three 4.9), and tensor memory holds S, O and P for
// two CTAs, i.e. two softmax warps per scheduler.  Halving the exponential work (ex2.f16x2 runs at
// half rate, so it gains nothing; a polynomial on the FMA pipe for a quarter of the elements: 5 %
// slower), 256-row ping-pong tiles and two threads per row with an exchange through shared memory
// (25 % slower) were measured and dropped.
#include "common.cuh"
#include "kernels.h"

namespace bt {

namespace {

long long g_dbg_force_kernel = 0;  // 0 = by shape, 1 = one CTA per item, 3 = persistent

constexpr int kQRows = 128;
constexpr int kKvRows = 128;
constexpr int kHeadDim = 64;
constexpr int kTileBytes = 128 * kHeadDim * 2;  // 16 KiB: Q, K or V tile

// One CTA per item: shared-memory and tensor-memory layout.
struct MhaCfg {
  static constexpr int kStages = 3;
  static constexpr int kThreads = 192;
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemK = kSmemQ + kTileBytes;
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr int kSmemBar = kSmemV + kStages * kTileBytes;
  static constexpr int kSmemBytes = kSmemBar + 256;
  static constexpr int kTmemCols = 256;
  static constexpr uint32_t kTmemO = 128;    // the S tile first, then the O tile
  static constexpr uint32_t kTmemPOff = 64;  // P aliases columns 64..127 of S
};

struct MhaArgs {
  __half* ctx;
  const int* batch_idx;
  int hidden;
  float scale_log2e;
  int* status;
  int rows;     // rows allocated in qkv / ctx
  int max_len;  // upper bound of every sequence length
  // General-mask variant (GENERAL = true): every sequence has `gen_seq_len` rows; the score of
  // (query q, key k) gets  attn_bias[head, q, k] + (1 - mask[b, q, k]) * -10000  added after scaling,
  // the rule of the reference's unfused softmax (bytetransformer/include/softmax.h:41-45).
  const __half* gen_mask;  // [batch, S, S]
  const __half* gen_bias;  // [heads, S, S] or null
  int gen_seq_len;
  float gen_inv_scale;     // 1 / (softmax scale): the additive term is applied to the unscaled score
  const int* gen_kv_bound; // [batch, query tiles]: leading keys that matter for the query tile, or null
  // A binary mask without bias is applied from one bit per (query, key) instead (gen_bits, rows
  // `gen_bits_stride` words apart; usable when *gen_bits_flag == 0): the scores stay where they are
  const uint32_t* gen_bits;
  const int* gen_bits_flag;
  int gen_bits_stride;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Packed fp32 pairs (fma.rn.f32x2 / add.rn.f32x2 of sm_100: one issue slot for two values): the scale-and-shift
// in front of the exponentials and the row sums behind them take half the instructions.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  unpack_f32x2(fma_f32x2(pack_f32x2(a0, a1), pack_f32x2(b, b), pack_f32x2(c, c)), d0, d1);
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {
  unpack_f32x2(add_f32x2(pack_f32x2(d0, d1), pack_f32x2(a0, a1)), d0, d1);
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (P, fp16 pairs) is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Row maximum of S over the valid keys.  The next 32-column chunk is requested from
// tensor memory before the current one is reduced, so only the first load is exposed.
template <bool MASKED>
__device__ __forceinline__ float chunk_max(const uint32_t (&v)[32], int cbase, int kv_valid) {
  float m0 = -INFINITY, m1 = -INFINITY;
  if (MASKED) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      m0 = fmaxf(m0, (cbase + i < kv_valid) ? __uint_as_float(v[i]) : -INFINITY);
      m1 = fmaxf(m1, (cbase + i + 1 < kv_valid) ? __uint_as_float(v[i + 1]) : -INFINITY);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
    }
  }
  return fmaxf(m0, m1);
}
template <bool MASKED>
__device__ __forceinline__ float tile_row_max(uint32_t t_s, int kv_valid) {
  uint32_t va[32], vb[32];
  tmem_ld_32x32(t_s, va);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 32, vb);
  float mx = chunk_max<MASKED>(va, 0, kv_valid);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 64, va);
  mx = fmaxf(mx, chunk_max<MASKED>(vb, 32, kv_valid));
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 96, vb);
  mx = fmaxf(mx, chunk_max<MASKED>(va, 64, kv_valid));
  tmem_ld_wait();
  return fmaxf(mx, chunk_max<MASKED>(vb, 96, kv_valid));
}

// One 32-column chunk of S -> 16 cells of fp16 pairs, plus this chunk's row sum (2^x in fp32, one
// special-function op per key, fp32 row sum).
template <bool MASKED>
__device__ __forceinline__ float chunk_probs(const uint32_t (&v)[32], int cbase, int kv_valid, float c, float m_ref,
                                             uint32_t (&out)[16]) {
  float l0 = 0.f, l1 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float t0, t1;
    fma2(t0, t1, __uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]), c, -m_ref);
    float p0 = ex2_approx(t0);
    float p1 = ex2_approx(t1);
    if (MASKED) {
      p0 = (cbase + 2 * i < kv_valid) ? p0 : 0.f;
      p1 = (cbase + 2 * i + 1 < kv_valid) ? p1 : 0.f;
    }
    add2(l0, l1, p0, p1);
    out[i] = pack_half2(p0, p1);
  }
  return l0 + l1;
}

// Second pass over one S tile, from the last chunk to the first; P chunk c lands in cells
// [64 + 16c, 64 + 16c + 16) of the same tile, which lie in chunks that were already read.
template <bool MASKED>
__device__ __forceinline__ float tile_probs(uint32_t t_s, int kv_valid, float c, float m_ref) {
  const uint32_t t_p = t_s + 64;
  uint32_t va[32], vb[32], pk[16];
  float l = 0.f;
  tmem_ld_32x32(t_s + 96, va);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 64, vb);  // in flight while chunk 3 is processed
  l += chunk_probs<MASKED>(va, 96, kv_valid, c, m_ref, pk);
  tmem_ld_wait();               // chunk 2 is in registers: its cells may now be overwritten
  tmem_st_32x16(t_p + 48, pk);
  tmem_ld_32x32(t_s + 32, va);
  l += chunk_probs<MASKED>(vb, 64, kv_valid, c, m_ref, pk);
  tmem_ld_wait();
  tmem_st_32x16(t_p + 32, pk);
  tmem_ld_32x32(t_s, vb);
  l += chunk_probs<MASKED>(va, 32, kv_valid, c, m_ref, pk);
  tmem_ld_wait();
  tmem_st_32x16(t_p + 16, pk);
  l += chunk_probs<MASKED>(vb, 0, kv_valid, c, m_ref, pk);
  tmem_st_32x16(t_p, pk);
  tmem_st_wait();
  return l;
}

// Binary mask from bits: a key whose bit is clear has `neg` (= -10000 / scale) added to its score, exactly
// what the additive form below does for mask values 0 and 1, without a pass over S.  `w` holds the bits of
// the chunk's 32 keys.
template <bool MASKED>
__device__ __forceinline__ float chunk_max_bits(const uint32_t (&v)[32], int cbase, int kv_valid, uint32_t w, float neg) {
  float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float a = __uint_as_float(v[i]), b = __uint_as_float(v[i + 1]);
    a = ((w >> i) & 1u) ? a : a + neg;
    b = ((w >> (i + 1)) & 1u) ? b : b + neg;
    if (MASKED) {
      a = (cbase + i < kv_valid) ? a : -INFINITY;
      b = (cbase + i + 1 < kv_valid) ? b : -INFINITY;
    }
    m0 = fmaxf(m0, a);
    m1 = fmaxf(m1, b);
  }
  return fmaxf(m0, m1);
}
template <bool MASKED>
__device__ __forceinline__ float tile_row_max_bits(uint32_t t_s, int kv_valid, const uint4& bw, float neg) {
  uint32_t va[32], vb[32];
  tmem_ld_32x32(t_s, va);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 32, vb);
  float mx = chunk_max_bits<MASKED>(va, 0, kv_valid, bw.x, neg);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 64, va);
  mx = fmaxf(mx, chunk_max_bits<MASKED>(vb, 32, kv_valid, bw.y, neg));
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 96, vb);
  mx = fmaxf(mx, chunk_max_bits<MASKED>(va, 64, kv_valid, bw.z, neg));
  tmem_ld_wait();
  return fmaxf(mx, chunk_max_bits<MASKED>(vb, 96, kv_valid, bw.w, neg));
}
template <bool MASKED>
__device__ __forceinline__ float chunk_probs_bits(const uint32_t (&v)[32], int cbase, int kv_valid, float c, float m_ref,
                                                  uint32_t w, float neg, uint32_t (&out)[16]) {
  float l0 = 0.f, l1 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float a = __uint_as_float(v[2 * i]), b = __uint_as_float(v[2 * i + 1]);
    a = ((w >> (2 * i)) & 1u) ? a : a + neg;
    b = ((w >> (2 * i + 1)) & 1u) ? b : b + neg;
    float t0, t1;
    fma2(t0, t1, a, b, c, -m_ref);
    float p0 = ex2_approx(t0);
    float p1 = ex2_approx(t1);
    if (MASKED) {
      p0 = (cbase + 2 * i < kv_valid) ? p0 : 0.f;
      p1 = (cbase + 2 * i + 1 < kv_valid) ? p1 : 0.f;
    }
    add2(l0, l1, p0, p1);
    out[i] = pack_half2(p0, p1);
  }
  return l0 + l1;
}
template <bool MASKED>
__device__ __forceinline__ float tile_probs_bits(uint32_t t_s, int kv_valid, float c, float m_ref, const uint4& bw,
                                                 float neg) {
  const uint32_t t_p = t_s + 64;
  uint32_t va[32], vb[32], pk[16];
  float l = 0.f;
  tmem_ld_32x32(t_s + 96, va);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 64, vb);
  l += chunk_probs_bits<MASKED>(va, 96, kv_valid, c, m_ref, bw.w, neg, pk);
  tmem_ld_wait();
  tmem_st_32x16(t_p + 48, pk);
  tmem_ld_32x32(t_s + 32, va);
  l += chunk_probs_bits<MASKED>(vb, 64, kv_valid, c, m_ref, bw.z, neg, pk);
  tmem_ld_wait();
  tmem_st_32x16(t_p + 32, pk);
  tmem_ld_32x32(t_s, vb);
  l += chunk_probs_bits<MASKED>(va, 32, kv_valid, c, m_ref, bw.y, neg, pk);
  tmem_ld_wait();
  tmem_st_32x16(t_p + 16, pk);
  l += chunk_probs_bits<MASKED>(vb, 0, kv_valid, c, m_ref, bw.x, neg, pk);
  tmem_st_32x16(t_p, pk);
  tmem_st_wait();
  return l;
}

// General-mask variant: S(q, k) += (attn_bias[h,q,k] - 10000 * (1 - mask[b,q,k])) / scale for the 128
// keys of this tile, in tensor memory, before the two softmax passes read it.  `mrow` / `brow`
// point at (q, first key of the tile); `n_keys` keys exist from there on (the others are
// dropped later by the key-count mask); `vec` says that 16-byte loads are aligned.  The
// tensor-memory loads and stores are warp-wide instructions: every lane of the warp must call
// this function, lanes whose query row does not exist pass n_keys = 0 and add nothing.
__device__ __forceinline__ void tile_add_mask_bias(uint32_t t_s, const __half* mrow, const __half* brow, int n_keys,
                                                   bool vec, float inv_scale) {
#pragma unroll 1
  for (int cb = 0; cb < kKvRows; cb += 32) {
    uint32_t v[32];
    tmem_ld_32x32(t_s + cb, v);
    float add[32];
    if (vec && cb + 32 <= n_keys) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 m4 = __ldg(reinterpret_cast<const uint4*>(mrow + cb) + q);
        const __half2* mh = reinterpret_cast<const __half2*>(&m4);
        uint4 b4 = make_uint4(0u, 0u, 0u, 0u);
        if (brow != nullptr) b4 = __ldg(reinterpret_cast<const uint4*>(brow + cb) + q);
        const __half2* bh = reinterpret_cast<const __half2*>(&b4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fm = __half22float2(mh[j]);
          const float2 fb = __half22float2(bh[j]);
          add[q * 8 + 2 * j] = fb.x - 10000.0f * (1.0f - fm.x);
          add[q * 8 + 2 * j + 1] = fb.y - 10000.0f * (1.0f - fm.y);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float a = 0.f;
        if (cb + i < n_keys) {
          a = -10000.0f * (1.0f - __half2float(__ldg(mrow + cb + i)));
          if (brow != nullptr) a += __half2float(__ldg(brow + cb + i));
        }
        add[i] = a;
      }
    }
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(fmaf(add[i], inv_scale, __uint_as_float(v[i])));
    tmem_st_32x32(t_s + cb, v);
  }
  tmem_st_wait();
}

template <bool GENERAL>
__global__ void __launch_bounds__(MhaCfg::kThreads, 2)
mha_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const MhaArgs args) {
  using Cfg = MhaCfg;
  constexpr int TILES = 1;  // query tiles per CTA (the loops over `t` below have one trip)
  constexpr int kStages = Cfg::kStages;
  // the exponent reference may lag the running maximum by at most 2^8
  constexpr float kRescaleThreshold = 8.0f;
  extern __shared__ __align__(1024) uint8_t smem[];

  pdl_launch_dependents();
  pdl_wait();  // batch_idx and the QKV buffer come from earlier kernels
  const int b = blockIdx.z;
  const int head = blockIdx.y;
  const int seq_start = __ldg(args.batch_idx + b);
  const int L = __ldg(args.batch_idx + b + 1) - seq_start;
  const int q0 = blockIdx.x * (kQRows * TILES);
  if (seq_start < 0 || L < 0 || L > args.max_len || seq_start > args.rows - L) {
    // offsets that do not describe rows of the allocation: nothing is read or written for this sequence
    if (threadIdx.x == 0 && args.status != nullptr) atomicCAS(args.status, 0, kStatusBadOffsets);
    return;
  }
  if (q0 >= L) return;  // whole CTA leaves before any barrier / allocation exists
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && args.status != nullptr) atomicCAS(args.status, 0, kStatusMhaLoadTimeout + 0x10);
    return;
  }
  const int n_tiles = (TILES == 2 && q0 + kQRows < L) ? 2 : 1;  // query tiles with at least one valid row

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kSmemBar);
  uint64_t* q_full = bars;                       // [TILES]
  uint64_t* k_full = bars + 2;                   // [kStages]
  uint64_t* v_full = bars + 2 + kStages;         // [kStages]
  uint64_t* kv_empty = bars + 2 + 2 * kStages;   // [kStages]
  uint64_t* s_full = bars + 2 + 3 * kStages;     // [TILES]
  uint64_t* p_full = bars + 4 + 3 * kStages;     // [TILES]
  uint64_t* o_done = bars + 6 + 3 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7 + 3 * kStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // General masks: the key tiles behind the last key that any row of this query tile may see are left out
  int kv_rows = L;
  if (GENERAL && args.gen_kv_bound != nullptr) {
    const int bound = __ldg(args.gen_kv_bound + b * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x));
    kv_rows = bound < L ? (bound > 0 ? bound : 1) : L;
  }
  const int n_kv = (kv_rows + kKvRows - 1) / kKvRows;

  if (threadIdx.x == 0) {
    for (int t = 0; t < TILES; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int col_q = head * kHeadDim;
  const int col_k = args.hidden + head * kHeadDim;
  const int col_v = 2 * args.hidden + head * kHeadDim;

  if (warp == 0) {
    // ------------------------------------------------------------------ loads
    if (lane == 0) {
      tma_prefetch_desc(&tm_qkv);
      for (int t = 0; t < n_tiles; ++t) {
        mbar_arrive_expect_tx(&q_full[t], kTileBytes);
        tma_load_2d(smem + Cfg::kSmemQ + t * kTileBytes, &tm_qkv, &q_full[t], col_q, seq_start + q0 + t * kQRows);
      }
      int stage = 0;
      uint32_t phase = 0;
      for (int j = 0; j < n_kv; ++j) {
        if (!mbar_wait_bounded(&kv_empty[stage], phase ^ 1u, abort_flag, args.status, kStatusMhaLoadTimeout)) break;
        const int row = seq_start + j * kKvRows;
        mbar_arrive_expect_tx(&k_full[stage], kTileBytes);
        tma_load_2d(smem + Cfg::kSmemK + stage * kTileBytes, &tm_qkv, &k_full[stage], col_k, row);
        mbar_arrive_expect_tx(&v_full[stage], kTileBytes);
        tma_load_2d(smem + Cfg::kSmemV + stage * kTileBytes, &tm_qkv, &v_full[stage], col_v, row);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issue
    if (lane == 0) {
      // K-major operands (Q, K): 8-row groups 1024 B apart.
      constexpr uint64_t kDescK = make_smem_desc_hi(16, 1024);
      // V: MN-major, one 64-wide chunk (LBO unused), 8-key groups 1024 B apart.
      constexpr uint64_t kDescV = make_smem_desc_hi(kTileBytes, 1024);
      constexpr uint32_t kIdescS = make_idesc_f16(128, 128, 0, 0);
      constexpr uint32_t kIdescO = make_idesc_f16(128, 64, 0, 1);
      const uint32_t s_q = smem_u32(smem + Cfg::kSmemQ);
      const uint32_t s_k = smem_u32(smem + Cfg::kSmemK);
      const uint32_t s_v = smem_u32(smem + Cfg::kSmemV);
      auto issue_s = [&](int t, int stage) {
        const uint32_t sq = s_q + t * kTileBytes;
        const uint32_t sk = s_k + stage * kTileBytes;
#pragma unroll
        for (int k = 0; k < kHeadDim / 16; ++k)
          umma_f16_ss(tmem_base + t * 128, smem_desc(kDescK, sq + k * 32), smem_desc(kDescK, sk + k * 32), kIdescS,
                      k != 0 ? 1u : 0u);
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t tp = tmem_base + t * 128 + Cfg::kTmemPOff;  // 8 cells (16 keys) per MMA
        const uint32_t sv = s_v + stage * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kKvRows / 16; ++kk)
          umma_f16_ts(tmem_base + Cfg::kTmemO + t * 64, tp + kk * 8, smem_desc(kDescV, sv + kk * 2048), kIdescO,
                      (accumulate || kk != 0) ? 1u : 0u);
      };
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t)
        ok = mbar_wait_bounded(&q_full[t], 0, abort_flag, args.status, kStatusMhaMmaTimeout);
      if (ok) ok = mbar_wait_bounded(&k_full[0], 0, abort_flag, args.status, kStatusMhaMmaTimeout);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < n_tiles; ++t) issue_s(t, 0);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t jpar = j & 1;
        const int st_n = (st + 1 == kStages) ? 0 : st + 1;
        const uint32_t ph_n = (st + 1 == kStages) ? (ph ^ 1u) : ph;
        const bool more = j + 1 < n_kv;
        // ---- tile 0: O0 += P0 V(j), then S0(j+1).  The MMAs of one thread execute in issue
        // order, so S0(j+1) cannot overwrite P0(j) (same columns) before PV0(j) has read it.
        if (!mbar_wait_bounded(&p_full[0], jpar, abort_flag, args.status, kStatusMhaMmaTimeout)) break;
        if (!mbar_wait_bounded(&v_full[st], ph, abort_flag, args.status, kStatusMhaMmaTimeout)) break;
        tc_fence_after();
        issue_pv(0, st, j > 0);
        if (more) {
          if (!mbar_wait_bounded(&k_full[st_n], ph_n, abort_flag, args.status, kStatusMhaMmaTimeout)) break;
          tc_fence_after();
          issue_s(0, st_n);
        }
        // ---- tile 1
        if (n_tiles == 2) {
          if (!mbar_wait_bounded(&p_full[1], jpar, abort_flag, args.status, kStatusMhaMmaTimeout)) break;
          tc_fence_after();
          issue_pv(1, st, j > 0);
        }
        umma_commit(&kv_empty[st]);  // every MMA that reads K/V stage `st` has been issued
        if (n_tiles == 2 && more) issue_s(1, st_n);
        st = st_n;
        ph = ph_n;
      }
      umma_commit(o_done);
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int t = (warp - 2) >> 2;  // query tile of this warpgroup
    if (t < n_tiles) {
      const int quarter = warp & 3;
      const int r = quarter * 32 + lane;  // query row inside the tile == TMEM lane
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t t_s = t_lane + t * 128;
      const uint32_t t_o = t_lane + Cfg::kTmemO + t * 64;
      const float c = args.scale_log2e;
      float m_ref = -INFINITY;  // exponent reference, in log2 units
      float l_run = 0.f;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // binary mask, no bias: applied from bits inside the two softmax passes
      const bool use_bits = GENERAL && args.gen_bits != nullptr && __ldg(args.gen_bits_flag) == 0;
      const float bits_neg = -10000.0f * args.gen_inv_scale;
      for (int j = 0; j < n_kv; ++j) {
        const uint32_t jpar = j & 1;
        const int kv_valid = min(kKvRows, L - j * kKvRows);
        const bool full_tile = kv_valid == kKvRows;
        if (!mbar_wait_bounded(&s_full[t], jpar, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint4 bw = make_uint4(~0u, ~0u, ~0u, ~0u);  // a row that does not exist masks nothing
        if (GENERAL && use_bits) {
          const int q_row = q0 + t * kQRows + r;
          if (q_row < args.gen_seq_len)
            bw = __ldg(reinterpret_cast<const uint4*>(args.gen_bits + (static_cast<size_t>(b) * args.gen_seq_len + q_row) *
                                                                          args.gen_bits_stride) + j);
        } else if (GENERAL) {
          const int S = args.gen_seq_len;
          const int q_row = q0 + t * kQRows + r;
          const bool q_ok = q_row < S;
          const size_t off = static_cast<size_t>(q_ok ? q_row : 0) * S + static_cast<size_t>(j) * kKvRows;
          tile_add_mask_bias(t_s, args.gen_mask + static_cast<size_t>(b) * S * S + off,
                             args.gen_bias != nullptr ? args.gen_bias + static_cast<size_t>(head) * S * S + off : nullptr,
                             q_ok ? kv_valid : 0, (S & 7) == 0, args.gen_inv_scale);
        }
        // pass 1: row maximum (scaled to log2 units)
        float mx;
        if (GENERAL && use_bits)
          mx = c * (full_tile ? tile_row_max_bits<false>(t_s, kv_valid, bw, bits_neg)
                              : tile_row_max_bits<true>(t_s, kv_valid, bw, bits_neg));
        else
          mx = c * (full_tile ? tile_row_max<false>(t_s, kv_valid) : tile_row_max<true>(t_s, kv_valid));
        if (j == 0) {
          m_ref = mx;
        } else {
          const float m_new = fmaxf(m_ref, mx);
          const bool need = (m_new - m_ref) > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            // the PV of the previous key tile has retired (S of this tile was issued after it)
            const float f = ex2_approx(m_ref - m_new);
#pragma unroll
            for (int cb = 0; cb < kHeadDim; cb += 32) {
              uint32_t v[32];
              tmem_ld_32x32(t_o + cb, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
              tmem_st_32x32(t_o + cb, v);
            }
            l_run *= f;
            m_ref = m_new;
          }
        }
        // pass 2: probabilities -> fp16 pairs -> tensor memory (over S), row sum
        if (GENERAL && use_bits)
          l_run += full_tile ? tile_probs_bits<false>(t_s, kv_valid, c, m_ref, bw, bits_neg)
                             : tile_probs_bits<true>(t_s, kv_valid, c, m_ref, bw, bits_neg);
        else
          l_run += full_tile ? tile_probs<false>(t_s, kv_valid, c, m_ref)
                             : tile_probs<true>(t_s, kv_valid, c, m_ref);
        if (!full_tile && t == 0) {
          // tail tile: blank the V rows of keys that do not belong to this sequence
          // (tile 0's PV is issued before tile 1's, so tile 0's warpgroup does it for both)
          if (!mbar_wait_bounded(&v_full[stage], phase, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
            ok = false;
            break;
          }
          if (r >= kv_valid) {
            uint4* vr = reinterpret_cast<uint4*>(smem + Cfg::kSmemV + stage * kTileBytes + r * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) vr[i] = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async_smem();
        }
        tc_fence_before();
        mbar_arrive(&p_full[t]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) ok = mbar_wait_bounded(o_done, 0, abort_flag, args.status, kStatusMhaSoftmaxTimeout);
      tc_fence_after();
      if (ok) {
        const int q_row = q0 + t * kQRows + r;
        const float inv = 1.0f / l_run;
        uint4* dst = reinterpret_cast<uint4*>(args.ctx + static_cast<size_t>(seq_start + q_row) * args.hidden +
                                              head * kHeadDim);
#pragma unroll
        for (int cb = 0; cb < kHeadDim; cb += 32) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + cb, v);
          tmem_ld_wait();
          if (q_row < L) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 w;
              w.x = pack_half2(__uint_as_float(v[u * 8 + 0]) * inv, __uint_as_float(v[u * 8 + 1]) * inv);
              w.y = pack_half2(__uint_as_float(v[u * 8 + 2]) * inv, __uint_as_float(v[u * 8 + 3]) * inv);
              w.z = pack_half2(__uint_as_float(v[u * 8 + 4]) * inv, __uint_as_float(v[u * 8 + 5]) * inv);
              w.w = pack_half2(__uint_as_float(v[u * 8 + 6]) * inv, __uint_as_float(v[u * 8 + 7]) * inv);
              dst[(cb >> 3) + u] = w;
            }
          }
        }
      }
      tc_fence_before();
    }
  }

  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// Persistent kernel: each CTA (256 threads, two per SM) walks a static list of work items
// (sequence, 128-row query tile, head).  Barriers, tensor memory and the launch are paid once per
// CTA instead of once per item, and the loader runs ahead: the next item's Q/K/V tiles are requested
// while the current item's last key tiles are still being processed.
//
// Tensor memory: S columns 0..127, O 128..191, P 192..255 (P has its own columns, so S is never
// overwritten by P).  A softmax thread reads its whole row of S (128 fp32 values) into registers in one
// go and at once hands S back (`s_free`): the tensor core forms S(j+1) = Q K(j+1)^T while the
// exponentials of tile j are still being computed, so the MMA round trip (commit, issue, four MMAs,
// commit) is off the softmax warps' critical path.  With the row in registers the row maximum is exact
// before the first exponential, and all 128 exponentials are formed before P is touched, by which time
// the P V MMAs of the previous key tile (the owners of P and O until they retire) are long done.
// From the first load of S to the last store of P the code is one straight line: keys that do not
// exist in a sequence's last tile are set to -inf beforehand (probability 0) rather than skipped,
// because a branch per 32-key chunk cost more (the scheduler cannot overlap across it) than the
// exponentials it saved.
//
// Warps 0-3 softmax (one warpgroup, 216 registers each after setmaxnreg), warp 4 loads, warp 5 issues
// the MMAs, warps 6-7 only give their registers away (setmaxnreg works on whole warpgroups).  The two
// single-thread roles sleep between polls of a barrier so that they leave the issue slots of the
// schedulers they share with softmax warps alone.
//
// Items go to the CTAs in snake order (round k: item k*G + c for even k, k*G + G-1-c for odd k, G CTAs):
// with sequences sorted by length (longest first), which is how callers batch them, the items of a round
// get cheaper from first to last, and the snake evens out the per-CTA sums.
// ------------------------------------------------------------------------------------------
struct MhaPersistentArgs {
  __half* ctx;
  const int* batch_idx;
  int batch;
  int heads;
  int hidden;
  float scale_log2e;
  int* status;
  int rows;     // rows allocated in qkv / ctx
  int max_len;  // upper bound of every sequence length
  int tma_out;  // the kernel's second tensor map describes ctx: whole 32-row output slabs leave by bulk store
};

// Finds item n = (sequence b, query tile qt, head h); items are numbered sequence by sequence, inside
// a sequence query tile by query tile, heads fastest.  Called by all 32 lanes of a warp together: the
// lanes look at 32 sequences at a time (one coalesced read of their offsets, a warp scan of their item
// counts), because a loop over single sequences pays one L2 round trip per sequence, which with many
// short sequences cost more than the attention itself.  `cur_b` / `cur_first` is the caller's cursor
// (first item index of sequence cur_b, the same in all lanes); n never decreases.  A sequence whose
// offsets are not 0 <= start, 0 <= L <= max_len, start + L <= rows is left out (it yields no items, so
// nothing is read or written outside the buffers) and, when `report` is set (one warp per CTA),
// kStatusBadOffsets is recorded.
__device__ __forceinline__ bool decode_item(const MhaPersistentArgs& a, int n, int& cur_b, int& cur_first,
                                            int& seq_start, int& L, int& qt, int& h, bool report) {
  const int lane = static_cast<int>(threadIdx.x & 31u);
  while (cur_b < a.batch) {
    const int b = cur_b + lane;
    int start = 0, len = 0;
    if (b < a.batch) {
      start = __ldg(a.batch_idx + b);
      len = __ldg(a.batch_idx + b + 1) - start;
      if (start < 0 || len < 0 || len > a.max_len || start > a.rows - len) {
        if (report && a.status != nullptr) atomicCAS(a.status, 0, kStatusBadOffsets);
        len = 0;
      }
    }
    const int items = ((len + kQRows - 1) / kQRows) * a.heads;
    int incl = items;  // inclusive prefix sum over the 32 sequences
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    const unsigned found = __ballot_sync(0xffffffffu, b < a.batch && n < cur_first + incl);
    if (found != 0u) {
      const int src = __ffs(found) - 1;
      seq_start = __shfl_sync(0xffffffffu, start, src);
      L = __shfl_sync(0xffffffffu, len, src);
      cur_first += __shfl_sync(0xffffffffu, incl - items, src);
      cur_b += src;
      const int r = n - cur_first;
      qt = r / a.heads;
      h = r - qt * a.heads;
      return true;
    }
    cur_first += __shfl_sync(0xffffffffu, incl, 31);
    cur_b += 32;
  }
  return false;
}
__device__ __forceinline__ int snake_item(int round, int cta, int ctas) {
  return round * ctas + ((round & 1) ? ctas - 1 - cta : cta);
}

template <int B>
__device__ __forceinline__ void tmem_st_32x16_at(uint32_t taddr, const uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[B + 0]), "r"(r[B + 1]), "r"(r[B + 2]), "r"(r[B + 3]), "r"(r[B + 4]), "r"(r[B + 5]), "r"(r[B + 6]), "r"(r[B + 7]),
      "r"(r[B + 8]), "r"(r[B + 9]), "r"(r[B + 10]), "r"(r[B + 11]), "r"(r[B + 12]), "r"(r[B + 13]), "r"(r[B + 14]),
      "r"(r[B + 15])
      : "memory");
}
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// Bounded wait for the single-thread roles (loader, MMA issuer): between polls the thread sleeps, so that
// its polling does not take issue slots from the softmax warp that shares its scheduler.
__device__ __forceinline__ bool mbar_wait_role(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t polls = 0;
  while (true) {
    __nanosleep(40);
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 63u) == 0u) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > (1ll << 31)) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

constexpr int kPersistentThreads = 256;
constexpr int kPersistentStages = 2;  // Q, K and V tiles each
// Q, K, V rings, the softmax warps' output staging (4 x 32 rows x 128 B), barriers
constexpr int kPersistentSmemBytes = 3 * kPersistentStages * kTileBytes + kTileBytes + 256;

__global__ void __launch_bounds__(kPersistentThreads, 2)
mha_persistent_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_ctx,
                      const MhaPersistentArgs args) {
  constexpr int kStages = kPersistentStages;
  constexpr int kSmemQ = 0;
  constexpr int kSmemK = kSmemQ + kStages * kTileBytes;
  constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  constexpr int kSmemOut = kSmemV + kStages * kTileBytes;
  constexpr int kSmemBar = kSmemOut + kTileBytes;
  constexpr uint32_t kTmemS = 0, kTmemO = 128, kTmemP = 192;
  constexpr float kRescaleThreshold = 8.0f;
  extern __shared__ __align__(1024) uint8_t smem[];

  pdl_launch_dependents();
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBar);
  uint64_t* q_full = bars;                     // [kStages] by item
  uint64_t* q_empty = bars + kStages;          // [kStages] the item's last Q K^T has retired
  uint64_t* k_full = bars + 2 * kStages;       // [kStages] by key-tile step
  uint64_t* k_empty = bars + 3 * kStages;      // [kStages] the Q K^T that read the stage has retired
  uint64_t* v_full = bars + 4 * kStages;       // [kStages] by key-tile step
  uint64_t* v_empty = bars + 5 * kStages;      // [kStages] the P V that read the stage has retired
  uint64_t* s_full = bars + 6 * kStages;       // S(j) is in tensor memory
  uint64_t* s_free = s_full + 1;               // the softmax warps hold S(j) in registers (4 arrivals)
  uint64_t* p_full = s_full + 2;               // P(j) is in tensor memory, V rows blanked (4 arrivals)
  uint64_t* pv_done = s_full + 3;              // O += P(j) V(j) has retired
  uint64_t* o_done = s_full + 4;               // the item's last P V has retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool smem_ok = (smem_u32(smem) & 1023u) == 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 4);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    mbar_init(o_done, 1);
    *abort_flag = smem_ok ? 0 : 1;
    fence_mbar_init();
    if (!smem_ok && args.status != nullptr) atomicCAS(args.status, 0, kStatusMhaLoadTimeout + 0x10);
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // batch_idx and the QKV buffer come from earlier kernels

  const int G = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  int cur_b = 0, cur_first = 0, seq_start = 0, L = 0, qt = 0, head = 0;

  if (warp >= 4) {
    setmaxnreg_dec<40>();
    if (!smem_ok) {
      // fall through to the teardown
    } else if (warp == 4) {
      // ------------------------------------------------------------------ loads
      // (the whole warp finds the items, lane 0 does the rest)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int round = 0; ok && decode_item(args, snake_item(round, cta, G), cur_b, cur_first, seq_start, L, qt, head, true);
           ++round) {
        if (lane == 0) {
          const int n_kv = (L + kKvRows - 1) / kKvRows;
          const int qb = round % kStages;
          const uint32_t qph = static_cast<uint32_t>(round / kStages) & 1u;
          ok = mbar_wait_role(&q_empty[qb], qph ^ 1u, abort_flag, args.status, kStatusMhaLoadTimeout);
          if (ok) {
          mbar_arrive_expect_tx(&q_full[qb], kTileBytes);
          tma_load_2d(smem + kSmemQ + qb * kTileBytes, &tm_qkv, &q_full[qb], head * kHeadDim, seq_start + qt * kQRows);
          for (int j = 0; j < n_kv; ++j) {
            const int row = seq_start + j * kKvRows;
            if (!mbar_wait_role(&k_empty[stage], phase ^ 1u, abort_flag, args.status, kStatusMhaLoadTimeout)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&k_full[stage], kTileBytes);
            tma_load_2d(smem + kSmemK + stage * kTileBytes, &tm_qkv, &k_full[stage], args.hidden + head * kHeadDim, row);
            if (!mbar_wait_role(&v_empty[stage], phase ^ 1u, abort_flag, args.status, kStatusMhaLoadTimeout)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&v_full[stage], kTileBytes);
            tma_load_2d(smem + kSmemV + stage * kTileBytes, &tm_qkv, &v_full[stage], 2 * args.hidden + head * kHeadDim,
                        row);
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    } else if (warp == 5) {
      // -------------------------------------------------------------- MMA issue
      // (the whole warp finds the items, lane 0 does the rest)
      constexpr uint64_t kDescK = make_smem_desc_hi(16, 1024);
      constexpr uint64_t kDescV = make_smem_desc_hi(kTileBytes, 1024);
      constexpr uint32_t kIdescS = make_idesc_f16(128, 128, 0, 0);
      constexpr uint32_t kIdescO = make_idesc_f16(128, 64, 0, 1);
      const uint32_t s_q0 = smem_u32(smem + kSmemQ);
      const uint32_t s_k = smem_u32(smem + kSmemK);
      const uint32_t s_v = smem_u32(smem + kSmemV);
      // S = Q(item `round`) K(stage)^T
      auto issue_s = [&](int round, int stage) {
        const uint32_t s_q = s_q0 + (round % kStages) * kTileBytes;
        const uint32_t sk = s_k + stage * kTileBytes;
#pragma unroll
        for (int k = 0; k < kHeadDim / 16; ++k)
          umma_f16_ss(tmem_base + kTmemS, smem_desc(kDescK, s_q + k * 32), smem_desc(kDescK, sk + k * 32), kIdescS,
                      k != 0 ? 1u : 0u);
        umma_commit(s_full);
        umma_commit(&k_empty[stage]);
      };
      // the item's Q tile is free once its last Q K^T has been issued (and, by the commit, has retired)
      auto release_q = [&](int round) { umma_commit(&q_empty[round % kStages]); };
      auto q_ready = [&](int round) { return static_cast<uint32_t>(round / kStages) & 1u; };
      int st = 0;
      uint32_t ph = 0;
      uint32_t step = 0;
      // The first S = Q K^T of an item whose predecessor could not issue it ahead (lane 0).
      auto issue_first_s = [&](int round, int len) -> bool {
        // S(0) overwrites the S columns: the softmax warps must hold the previous item's last S in registers
        if (step > 0 && !mbar_wait_role(s_free, (step - 1u) & 1u, abort_flag, args.status, kStatusMhaMmaTimeout)) return false;
        if (!mbar_wait_role(&q_full[round % kStages], q_ready(round), abort_flag, args.status, kStatusMhaMmaTimeout)) return false;
        if (!mbar_wait_role(&k_full[st], ph, abort_flag, args.status, kStatusMhaMmaTimeout)) return false;
        tc_fence_after();
        issue_s(round, st);
        if (len <= kKvRows) release_q(round);  // the item's last (only) QK^T has been issued
        return true;
      };
      // Everything else of an item (lane 0): per key tile the NEXT S as soon as the softmax warps hold the
      // current one in registers, then O += P V.  On the item's last tile the next S is the first of the
      // CTA's next item, if its Q and K tiles have landed by then (`next_s_issued`): an item boundary then
      // costs the softmax warps no S round trip.  false when a wait gave up.
      auto issue_rest = [&](int round, int len, bool have_next, int len_next, bool& next_s_issued) -> bool {
        const int n_kv = (len + kKvRows - 1) / kKvRows;
        next_s_issued = false;
        for (int j = 0; j < n_kv; ++j, ++step) {
          const int st_n = (st + 1 == kStages) ? 0 : st + 1;
          const uint32_t ph_n = (st + 1 == kStages) ? (ph ^ 1u) : ph;
          if (j + 1 < n_kv) {
            // S(j) sits in the softmax warps' registers: S(j+1) goes now, long before P(j) is ready
            if (!mbar_wait_role(s_free, step & 1u, abort_flag, args.status, kStatusMhaMmaTimeout) ||
                !mbar_wait_role(&k_full[st_n], ph_n, abort_flag, args.status, kStatusMhaMmaTimeout))
              return false;
            tc_fence_after();
            issue_s(round, st_n);
            if (j + 2 == n_kv) release_q(round);
          } else if (have_next) {
            if (!mbar_wait_role(s_free, step & 1u, abort_flag, args.status, kStatusMhaMmaTimeout)) return false;
            if (mbar_test_wait(&q_full[(round + 1) % kStages], q_ready(round + 1)) && mbar_test_wait(&k_full[st_n], ph_n)) {
              tc_fence_after();
              issue_s(round + 1, st_n);
              if (len_next <= kKvRows) release_q(round + 1);
              next_s_issued = true;
            }
          }
          // P(j) is ready; this also tells that the softmax warps have finished the previous item's O
          // read-out, so the first P V of an item may overwrite O.
          if (!mbar_wait_role(p_full, step & 1u, abort_flag, args.status, kStatusMhaMmaTimeout) ||
              !mbar_wait_role(&v_full[st], ph, abort_flag, args.status, kStatusMhaMmaTimeout))
            return false;
          tc_fence_after();
          const uint32_t sv = s_v + st * kTileBytes;
          // only the 16-key steps that hold keys of this sequence
          const int kk_n = (min(kKvRows, len - j * kKvRows) + 15) >> 4;
#pragma unroll
          for (int kk = 0; kk < kKvRows / 16; ++kk)
            if (kk < kk_n)
              umma_f16_ts(tmem_base + kTmemO, tmem_base + kTmemP + kk * 8, smem_desc(kDescV, sv + kk * 2048), kIdescO,
                          (j > 0 || kk != 0) ? 1u : 0u);
          umma_commit(pv_done);
          umma_commit(&v_empty[st]);
          st = st_n;
          ph = ph_n;
        }
        umma_commit(o_done);
        return true;
      };
      bool ok = true;
      bool have = decode_item(args, snake_item(0, cta, G), cur_b, cur_first, seq_start, L, qt, head, false);
      int len = L;
      bool s_issued = false;  // S(0) of the item about to start has been issued already
      for (int round = 0; ok && have; ++round) {
        if (lane == 0 && !s_issued) ok = issue_first_s(round, len);
        // the item after this one is found while this item's first tile is on its way
        const bool have_next = decode_item(args, snake_item(round + 1, cta, G), cur_b, cur_first, seq_start, L, qt, head, false);
        const int len_next = L;
        bool next_s_issued = false;
        if (lane == 0 && ok) ok = issue_rest(round, len, have_next, len_next, next_s_issued);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        s_issued = __shfl_sync(0xffffffffu, next_s_issued ? 1 : 0, 0) != 0;
        have = have_next;
        len = len_next;
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax (warps 0..3)
    setmaxnreg_inc<216>();
    const int r = warp * 32 + lane;  // query row inside the tile == TMEM lane
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const uint32_t t_s = t_lane + kTmemS;
    const uint32_t t_o = t_lane + kTmemO;
    const uint32_t t_p = t_lane + kTmemP;
    const float c = args.scale_log2e;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t step = 0;
    bool ok = smem_ok;
    bool have = decode_item(args, snake_item(0, cta, G), cur_b, cur_first, seq_start, L, qt, head, false);
    for (int round = 0; ok && have; ++round) {
      const int n_kv = (L + kKvRows - 1) / kKvRows;
      float m_ref = -INFINITY;
      float l_run = 0.f;
      for (int j = 0; j < n_kv; ++j, ++step) {
        const int kv_valid = min(kKvRows, L - j * kKvRows);
        if (!mbar_wait_bounded(s_full, step & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t s[128];
        tmem_ld_32x32_at<0>(t_s, s);
        tmem_ld_32x32_at<32>(t_s + 32, s);
        tmem_ld_32x32_at<64>(t_s + 64, s);
        tmem_ld_32x32_at<96>(t_s + 96, s);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
        if (kv_valid != kKvRows) {
          // last tile of the sequence: keys that do not exist get -inf (probability 0), by selection
#pragma unroll
          for (int i = 0; i < 128; ++i) s[i] = (i < kv_valid) ? s[i] : 0xff800000u;
        }
        // ---- exact row maximum
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 128; i += 8) {
          mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
          mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
          mx2 = max3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
          mx3 = max3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
        }
        const float m_new = fmaxf(m_ref, c * max3(mx0, mx1, fmaxf(mx2, mx3)));
        bool pv_waited = (j == 0);  // (first tile of an item: the wait for the previous item's O covered it)
        if (j == 0) {
          m_ref = m_new;
        } else if (__any_sync(0xffffffffu, (m_new - m_ref) > kRescaleThreshold)) {
          // O belongs to the P V MMAs of the previous key tile until those have retired
          if (!mbar_wait_bounded(pv_done, (step - 1u) & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          pv_waited = true;
          const float f = ex2_approx(m_ref - m_new);
#pragma unroll
          for (int cb = 0; cb < kHeadDim; cb += 32) {
            uint32_t v[32];
            tmem_ld_32x32(t_o + cb, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
            tmem_st_32x32(t_o + cb, v);
          }
          l_run *= f;
          m_ref = m_new;
        }
        // ---- probabilities: fp16 pairs for P's own columns, fp32 row sum
        float l0 = 0.f, l1 = 0.f;
        uint32_t pk[64];
#pragma unroll
        float l2 = 0.f, l3 = 0.f;
        for (int i = 0; i < 64; ++i) {
          float t0, t1;
          fma2(t0, t1, __uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]), c, -m_ref);
          const float p0 = ex2_approx(t0);
          const float p1 = ex2_approx(t1);
          if (i & 1) add2(l2, l3, p0, p1); else add2(l0, l1, p0, p1);
          pk[i] = pack_half2(p0, p1);
        }
        l_run += (l0 + l1) + (l2 + l3);
        if (!pv_waited) {
          // P belongs to the P V MMAs of the previous key tile until those have retired
          if (!mbar_wait_bounded(pv_done, (step - 1u) & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
        }
        tmem_st_32x16_at<0>(t_p, pk);
        tmem_st_32x16_at<16>(t_p + 16, pk);
        tmem_st_32x16_at<32>(t_p + 32, pk);
        tmem_st_32x16_at<48>(t_p + 48, pk);
        if (kv_valid != kKvRows) {
          // tail tile: blank the V rows of keys that do not belong to this sequence
          if (!mbar_wait_bounded(&v_full[stage], phase, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
            ok = false;
            break;
          }
          if (r >= kv_valid) {
            uint4* vr = reinterpret_cast<uint4*>(smem + kSmemV + stage * kTileBytes + r * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) vr[i] = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async_smem();
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      // the next item is found while the last P V of this one runs
      int seq_start_n = 0, L_n = 0, qt_n = 0, head_n = 0;
      have = decode_item(args, snake_item(round + 1, cta, G), cur_b, cur_first, seq_start_n, L_n, qt_n, head_n, false);
      if (!mbar_wait_bounded(o_done, static_cast<uint32_t>(round) & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // O / row sum -> fp16 -> this warp's 32 x 128 B staging rows (16-byte units swizzled by the row, the
      // 128-byte swizzle of a tensor map) -> global memory.  A slab whose 32 rows all belong to the sequence
      // leaves by one bulk store (the stores of the threads took 1.0-1.5 k clocks per item on the softmax
      // warps' critical path); a slab that crosses the end of the sequence is stored by the threads, eight
      // per row, so that a store instruction covers four whole 128-byte lines and rows of the next sequence
      // are left alone.
      const float inv = 1.0f / l_run;
      if (lane == 0) tma_store_wait_read();  // the previous item's bulk store has read the staging rows
      __syncwarp();
      uint8_t* stage_out = smem + kSmemOut + warp * (32 * 128);
      uint32_t va[32], vb[32];
      tmem_ld_32x32(t_o, va);
      tmem_ld_32x32(t_o + 32, vb);
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 w;
        w.x = pack_half2(__uint_as_float(va[u * 8 + 0]) * inv, __uint_as_float(va[u * 8 + 1]) * inv);
        w.y = pack_half2(__uint_as_float(va[u * 8 + 2]) * inv, __uint_as_float(va[u * 8 + 3]) * inv);
        w.z = pack_half2(__uint_as_float(va[u * 8 + 4]) * inv, __uint_as_float(va[u * 8 + 5]) * inv);
        w.w = pack_half2(__uint_as_float(va[u * 8 + 6]) * inv, __uint_as_float(va[u * 8 + 7]) * inv);
        *reinterpret_cast<uint4*>(stage_out + lane * 128 + ((u ^ (lane & 7)) << 4)) = w;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 w;
        w.x = pack_half2(__uint_as_float(vb[u * 8 + 0]) * inv, __uint_as_float(vb[u * 8 + 1]) * inv);
        w.y = pack_half2(__uint_as_float(vb[u * 8 + 2]) * inv, __uint_as_float(vb[u * 8 + 3]) * inv);
        w.z = pack_half2(__uint_as_float(vb[u * 8 + 4]) * inv, __uint_as_float(vb[u * 8 + 5]) * inv);
        w.w = pack_half2(__uint_as_float(vb[u * 8 + 6]) * inv, __uint_as_float(vb[u * 8 + 7]) * inv);
        *reinterpret_cast<uint4*>(stage_out + lane * 128 + (((4 + u) ^ (lane & 7)) << 4)) = w;
      }
      const bool whole_slab = args.tma_out != 0 && qt * kQRows + warp * 32 + 32 <= L;
      if (whole_slab) fence_proxy_async_smem();
      __syncwarp();
      if (whole_slab) {
        if (lane == 0) {
          tma_store_2d(&tm_ctx, stage_out, head * kHeadDim, seq_start + qt * kQRows + warp * 32);
          tma_store_commit();
        }
      } else {
        const int sub = lane >> 3, unit = lane & 7;  // row within a group of four, 16-byte unit of the row
        const int row0 = qt * kQRows + warp * 32;     // first query row of this warp's slab, within the sequence
        __half* out_base = args.ctx + static_cast<size_t>(seq_start + row0) * args.hidden + head * kHeadDim + unit * 8;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int row = 4 * k + sub;
          const uint4 w = *reinterpret_cast<const uint4*>(stage_out + row * 128 + ((unit ^ (row & 7)) << 4));
          if (row0 + row < L) *reinterpret_cast<uint4*>(out_base + static_cast<size_t>(row) * args.hidden) = w;
        }
      }
      __syncwarp();  // the staging rows are rewritten at the end of the next item
      seq_start = seq_start_n;
      L = L_n;
      qt = qt_n;
      head = head_n;
    }
    if (lane == 0) tma_store_wait_all();  // the staging rows must outlive the last bulk store
    tc_fence_before();
  }

  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

cudaError_t launch_persistent(const MhaLaunch& a, cudaStream_t stream) {
  static bool attr_set[64] = {};
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(mha_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPersistentSmemBytes);
    if (e != cudaSuccess) return e;
    if (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms[dev] <= 0)
      sms[dev] = 148;
    attr_set[dev] = true;
  }
  MhaPersistentArgs args;
  args.ctx = a.ctx;
  args.batch_idx = a.batch_idx;
  args.batch = a.batch;
  args.heads = a.head_num;
  args.hidden = a.hidden;
  args.scale_log2e = a.scale_log2e;
  args.status = a.status;
  args.rows = a.rows;
  args.max_len = a.max_len;
  args.tma_out = a.has_tm_ctx ? 1 : 0;
  const long long items_max =
      static_cast<long long>(a.batch) * a.head_num * ((a.max_len + kQRows - 1) / kQRows);  // upper bound
  long long grid = 2LL * sms[dev];
  if (grid > items_max) grid = items_max;
  if (grid < 1) grid = 1;
  return launch_pdl(mha_persistent_kernel, dim3(static_cast<unsigned>(grid)), dim3(kPersistentThreads), kPersistentSmemBytes,
                    stream, a.tm_qkv, a.has_tm_ctx ? a.tm_ctx : a.tm_qkv, args);
}

template <bool GENERAL>
cudaError_t launch_per_item(const MhaLaunch& a, const MhaArgs& args, cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(mha_fwd_kernel<GENERAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, MhaCfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  dim3 grid((a.max_len + kQRows - 1) / kQRows, a.head_num, a.batch);
  return launch_pdl(mha_fwd_kernel<GENERAL>, grid, dim3(MhaCfg::kThreads), MhaCfg::kSmemBytes, stream, a.tm_qkv, args);
}

}  // namespace

cudaError_t launch_mha(const MhaLaunch& a, cudaStream_t stream) {
  if (a.batch <= 0 || a.max_len <= 0 || a.head_num <= 0) return cudaErrorInvalidValue;
  MhaArgs args;
  args.ctx = a.ctx;
  args.batch_idx = a.batch_idx;
  args.hidden = a.hidden;
  args.scale_log2e = a.scale_log2e;
  args.status = a.status;
  args.rows = a.rows;
  args.max_len = a.max_len;
  args.gen_mask = a.gen_mask;
  args.gen_bias = a.gen_bias;
  args.gen_seq_len = a.max_len;
  args.gen_inv_scale = a.gen_inv_scale;
  args.gen_kv_bound = a.gen_kv_bound;
  args.gen_bits = a.gen_bias == nullptr ? a.gen_bits : nullptr;
  args.gen_bits_flag = a.gen_bits_flag;
  args.gen_bits_stride = mask_bits_stride_words(a.max_len);
  // General [B,S,S] mask (+ optional bias): one CTA per (128 query rows, head, sequence).  A persistent-CTA
  // form of it (mask applied from the bits) was measured slower at batch 16 / 512 tokens (2.36 against 2.19 ms
  // per 12 layers): 768 items of one to four key tiles fill the 296 CTAs' last round unevenly, while one CTA
  // per item is balanced by the hardware's block scheduler.
  if (a.gen_mask != nullptr) return launch_per_item<true>(a, args, stream);
  // Measured on B200 (12 heads, 18.9k tokens): the persistent kernel is ahead at every length (sequences
  // of 64 / 128 / 256 / 384 / 1024 tokens: 70 / 40 / 47 / 57 / 105 us against 77 / 40 / 52 / 62 / 120) and for
  // few long sequences (one of 614 tokens: 12.8 against 14.0 us; 16 up to 512: 24 against 27); only a handful
  // of short items, fewer than the persistent CTAs, is served faster by one CTA per item (16 sequences up
  // to 64 tokens: 7.0 against 8.3 us).
  const long long items_max = static_cast<long long>(a.batch) * a.head_num * ((a.max_len + kQRows - 1) / kQRows);
  // (a few dozen items of a single sequence, e.g. one sequence of 307 tokens = 36 items: 0.622 against 0.641 ms
  // per 12-layer forward with one CTA per item; from ~100 items of long rows on the persistent kernel is ahead)
  const bool persistent =
      g_dbg_force_kernel == 3 ||
      (g_dbg_force_kernel == 0 && (items_max > 296 || (a.max_len > kQRows && items_max >= 64)));
  return persistent ? launch_persistent(a, stream) : launch_per_item<false>(a, args, stream);
}

}  // namespace bt

// Diagnostics hook (process-global, for tests and measurements; not part of the stable ABI): attention
// kernel 0 = chosen by shape, 1 = one CTA per item, 3 = persistent.
extern "C" int bt_debug_set_mha_tiles(long long kernel) {
  bt::g_dbg_force_kernel = kernel;
  return 0;
}
