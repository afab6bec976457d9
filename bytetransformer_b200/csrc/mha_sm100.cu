// Fused variable-length multi-head attention for sm_100a (head size 64, fp16 in/out).
//
// Stands in for the reference's packed attention kernels
// (bytetransformer/src/attention_fused.cu:295-414 for short sequences,
// bytetransformer/src/attention_fused_long.cu:171-312 and the grouped-GEMM path
// of bytetransformer/src/cutlass_attention.cu:150-210 for long ones).  One
// templated kernel, two instantiations:
//   TILES = 1  128 query rows per CTA, 192 threads, two CTAs per SM overlap each
//              other's phases (the default: fastest at every length 64..1024);
//   TILES = 2  256 query rows per CTA as two 128-row tiles that ping-pong on the
//              tensor core, 320 threads, one CTA per SM (selectable).
// Both run an online softmax over 128-key tiles, so no S x S logits ever reach
// HBM and any length works.
//
// Input is the packed QKV activation [rows, 3H] with bias already added by the
// QKV GEMM epilogue; head h of Q/K/V is the 64-column slice at h*64 / H+h*64 /
// 2H+h*64, fetched straight from that buffer by TMA (the reference's separate
// bias-add + head-split transpose kernel, attention_nofused_utils.cu:142-184, has
// no counterpart here).  Only `batch_idx` tells where sequences start and end;
// as in the reference's packed kernels the mask tensor is not consulted again.
//
// Roles: warp 0 TMA loads, warp 1 tcgen05.mma issue (+ tensor-memory allocation),
// then one warpgroup of 4 softmax warps per query tile (one query row per thread).
//   S = Q K^T      128x128x64, both operands from shared memory -> tensor memory,
//                  128 fp32 columns per tile
//   P = 2^(c*S-m)  fp16 pairs written back into tensor memory over the upper half of
//                  S (columns 64..127, key k in cell 64 + k/2) with tcgen05.st; the
//                  softmax walks S from the last 32-column chunk to the first, so a
//                  cell is only overwritten after it was read
//   O += P V       128x64x128 with the A operand (P) read from tensor memory and V
//                  consumed MN-major from shared memory exactly as it lies in the QKV
//                  buffer -> 64 fp32 columns per tile
// The persistent kernel for long sequences (further down) uses the free 64 columns of its 256
// for P instead (S 0..127, O 128..191, P 192..255): S stays intact, so the next S = Q K^T is
// issued before O += P V, and every key tile is read from tensor memory only once (the
// probabilities are formed with the reference of the earlier tiles and the tile is redone only
// when the row maximum jumped past the threshold).  The softmax is a chain of dependent
// latencies (tcgen05.ld, wait, arithmetic, tcgen05.st, barrier) run by two warps per scheduler
// (S, O and P take 256 of the 512 tensor-memory columns, so two CTAs fit on an SM), not a
// bandwidth problem: a read-only loop (tmem_probe.cu) gets 120-370 B/clk per SM out of tensor memory,
// the softmax consumes ~48.  Touching every score once instead of twice shortened that chain.
// P never touches shared memory.  O stays in tensor memory across key tiles.  The
// exponent reference m only moves when the running maximum grows by more than a
// threshold (then the O row is rescaled in tensor memory); otherwise P simply grows
// up to 2^threshold, which fp16 holds, and the final division by the row sum makes
// the result exact.
// Keys beyond the sequence end are masked by selection (never by arithmetic on
// the fetched values) and their V rows are zeroed in shared memory, so rows of
// neighbouring sequences or never-written workspace cannot leak in.
#include "common.cuh"
#include "kernels.h"

namespace bt {

namespace {

constexpr int kQRows = 128;
constexpr int kKvRows = 128;
constexpr int kHeadDim = 64;
constexpr int kTileBytes = 128 * kHeadDim * 2;  // 16 KiB: Q, K or V tile

template <int TILES>
struct MhaCfg {
  static constexpr int kStages = 3;
  static constexpr int kThreads = 64 + 128 * TILES;
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemK = kSmemQ + TILES * kTileBytes;
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr int kSmemBar = kSmemV + kStages * kTileBytes;
  static constexpr int kSmemBytes = kSmemBar + 256;
  static constexpr int kTmemCols = TILES == 2 ? 512 : 256;
  static constexpr uint32_t kTmemO = TILES * 128;  // S tiles first, then O tiles
  static constexpr uint32_t kTmemPOff = 64;        // P aliases columns 64..127 of its S tile
  static constexpr int kMinBlocks = TILES == 2 ? 1 : 2;
};

struct MhaArgs {
  __half* ctx;
  const int* batch_idx;
  int hidden;
  float scale_log2e;
  int* status;
  long long* timing;  // diagnostics: per CTA and key-tile step, clock64 stamps (null = off)
  // General-mask variant (GENERAL = true): every sequence has `gen_seq_len` rows; the score of
  // (query q, key k) gets  attn_bias[head, q, k] + (1 - mask[b, q, k]) * -10000  added after scaling,
  // the rule of the reference's unfused softmax (bytetransformer/include/softmax.h:41-45).
  const __half* gen_mask;  // [batch, S, S]
  const __half* gen_bias;  // [heads, S, S] or null
  int gen_seq_len;
  float gen_inv_scale;     // 1 / (softmax scale): the additive term is applied to the unscaled score
  const int* gen_kv_bound; // [batch, query tiles]: leading keys that matter for the query tile, or null
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// two exponentials per special-function op, fp16 in / fp16 out
__device__ __forceinline__ uint32_t ex2_f16x2(uint32_t x) {
  uint32_t y;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
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

// One 32-column chunk of S -> 16 cells of fp16 pairs, plus this chunk's row sum.
//   EXP16 = false: 2^x in fp32 (one special-function op per key), fp32 row sum.
//   EXP16 = true : x is rounded to fp16 first and two exponentials share one op; the row
//                  sum is formed from the fp16 results (pairwise tree, then fp32).
template <bool MASKED, bool EXP16>
__device__ __forceinline__ float chunk_probs(const uint32_t (&v)[32], int cbase, int kv_valid, float c, float m_ref,
                                             uint32_t (&out)[16]) {
  if (EXP16) {
    __half2 acc[4];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float x0 = fmaf(__uint_as_float(v[2 * i]), c, -m_ref);
      float x1 = fmaf(__uint_as_float(v[2 * i + 1]), c, -m_ref);
      if (MASKED) {
        // 2^-inf = 0 for keys that do not exist
        x0 = (cbase + 2 * i < kv_valid) ? x0 : -INFINITY;
        x1 = (cbase + 2 * i + 1 < kv_valid) ? x1 : -INFINITY;
      }
      out[i] = ex2_f16x2(pack_half2(x0, x1));
      const __half2 h = *reinterpret_cast<const __half2*>(&out[i]);
      acc[i & 3] = (i < 4) ? h : __hadd2(acc[i & 3], h);
    }
    const float2 s01 = __half22float2(__hadd2(acc[0], acc[1]));
    const float2 s23 = __half22float2(__hadd2(acc[2], acc[3]));
    return (s01.x + s01.y) + (s23.x + s23.y);
  } else {
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float p0 = ex2_approx(fmaf(__uint_as_float(v[2 * i]), c, -m_ref));
      float p1 = ex2_approx(fmaf(__uint_as_float(v[2 * i + 1]), c, -m_ref));
      if (MASKED) {
        p0 = (cbase + 2 * i < kv_valid) ? p0 : 0.f;
        p1 = (cbase + 2 * i + 1 < kv_valid) ? p1 : 0.f;
      }
      l0 += p0;
      l1 += p1;
      out[i] = pack_half2(p0, p1);
    }
    return l0 + l1;
  }
}

// Second pass over one S tile, from the last chunk to the first; P chunk c lands in cells
// [64 + 16c, 64 + 16c + 16) of the same tile, which lie in chunks that were already read.
template <bool MASKED, bool EXP16>
__device__ __forceinline__ float tile_probs(uint32_t t_s, int kv_valid, float c, float m_ref) {
  const uint32_t t_p = t_s + 64;
  uint32_t va[32], vb[32], pk[16];
  float l = 0.f;
  tmem_ld_32x32(t_s + 96, va);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 64, vb);  // in flight while chunk 3 is processed
  l += chunk_probs<MASKED, EXP16>(va, 96, kv_valid, c, m_ref, pk);
  tmem_ld_wait();               // chunk 2 is in registers: its cells may now be overwritten
  tmem_st_32x16(t_p + 48, pk);
  tmem_ld_32x32(t_s + 32, va);
  l += chunk_probs<MASKED, EXP16>(vb, 64, kv_valid, c, m_ref, pk);
  tmem_ld_wait();
  tmem_st_32x16(t_p + 32, pk);
  tmem_ld_32x32(t_s, vb);
  l += chunk_probs<MASKED, EXP16>(va, 32, kv_valid, c, m_ref, pk);
  tmem_ld_wait();
  tmem_st_32x16(t_p + 16, pk);
  l += chunk_probs<MASKED, EXP16>(vb, 0, kv_valid, c, m_ref, pk);
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

// One 32-column chunk with the exponent reference of the EARLIER key tiles: probabilities, their
// sum, and the largest exponent seen (to tell afterwards whether the reference was good enough).
template <bool MASKED>
__device__ __forceinline__ float chunk_probs_track(const uint32_t (&v)[32], int cbase, int kv_valid, float c, float m_ref,
                                                   uint32_t (&out)[16], float& xmax) {
  float l0 = 0.f, l1 = 0.f, x0m = xmax, x1m = xmax;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float x0 = fmaf(__uint_as_float(v[2 * i]), c, -m_ref);
    float x1 = fmaf(__uint_as_float(v[2 * i + 1]), c, -m_ref);
    if (MASKED) {
      x0 = (cbase + 2 * i < kv_valid) ? x0 : -INFINITY;
      x1 = (cbase + 2 * i + 1 < kv_valid) ? x1 : -INFINITY;
    }
    x0m = fmaxf(x0m, x0);
    x1m = fmaxf(x1m, x1);
    const float p0 = ex2_approx(x0);
    const float p1 = ex2_approx(x1);
    l0 += p0;
    l1 += p1;
    out[i] = pack_half2(p0, p1);
  }
  xmax = fmaxf(x0m, x1m);
  return l0 + l1;
}

// Same pass with P in its own tensor-memory columns (`t_p`, 64 cells): the chunk order is free and
// nothing of S is overwritten, so the next S = Q K^T may be issued as soon as this pass has read S.
template <bool MASKED>
__device__ __forceinline__ float tile_probs_sep(uint32_t t_s, uint32_t t_p, int kv_valid, float c, float m_ref) {
  uint32_t va[32], vb[32], pk[16];
  float l = 0.f;
  tmem_ld_32x32(t_s, va);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 32, vb);
  l += chunk_probs<MASKED, false>(va, 0, kv_valid, c, m_ref, pk);
  tmem_st_32x16(t_p, pk);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 64, va);
  l += chunk_probs<MASKED, false>(vb, 32, kv_valid, c, m_ref, pk);
  tmem_st_32x16(t_p + 16, pk);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 96, vb);
  l += chunk_probs<MASKED, false>(va, 64, kv_valid, c, m_ref, pk);
  tmem_st_32x16(t_p + 32, pk);
  tmem_ld_wait();
  l += chunk_probs<MASKED, false>(vb, 96, kv_valid, c, m_ref, pk);
  tmem_st_32x16(t_p + 48, pk);
  tmem_st_wait();
  return l;
}

__device__ __forceinline__ void stamp(long long* timing, int j, int slot) {
  if (timing != nullptr && j < 8) {
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta < 4096) timing[(static_cast<size_t>(cta) * 8 + j) * 8 + slot] = clock64();
  }
}

template <int TILES, bool EXP16, bool GENERAL = false>
__global__ void __launch_bounds__(MhaCfg<TILES>::kThreads, MhaCfg<TILES>::kMinBlocks)
mha_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const MhaArgs args) {
  using Cfg = MhaCfg<TILES>;
  constexpr int kStages = Cfg::kStages;
  // With fp16 exponents the reference may lag the running maximum by at most 2^1 (keeps the
  // rounding of the exponent small); with fp32 exponents by 2^8.
  constexpr float kRescaleThreshold = EXP16 ? 1.0f : 8.0f;
  extern __shared__ __align__(1024) uint8_t smem[];

  pdl_launch_dependents();
  pdl_wait();  // batch_idx and the QKV buffer come from earlier kernels
  const int b = blockIdx.z;
  const int head = blockIdx.y;
  const int seq_start = __ldg(args.batch_idx + b);
  const int L = __ldg(args.batch_idx + b + 1) - seq_start;
  const int q0 = blockIdx.x * (kQRows * TILES);
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
        stamp(args.timing, j, 4);
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
        stamp(args.timing, j, 5);
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
      for (int j = 0; j < n_kv; ++j) {
        const uint32_t jpar = j & 1;
        const int kv_valid = min(kKvRows, L - j * kKvRows);
        const bool full_tile = kv_valid == kKvRows;
        if (!mbar_wait_bounded(&s_full[t], jpar, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (warp == 2 && lane == 0) stamp(args.timing, j, 0);
        if (GENERAL) {
          const int S = args.gen_seq_len;
          const int q_row = q0 + t * kQRows + r;
          const bool q_ok = q_row < S;
          const size_t off = static_cast<size_t>(q_ok ? q_row : 0) * S + static_cast<size_t>(j) * kKvRows;
          tile_add_mask_bias(t_s, args.gen_mask + static_cast<size_t>(b) * S * S + off,
                             args.gen_bias != nullptr ? args.gen_bias + static_cast<size_t>(head) * S * S + off : nullptr,
                             q_ok ? kv_valid : 0, (S & 7) == 0, args.gen_inv_scale);
        }
        // pass 1: row maximum (scaled to log2 units)
        const float mx = c * (full_tile ? tile_row_max<false>(t_s, kv_valid) : tile_row_max<true>(t_s, kv_valid));
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
        if (warp == 2 && lane == 0) stamp(args.timing, j, 1);
        // pass 2: probabilities -> fp16 pairs -> tensor memory (over S), row sum
        l_run += full_tile ? tile_probs<false, EXP16>(t_s, kv_valid, c, m_ref)
                           : tile_probs<true, EXP16>(t_s, kv_valid, c, m_ref);
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
        if (warp == 2 && lane == 0) stamp(args.timing, j, 2);
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
// Persistent variant: each CTA (192 threads, two per SM) walks a static list of work items
// (sequence, 128-row query tile, head), item n going to CTA n mod gridDim.x.  Barriers,
// tensor memory and the launch are paid once per CTA instead of once per item, and the
// loader runs ahead: the next item's Q/K/V tiles are requested while the current item's last
// key tiles are still being processed.  Per item the MMAs are those of mha_fwd_kernel<1>; the
// softmax follows the PSEP / ONEPASS scheme described at the kernel (default) or, selectable, the
// two-pass scheme of mha_fwd_kernel<1> (same tile_row_max / tile_probs).
// ------------------------------------------------------------------------------------------
struct MhaPersistentArgs {
  __half* ctx;
  const int* batch_idx;
  int batch;
  int heads;
  int hidden;
  float scale_log2e;
  int* status;
};

// Finds item n = (sequence b, query tile qt, head h); items are numbered sequence by
// sequence, inside a sequence query tile by query tile, heads fastest.  `cur_b` / `cur_first`
// is the caller's cursor (first item index of sequence cur_b); n never decreases.
__device__ __forceinline__ bool decode_item(const int* __restrict__ batch_idx, int B, int heads, int n, int& cur_b,
                                            int& cur_first, int& seq_start, int& L, int& qt, int& h) {
  while (cur_b < B) {
    seq_start = __ldg(batch_idx + cur_b);
    L = __ldg(batch_idx + cur_b + 1) - seq_start;
    const int items = ((L + kQRows - 1) / kQRows) * heads;
    if (n < cur_first + items) {
      const int r = n - cur_first;
      qt = r / heads;
      h = r - qt * heads;
      return true;
    }
    cur_first += items;
    ++cur_b;
  }
  return false;
}

// PSEP = true: P lives in its own 64 tensor-memory columns instead of over the upper half of S.  The
// MMA warp can then issue S(j+1) = Q K(j+1)^T BEFORE O += P(j) V(j): the next softmax starts after
// four MMAs instead of twelve, and P V runs in its shadow.  The softmax waits for `pv_done` of the
// previous key tile before it rescales O or overwrites P.
// ONEPASS (needs PSEP): key tiles after the first are read from tensor memory ONCE: probabilities are
// formed with the reference of the earlier tiles while the largest exponent is tracked; only when that
// exceeds the threshold (the row maximum jumped by more than 2^8) is the tile redone with a new
// reference, which is possible because S is still intact.  The second read of every score (load, wait,
// arithmetic) was the longest avoidable piece of the softmax's latency chain.
template <bool EXP16, bool PSEP = false, bool ONEPASS = false>
__global__ void __launch_bounds__(192, 2)
mha_persistent_kernel(const __grid_constant__ CUtensorMap tm_qkv, const MhaPersistentArgs args) {
  constexpr int kStages = 3;
  constexpr int kSmemQ = 0;
  constexpr int kSmemK = kSmemQ + kTileBytes;
  constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  constexpr int kSmemBar = kSmemV + kStages * kTileBytes;
  constexpr uint32_t kTmemS = 0, kTmemP = PSEP ? 192 : 64, kTmemO = 128;
  constexpr float kRescaleThreshold = EXP16 ? 1.0f : 8.0f;
  extern __shared__ __align__(1024) uint8_t smem[];

  pdl_launch_dependents();
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBar);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;                  // [kStages]
  uint64_t* v_full = bars + 2 + kStages;        // [kStages]
  uint64_t* kv_empty = bars + 2 + 2 * kStages;  // [kStages]
  uint64_t* s_full = bars + 2 + 3 * kStages;
  uint64_t* p_full = bars + 3 + 3 * kStages;
  uint64_t* o_done = bars + 4 + 3 * kStages;
  uint64_t* pv_done = bars + 5 + 3 * kStages;   // PSEP: the P V MMAs of a key tile have retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6 + 3 * kStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool smem_ok = (smem_u32(smem) & 1023u) == 0u;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_done, 1);
    mbar_init(pv_done, 1);
    *abort_flag = smem_ok ? 0 : 1;
    fence_mbar_init();
    if (!smem_ok && args.status != nullptr) atomicCAS(args.status, 0, kStatusMhaLoadTimeout + 0x10);
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // batch_idx and the QKV buffer come from earlier kernels

  const int B = args.batch, heads = args.heads;
  int cur_b = 0, cur_first = 0, seq_start = 0, L = 0, qt = 0, head = 0;

  if (!smem_ok) {
    // fall through to the teardown
  } else if (warp == 0) {
    // ------------------------------------------------------------------ loads
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t item = 0;
      bool ok = true;
      for (int n = blockIdx.x; ok && decode_item(args.batch_idx, B, heads, n, cur_b, cur_first, seq_start, L, qt, head);
           n += gridDim.x, ++item) {
        const int n_kv = (L + kKvRows - 1) / kKvRows;
        if (!mbar_wait_bounded(q_empty, (item & 1u) ^ 1u, abort_flag, args.status, kStatusMhaLoadTimeout)) break;
        mbar_arrive_expect_tx(q_full, kTileBytes);
        tma_load_2d(smem + kSmemQ, &tm_qkv, q_full, head * kHeadDim, seq_start + qt * kQRows);
        for (int j = 0; j < n_kv; ++j) {
          if (!mbar_wait_bounded(&kv_empty[stage], phase ^ 1u, abort_flag, args.status, kStatusMhaLoadTimeout)) {
            ok = false;
            break;
          }
          const int row = seq_start + j * kKvRows;
          mbar_arrive_expect_tx(&k_full[stage], kTileBytes);
          tma_load_2d(smem + kSmemK + stage * kTileBytes, &tm_qkv, &k_full[stage], args.hidden + head * kHeadDim, row);
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
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint64_t kDescK = make_smem_desc_hi(16, 1024);
      constexpr uint64_t kDescV = make_smem_desc_hi(kTileBytes, 1024);
      constexpr uint32_t kIdescS = make_idesc_f16(128, 128, 0, 0);
      constexpr uint32_t kIdescO = make_idesc_f16(128, 64, 0, 1);
      const uint32_t s_q = smem_u32(smem + kSmemQ);
      const uint32_t s_k = smem_u32(smem + kSmemK);
      const uint32_t s_v = smem_u32(smem + kSmemV);
      auto issue_s = [&](int stage) {
        const uint32_t sk = s_k + stage * kTileBytes;
#pragma unroll
        for (int k = 0; k < kHeadDim / 16; ++k)
          umma_f16_ss(tmem_base + kTmemS, smem_desc(kDescK, s_q + k * 32), smem_desc(kDescK, sk + k * 32), kIdescS,
                      k != 0 ? 1u : 0u);
        umma_commit(s_full);
      };
      int st = 0;
      uint32_t ph = 0;
      uint32_t step = 0, item = 0;
      bool ok = true;
      for (int n = blockIdx.x; ok && decode_item(args.batch_idx, B, heads, n, cur_b, cur_first, seq_start, L, qt, head);
           n += gridDim.x, ++item) {
        const int n_kv = (L + kKvRows - 1) / kKvRows;
        if (!mbar_wait_bounded(q_full, item & 1u, abort_flag, args.status, kStatusMhaMmaTimeout)) break;
        if (!mbar_wait_bounded(&k_full[st], ph, abort_flag, args.status, kStatusMhaMmaTimeout)) break;
        tc_fence_after();
        issue_s(st);
        if (n_kv == 1) umma_commit(q_empty);  // the item's last (only) QK^T has been issued
        for (int j = 0; j < n_kv; ++j, ++step) {
          const int st_n = (st + 1 == kStages) ? 0 : st + 1;
          const uint32_t ph_n = (st + 1 == kStages) ? (ph ^ 1u) : ph;
          // P of this step is ready; it also tells that the softmax warps have finished the
          // previous item's O read-out, so the first PV of an item may overwrite O.
          if (!mbar_wait_bounded(p_full, step & 1u, abort_flag, args.status, kStatusMhaMmaTimeout)) {
            ok = false;
            break;
          }
          if (PSEP && j + 1 < n_kv) {
            // the softmax has read S(j) completely and P(j) sits elsewhere: S(j+1) goes first
            if (!mbar_wait_bounded(&k_full[st_n], ph_n, abort_flag, args.status, kStatusMhaMmaTimeout)) {
              ok = false;
              break;
            }
            tc_fence_after();
            issue_s(st_n);
            if (j + 2 == n_kv) umma_commit(q_empty);
          }
          if (!mbar_wait_bounded(&v_full[st], ph, abort_flag, args.status, kStatusMhaMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sv = s_v + st * kTileBytes;
          // only the 16-key steps that hold keys of this sequence (in the last tile the softmax leaves
          // the P columns of 32-key chunks without any key unwritten)
          const int kk_n = (min(kKvRows, L - j * kKvRows) + 15) >> 4;
#pragma unroll
          for (int kk = 0; kk < kKvRows / 16; ++kk)
            if (kk < kk_n)
              umma_f16_ts(tmem_base + kTmemO, tmem_base + kTmemP + kk * 8, smem_desc(kDescV, sv + kk * 2048), kIdescO,
                          (j > 0 || kk != 0) ? 1u : 0u);
          if (PSEP) umma_commit(pv_done);
          if (!PSEP && j + 1 < n_kv) {
            if (!mbar_wait_bounded(&k_full[st_n], ph_n, abort_flag, args.status, kStatusMhaMmaTimeout)) {
              ok = false;
              break;
            }
            tc_fence_after();
            issue_s(st_n);  // executes after the PV above (issue order), so P is not overwritten early
            if (j + 2 == n_kv) umma_commit(q_empty);
          }
          umma_commit(&kv_empty[st]);
          st = st_n;
          ph = ph_n;
        }
        if (ok) umma_commit(o_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // query row inside the tile == TMEM lane
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t t_s = t_lane + kTmemS;
    const uint32_t t_o = t_lane + kTmemO;
    const float c = args.scale_log2e;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t step = 0, item = 0;
    bool ok = true;
    for (int n = blockIdx.x; ok && decode_item(args.batch_idx, B, heads, n, cur_b, cur_first, seq_start, L, qt, head);
         n += gridDim.x, ++item) {
      const int n_kv = (L + kKvRows - 1) / kKvRows;
      float m_ref = -INFINITY;
      float l_run = 0.f;
      for (int j = 0; j < n_kv; ++j, ++step) {
        const int kv_valid = min(kKvRows, L - j * kKvRows);
        const bool full_tile = kv_valid == kKvRows;
        if (!mbar_wait_bounded(s_full, step & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (ONEPASS) {
          // ---- optimistic single pass with the reference of the earlier tiles (first tile of an item:
          // with the maximum of its first 32 keys)
          const uint32_t t_p = t_lane + kTmemP;
          uint32_t va[32], vb[32], pk0[16], pk1[16];
          float xmax = -INFINITY, l_tile = 0.f;
          if (full_tile) {
            tmem_ld_32x32(t_s, va);
            tmem_ld_wait();
            tmem_ld_32x32(t_s + 32, vb);
            if (j == 0) m_ref = c * (chunk_max<false>(va, 0, kv_valid));
            l_tile += chunk_probs_track<false>(va, 0, kv_valid, c, m_ref, pk0, xmax);
            tmem_ld_wait();
            tmem_ld_32x32(t_s + 64, va);
            l_tile += chunk_probs_track<false>(vb, 32, kv_valid, c, m_ref, pk1, xmax);
            // P (and O) belong to the P V MMAs of the previous key tile until those have retired; the first
            // two chunks were computed in the meantime.  (First tile of an item: the wait for the previous
            // item's O at its end already covered that.)
            if (j > 0) {
              if (!mbar_wait_bounded(pv_done, (step - 1u) & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
                ok = false;
                break;
              }
              tc_fence_after();
            }
            tmem_st_32x16(t_p, pk0);
            tmem_st_32x16(t_p + 16, pk1);
            tmem_ld_wait();
            tmem_ld_32x32(t_s + 96, vb);
            l_tile += chunk_probs_track<false>(va, 64, kv_valid, c, m_ref, pk0, xmax);
            tmem_st_32x16(t_p + 32, pk0);
            tmem_ld_wait();
            l_tile += chunk_probs_track<false>(vb, 96, kv_valid, c, m_ref, pk1, xmax);
            tmem_st_32x16(t_p + 48, pk1);
          } else {
            // last tile of the sequence: only the 32-key chunks that hold at least one key are read and
            // exponentiated; the P columns of the others stay unwritten (the P V steps stop before them)
            const int n_chunks = (kv_valid + 31) >> 5;
            for (int ch = 0; ch < n_chunks; ++ch) {
              tmem_ld_32x32(t_s + ch * 32, va);
              tmem_ld_wait();
              if (j == 0 && ch == 0) m_ref = c * chunk_max<true>(va, 0, kv_valid);
              l_tile += chunk_probs_track<true>(va, ch * 32, kv_valid, c, m_ref, pk0, xmax);
              if (ch == 0 && j > 0) {
                if (!mbar_wait_bounded(pv_done, (step - 1u) & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
                  ok = false;
                  break;
                }
                tc_fence_after();
              }
              tmem_st_32x16(t_p + ch * 16, pk0);
            }
            if (!ok) break;
          }
          if (__any_sync(0xffffffffu, xmax > kRescaleThreshold)) {
            // the reference was too low for some row of this warp: move it, rescale O and the running
            // sum, and form this tile's probabilities again from S (rows that did not need it get f = 1)
            const float m_new = m_ref + fmaxf(xmax, 0.f);
            const float f = ex2_approx(m_ref - m_new);
#pragma unroll
            for (int cb = 0; cb < (j > 0 ? kHeadDim : 0); cb += 32) {  // (no O yet on the first tile)
              uint32_t v[32];
              tmem_ld_32x32(t_o + cb, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
              tmem_st_32x32(t_o + cb, v);
            }
            l_run *= f;
            m_ref = m_new;
            tmem_st_wait();
            l_tile = full_tile ? tile_probs_sep<false>(t_s, t_p, kv_valid, c, m_ref)
                               : tile_probs_sep<true>(t_s, t_p, kv_valid, c, m_ref);
          } else {
            tmem_st_wait();
          }
          l_run += l_tile;
        } else {
        const float mx = c * (full_tile ? tile_row_max<false>(t_s, kv_valid) : tile_row_max<true>(t_s, kv_valid));
        if (PSEP && j > 0) {
          // O and P still belong to the P V MMAs of the previous key tile until those have retired
          if (!mbar_wait_bounded(pv_done, (step - 1u) & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
        }
        if (j == 0) {
          m_ref = mx;
        } else {
          const float m_new = fmaxf(m_ref, mx);
          const bool need = (m_new - m_ref) > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
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
        if (PSEP)
          l_run += full_tile ? tile_probs_sep<false>(t_s, t_lane + kTmemP, kv_valid, c, m_ref)
                             : tile_probs_sep<true>(t_s, t_lane + kTmemP, kv_valid, c, m_ref);
        else
          l_run += full_tile ? tile_probs<false, EXP16>(t_s, kv_valid, c, m_ref)
                             : tile_probs<true, EXP16>(t_s, kv_valid, c, m_ref);
        }
        if (!full_tile) {
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
        tc_fence_before();
        mbar_arrive(p_full);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok || !mbar_wait_bounded(o_done, item & 1u, abort_flag, args.status, kStatusMhaSoftmaxTimeout)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int q_row = qt * kQRows + r;
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

  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

template <bool EXP16, bool PSEP = false, bool ONEPASS = false>
cudaError_t launch_persistent(const MhaLaunch& a, cudaStream_t stream) {
  constexpr int kSmemBytes = 7 * kTileBytes + 256;
  static bool attr_set[64] = {};
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(mha_persistent_kernel<EXP16, PSEP, ONEPASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
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
  const long long items_max =
      static_cast<long long>(a.batch) * a.head_num * ((a.max_len + kQRows - 1) / kQRows);  // upper bound
  long long grid = 2LL * sms[dev];
  if (grid > items_max) grid = items_max;
  if (grid < 1) grid = 1;
  return launch_pdl(mha_persistent_kernel<EXP16, PSEP, ONEPASS>, dim3(static_cast<unsigned>(grid)), dim3(192), kSmemBytes, stream,
                    a.tm_qkv, args);
}

template <int TILES, bool EXP16>
cudaError_t launch_tiles(const MhaLaunch& a, const MhaArgs& args, cudaStream_t stream) {
  using Cfg = MhaCfg<TILES>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(mha_fwd_kernel<TILES, EXP16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const int rows_per_cta = kQRows * TILES;
  dim3 grid((a.max_len + rows_per_cta - 1) / rows_per_cta, a.head_num, a.batch);
  return launch_pdl(mha_fwd_kernel<TILES, EXP16>, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, a.tm_qkv, args);
}

long long g_dbg_force_tiles = 0;
long long* g_dbg_timing = nullptr;
constexpr int kTimingCtas = 4096, kTimingSteps = 8, kTimingSlots = 8;
long long g_dbg_exp16 = 0;  // 0 = default (fp32 exponentials), 1 = fp16x2 exponentials

}  // namespace

cudaError_t launch_mha(const MhaLaunch& a, cudaStream_t stream) {
  if (a.batch <= 0 || a.max_len <= 0 || a.head_num <= 0) return cudaErrorInvalidValue;
  MhaArgs args;
  args.ctx = a.ctx;
  args.batch_idx = a.batch_idx;
  args.hidden = a.hidden;
  args.scale_log2e = a.scale_log2e;
  args.status = a.status;
  args.timing = g_dbg_timing;
  args.gen_mask = a.gen_mask;
  args.gen_bias = a.gen_bias;
  args.gen_seq_len = a.max_len;
  args.gen_inv_scale = a.gen_inv_scale;
  args.gen_kv_bound = a.gen_kv_bound;
  if (a.gen_mask != nullptr) {
    // general [B,S,S] mask (+ optional bias): one CTA per (128 query rows, head, sequence)
    using Cfg = MhaCfg<1>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(mha_fwd_kernel<1, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           Cfg::kSmemBytes);
      if (e != cudaSuccess) return e;
      attr_set[dev] = true;
    }
    dim3 grid((a.max_len + kQRows - 1) / kQRows, a.head_num, a.batch);
    return launch_pdl(mha_fwd_kernel<1, false, true>, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, a.tm_qkv, args);
  }
  // Measured on B200 (18.9k packed tokens, 12 heads): the one-tile variant with two
  // co-resident CTAs per SM is faster at every length from 64 to 1024, so it is the
  // default; the two-tile variant stays selectable.
  const bool exp16 = g_dbg_exp16 == 1;
  // Default: the persistent kernel once sequences span more than two key tiles (measured at
  // 18.9k tokens: +4..7 % at lengths 384..1024, +12 % on lengths uniform in [16,1024]); for
  // short sequences one CTA per item is faster (lengths 64 / 128: 77 vs 89 us, 40 vs 47 us).
  // With fewer than ~600 items (two per persistent CTA) the static item lists are too short to
  // balance and the hardware's own block scheduling of one CTA per item is as good or better
  // (12 layers, batch 1, 307 of 512 tokens: 0.756 vs 0.785 ms; batch 16 at max_seq 512: 1.544 vs 1.503 ms).
  const long long items_max = static_cast<long long>(a.batch) * a.head_num * ((a.max_len + kQRows - 1) / kQRows);
  if (g_dbg_force_tiles == 0 && a.max_len > 256 && items_max >= 600)
    return exp16 ? launch_persistent<true>(a, stream) : launch_persistent<false, true, true>(a, stream);
  if (g_dbg_force_tiles == 3) return exp16 ? launch_persistent<true>(a, stream) : launch_persistent<false, true, true>(a, stream);
  if (g_dbg_force_tiles == 6) return launch_persistent<false>(a, stream);  // P over the upper half of S, two reads of S per key tile
  if (g_dbg_force_tiles == 4) return launch_persistent<false, true>(a, stream);  // P in its own columns, S(j+1) before P V(j)
  if (g_dbg_force_tiles == 5) return launch_persistent<false, true, true>(a, stream);  // + one read of S per key tile
  int tiles = 1;
  if (g_dbg_force_tiles == 1 || g_dbg_force_tiles == 2) tiles = static_cast<int>(g_dbg_force_tiles);
  if (tiles == 1) return exp16 ? launch_tiles<1, true>(a, args, stream) : launch_tiles<1, false>(a, args, stream);
  return exp16 ? launch_tiles<2, true>(a, args, stream) : launch_tiles<2, false>(a, args, stream);
}

}  // namespace bt

// Diagnostics hooks (not part of the stable ABI): attention variant (0 = default: persistent
// for max_len > 256, else one CTA per item; 1 / 2 = one CTA per item with one / two query
// tiles; 3 = always persistent) and exponential flavour (0 = fp32, 1 = fp16x2).
extern "C" int bt_debug_set_mha_tiles(long long tiles) {
  bt::g_dbg_force_tiles = tiles;
  return 0;
}
// Device buffer of 4096 CTAs x 8 steps x 8 slots of long long for clock64 stamps (null = off).
extern "C" int bt_debug_set_mha_timing(long long* device_buffer) {
  bt::g_dbg_timing = device_buffer;
  return 0;
}
extern "C" int bt_debug_set_mha_exp16(long long on) {
  bt::g_dbg_exp16 = on;
  return 0;
}
