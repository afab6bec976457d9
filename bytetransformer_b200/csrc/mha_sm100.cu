// Fused variable-length multi-head attention for sm_100a (head size 64, fp16 in/out).
//
// Stands in for the reference's packed attention kernels
// (bytetransformer/src/attention_fused.cu:295-414 for short sequences,
// bytetransformer/src/attention_fused_long.cu:171-312 and the grouped-GEMM path
// of bytetransformer/src/cutlass_attention.cu:150-210 for long ones).  One
// templated kernel, two instantiations:
//   TILES = 1  short sequences (max length <= 128): 128 query rows per CTA,
//              192 threads, two CTAs per SM overlap each other's phases;
//   TILES = 2  long sequences: 256 query rows per CTA as two 128-row tiles that
//              ping-pong on the tensor core (while one tile's softmax runs, the
//              other tile's QK^T / PV MMAs execute), 320 threads, one CTA per SM.
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
//   S = Q K^T      128x128x64  -> tensor memory, 128 columns per tile
//   P = 2^(c*S-m)  fp16, written into 128B-swizzled shared memory (A operand)
//   O += P V       128x64x128  -> tensor memory, 64 columns per tile; V is
//                  consumed MN-major exactly as it lies in the QKV buffer
// O stays in tensor memory across key tiles.  The exponent reference m only
// moves when the running maximum grows by more than 2^8 (then the O row is
// rescaled in tensor memory); otherwise P simply grows up to 2^8, which fp16
// holds, and the final division by the row sum makes the result exact.
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
constexpr int kPBytes = kQRows * kKvRows * 2;   // 32 KiB
constexpr float kRescaleThreshold = 8.0f;       // log2 units

template <int TILES>
struct MhaCfg {
  static constexpr int kStages = TILES == 2 ? 3 : 2;
  static constexpr int kThreads = 64 + 128 * TILES;
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemK = kSmemQ + TILES * kTileBytes;
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr int kSmemP = kSmemV + kStages * kTileBytes;
  static constexpr int kSmemBar = kSmemP + TILES * kPBytes;
  static constexpr int kSmemBytes = kSmemBar + 256;
  static constexpr int kTmemCols = TILES == 2 ? 512 : 256;
  static constexpr uint32_t kTmemO = TILES * 128;  // S tiles first, then O tiles
  static constexpr int kMinBlocks = TILES == 2 ? 1 : 2;
};

struct MhaArgs {
  __half* ctx;
  const int* batch_idx;
  int hidden;
  float scale_log2e;
  int* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Row maximum of S over the valid keys.  The next 32-column chunk is requested from
// tensor memory before the current one is reduced, so only the first load is exposed.
template <bool MASKED>
__device__ __forceinline__ float chunk_max(const uint32_t (&v)[32], int cbase, int kv_valid) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    m0 = fmaxf(m0, (!MASKED || cbase + i < kv_valid) ? __uint_as_float(v[i]) : -INFINITY);
    m1 = fmaxf(m1, (!MASKED || cbase + i + 1 < kv_valid) ? __uint_as_float(v[i + 1]) : -INFINITY);
    m2 = fmaxf(m2, (!MASKED || cbase + i + 2 < kv_valid) ? __uint_as_float(v[i + 2]) : -INFINITY);
    m3 = fmaxf(m3, (!MASKED || cbase + i + 3 < kv_valid) ? __uint_as_float(v[i + 3]) : -INFINITY);
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
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

// One 32-column chunk: p = 2^(c*s - m_ref) (0 for masked keys), partial row sums, running
// raw maximum, fp16 pack and store into the 128B-swizzled P row.
template <bool MASKED>
__device__ __forceinline__ void chunk_softmax(const uint32_t (&v)[32], int cbase, int kv_valid, float c, float m_ref,
                                              uint8_t* p_row, int sw, float (&l)[4], float (&mx)[4]) {
  float p[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float s = __uint_as_float(v[i]);
    const float e = ex2_approx(fmaf(s, c, -m_ref));
    const bool ok = !MASKED || (cbase + i < kv_valid);
    p[i] = ok ? e : 0.f;
    mx[i & 3] = fmaxf(mx[i & 3], ok ? s : -INFINITY);
    l[i & 3] += p[i];
  }
#pragma unroll
  for (int u4 = 0; u4 < 4; ++u4) {
    const int u = (cbase >> 3) + u4;  // 16-byte unit index along the 128 keys
    uint4 w;
    w.x = pack_half2(p[u4 * 8 + 0], p[u4 * 8 + 1]);
    w.y = pack_half2(p[u4 * 8 + 2], p[u4 * 8 + 3]);
    w.z = pack_half2(p[u4 * 8 + 4], p[u4 * 8 + 5]);
    w.w = pack_half2(p[u4 * 8 + 6], p[u4 * 8 + 7]);
    *reinterpret_cast<uint4*>(p_row + (u >> 3) * (kQRows * 128) + (((u & 7) ^ sw) << 4)) = w;
  }
}
template <bool MASKED>
__device__ __forceinline__ void tile_softmax(uint32_t t_s, int kv_valid, float c, float m_ref, uint8_t* p_row, int sw,
                                             float& l_tile, float& mx_tile) {
  float l[4] = {0.f, 0.f, 0.f, 0.f};
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  uint32_t va[32], vb[32];
  tmem_ld_32x32(t_s, va);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 32, vb);  // in flight while chunk 0 is processed
  chunk_softmax<MASKED>(va, 0, kv_valid, c, m_ref, p_row, sw, l, mx);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 64, va);
  chunk_softmax<MASKED>(vb, 32, kv_valid, c, m_ref, p_row, sw, l, mx);
  tmem_ld_wait();
  tmem_ld_32x32(t_s + 96, vb);
  chunk_softmax<MASKED>(va, 64, kv_valid, c, m_ref, p_row, sw, l, mx);
  tmem_ld_wait();
  chunk_softmax<MASKED>(vb, 96, kv_valid, c, m_ref, p_row, sw, l, mx);
  l_tile = (l[0] + l[1]) + (l[2] + l[3]);
  mx_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

template <int TILES>
__global__ void __launch_bounds__(MhaCfg<TILES>::kThreads, MhaCfg<TILES>::kMinBlocks)
mha_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const MhaArgs args) {
  using Cfg = MhaCfg<TILES>;
  constexpr int kStages = Cfg::kStages;
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
  const int n_kv = (L + kKvRows - 1) / kKvRows;

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
      // K-major operands (Q, K, P): 8-row groups 1024 B apart.
      constexpr uint64_t kDescK = make_smem_desc_hi(16, 1024);
      // V: MN-major, one 64-wide chunk (LBO unused), 8-key groups 1024 B apart.
      constexpr uint64_t kDescV = make_smem_desc_hi(kTileBytes, 1024);
      constexpr uint32_t kIdescS = make_idesc_f16(128, 128, 0, 0);
      constexpr uint32_t kIdescO = make_idesc_f16(128, 64, 0, 1);
      const uint32_t s_q = smem_u32(smem + Cfg::kSmemQ);
      const uint32_t s_k = smem_u32(smem + Cfg::kSmemK);
      const uint32_t s_v = smem_u32(smem + Cfg::kSmemV);
      const uint32_t s_p = smem_u32(smem + Cfg::kSmemP);
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
        const uint32_t sp = s_p + t * kPBytes;
        const uint32_t sv = s_v + stage * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kKvRows / 16; ++kk) {
          const uint32_t pa = sp + (kk >> 2) * (kQRows * 128) + (kk & 3) * 32;
          umma_f16_ss(tmem_base + Cfg::kTmemO + t * 64, smem_desc(kDescK, pa), smem_desc(kDescV, sv + kk * 2048),
                      kIdescO, (accumulate || kk != 0) ? 1u : 0u);
        }
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
        // ---- tile 0: O0 += P0 V(j), then S0(j+1)
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
      uint8_t* p_row = smem + Cfg::kSmemP + t * kPBytes + r * 128;
      const int sw = r & 7;
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
        // The exponent reference m_ref is known from earlier key tiles (for the first
        // tile it is this tile's own row maximum), so one pass over S suffices: it
        // computes 2^(c*s - m_ref), the row sum AND the row maximum.  Only if the maximum
        // outgrew m_ref by more than 2^8 is the O row rescaled and the pass repeated.
        if (j == 0) m_ref = c * (full_tile ? tile_row_max<false>(t_s, kv_valid) : tile_row_max<true>(t_s, kv_valid));
        float l_tile, mx_tile;
        if (full_tile)
          tile_softmax<false>(t_s, kv_valid, c, m_ref, p_row, sw, l_tile, mx_tile);
        else
          tile_softmax<true>(t_s, kv_valid, c, m_ref, p_row, sw, l_tile, mx_tile);
        if (j > 0) {
          const float m_new = fmaxf(m_ref, mx_tile * c);
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
            tmem_st_wait();
            l_run *= f;
            m_ref = m_new;
            if (full_tile)
              tile_softmax<false>(t_s, kv_valid, c, m_ref, p_row, sw, l_tile, mx_tile);
            else
              tile_softmax<true>(t_s, kv_valid, c, m_ref, p_row, sw, l_tile, mx_tile);
          }
        }
        l_run += l_tile;
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
        }
        fence_proxy_async_smem();
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

template <int TILES>
cudaError_t launch_tiles(const MhaLaunch& a, const MhaArgs& args, cudaStream_t stream) {
  using Cfg = MhaCfg<TILES>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(mha_fwd_kernel<TILES>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const int rows_per_cta = kQRows * TILES;
  dim3 grid((a.max_len + rows_per_cta - 1) / rows_per_cta, a.head_num, a.batch);
  return launch_pdl(mha_fwd_kernel<TILES>, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, a.tm_qkv, args);
}

long long g_dbg_force_tiles = 0;

}  // namespace

cudaError_t launch_mha(const MhaLaunch& a, cudaStream_t stream) {
  if (a.batch <= 0 || a.max_len <= 0 || a.head_num <= 0) return cudaErrorInvalidValue;
  MhaArgs args;
  args.ctx = a.ctx;
  args.batch_idx = a.batch_idx;
  args.hidden = a.hidden;
  args.scale_log2e = a.scale_log2e;
  args.status = a.status;
  // Measured on B200 (18.9k packed tokens, 12 heads): the one-tile variant with two
  // co-resident CTAs per SM is faster at every length from 64 to 1024 (404 vs 372
  // TFLOP/s at 1024), so it is the default; the two-tile variant stays selectable.
  int tiles = 1;
  if (g_dbg_force_tiles == 1 || g_dbg_force_tiles == 2) tiles = static_cast<int>(g_dbg_force_tiles);
  return tiles == 1 ? launch_tiles<1>(a, args, stream) : launch_tiles<2>(a, args, stream);
}

}  // namespace bt

// Diagnostics hook (not part of the stable ABI): 0 = choose by max length,
// 1 / 2 = force the short / long attention variant.
extern "C" int bt_debug_set_mha_tiles(long long tiles) {
  bt::g_dbg_force_tiles = tiles;
  return 0;
}
