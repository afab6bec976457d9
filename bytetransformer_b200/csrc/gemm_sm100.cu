// Dense fp16 GEMM for sm_100a:  out[M,N] = epilogue(A[M,K] * W[K,N]),  fp32 accumulation.
//
// Replaces the reference's cuBLAS / CUTLASS-2.x calls on the encoder path
// (bytetransformer/src/gemm.cu:32-39, bytetransformer/src/gemm_bias_act.cu:76-148).
//
// Two persistent kernels share one epilogue:
//
//  gemm_f16_kernel<BLOCK_N, EPI>      one CTA per SM, tile 128 x BLOCK_N (256/128/64),
//                                     tcgen05.mma.cta_group::1.
//  gemm_f16_pair_kernel<EPI>          clusters of two CTAs on an SM pair, tile 256 x 256:
//                                     each CTA loads its 128 rows of A and HALF of the W
//                                     tile (128 of the 256 columns); the leader CTA issues
//                                     tcgen05.mma.cta_group::2 (M = 256), which feeds both
//                                     SMs' tensor cores from the two halves.  Per SM this
//                                     halves the shared-memory fill and the L2 traffic of
//                                     W and makes room for a 6-stage ring.  Used whenever
//                                     the problem has enough 256-row tiles.
//
// Roles in every CTA (320 threads):
//   warp 0      TMA producer: A tile [128 x 64] (K-major) and W tile [64 x n] (N contiguous
//               = MN-major for UMMA, so the reference's [in,out] weight layout is consumed
//               as is, no transposed copy) into a 128B-swizzled shared-memory ring.
//   warp 1      allocates tensor memory and (leader only, for the pair kernel) issues the
//               MMAs from one lane; accumulators are double buffered in tensor memory
//               (2 x 256 columns) so the epilogue of tile i overlaps the main loop of i+1.
//   warps 2..9  epilogue: tcgen05.ld -> +bias -> GELU / +residual -> fp16 (or fp32)
//               -> 128B-swizzled staging rows in shared memory -> TMA bulk store
//               (full 128-byte lines); a 32-row slab that crosses M falls back to
//               row-predicated 16-byte stores, so rows >= M are never written.
// M is read from device memory (the packed token count is only known on the device), so
// the host never blocks; the grid is sized from the allocated rows.  Every mbarrier wait
// is bounded: on expiry the CTA records a code in the status word and all roles drain to
// a common exit that frees tensor memory.  No TMA load uses cluster multicast.
#include "common.cuh"
#include "kernels.h"
#include "../../include/bt_b200.h"

namespace bt {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;
constexpr int kGemmThreads = 320;
constexpr int kEpiWarps = 8;
constexpr int kABytes = kBlockM * kBlockK * 2;  // 16 KiB
constexpr int kStagingBytesPerWarp = 32 * 128;  // 32 rows x 128 B

template <int BLOCK_N>
struct GemmCfg {
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BLOCK_N == 256) ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BLOCK_N;
  // Output leaves through per-warp staging rows + TMA bulk stores when a warp's
  // column share is at least 128 bytes wide (BLOCK_N >= 128).
  static constexpr bool kTmaStore = BLOCK_N >= 128;
  static constexpr int kStagingBytes = kEpiWarps * kStagingBytesPerWarp;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

// Pair kernel: per CTA 128 rows of A and 128 of the tile's 256 W columns per stage.
struct PairCfg {
  static constexpr int kTileN = 256;
  static constexpr int kBHalfBytes = 128 * kBlockK * 2;  // 16 KiB
  static constexpr int kStageBytes = kABytes + kBHalfBytes;
  static constexpr int kStages = 6;
  static constexpr int kTmemCols = 512;
  static constexpr int kStagingBufs = 1;  // per epilogue warp (two were measured: no gain, and they cost a stage)
  static constexpr int kStagingBytes = kStagingBufs * kEpiWarps * kStagingBytesPerWarp;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 256;
};

struct GemmArgs {
  __half* out;
  const __half* bias;
  const __half* residual;
  const int* m_dev;
  int m_rows;
  int N;
  int K;
  int gelu_kind;
  int* status;
  // fused LayerNorm (BT_EPI_BIAS_RESIDUAL_LAYERNORM): `out` is the scratch for the row
  // statistics partials (8 * N/128 bytes per row), `out_ln` the fp16 result
  __half* out_ln;
  const void* gamma;
  const void* beta;
  int gb_fp32;
  float eps;
  uint32_t ln_epoch;  // fused LayerNorm: tag of this launch in the statistics scratch (see gemm_f16_ln_kernel)
  // split-K (kEpiSplitKF32): K is cut into `split_k` ranges, range s writes its fp32 partial sum to
  // out + s * split_stride floats; range 0 also adds bias and residual
  int split_k;
  long long split_stride;
  int early_w;  // one-CTA kernel: request the first tile's W blocks before the wait for the kernel before
  long long* timing;  // diagnostics: clock64 stamps per CTA and tile (null = off)
  uint64_t a_desc_hi;
  uint64_t b_desc_hi;
  uint32_t a_kstep_bytes;
  uint32_t b_kstep_bytes;
  uint32_t idesc;
};

// Debug overrides (0 = default): W descriptor fields, forced tile width, pair kernel on/off.
long long* g_dbg_gemm_timing = nullptr;  // [148 CTAs][16 tiles][8 slots]
__device__ __forceinline__ void gstamp(long long* timing, int it, int slot) {
  if (timing != nullptr && it < 16 && blockIdx.x < 148) timing[(blockIdx.x * 16 + it) * 8 + slot] = clock64();
}
long long g_dbg_b_lbo = 0, g_dbg_b_sbo = 0, g_dbg_b_kstep = 0, g_dbg_force_block_n = 0, g_dbg_pair_mode = 0;
long long g_dbg_early_w = 1;  // 1 = W blocks of the first tile requested before the dependency wait
long long g_dbg_ln_pair = 0;  // GEMM + LayerNorm on SM pairs: 0 = for K >= 2048 (default), 1 = always, anything else = never
long long g_dbg_split_k = 0;  // 0 = policy, < 0 = never, > 0 = that many ranges whenever the shape allows

// ------------------------------------------------------------------------------------------
// Epilogue of one 128 x TILE_N accumulator tile, executed by the 8 epilogue warps of a CTA.
// The warp owns TMEM lanes (warp_id % 4) * 32 .. +31 (`quarter`) and one half of the tile's
// columns (`col_half`).  `tm_out` is the store map (box 128 B x 32 rows).
// ------------------------------------------------------------------------------------------
template <int N>
__device__ __forceinline__ void tma_store_wait_read_n() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// STG_BUFS staging buffers of 32 rows x 128 B per warp are used in turn, so a bulk store
// only has to wait for the store issued STG_BUFS chunks earlier.  The accumulator chunk
// c+1 is requested from tensor memory before chunk c is processed.
template <int TILE_N, int EPI, bool TMA_STORE, int STG_BUFS>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& args, const CUtensorMap* tm_out, uint8_t* stg,
                                              uint32_t tmem_acc, int m0, int n0, int M, int quarter, int col_half,
                                              int lane, const uint4* resv, int split = 0) {
  constexpr int kColsPerWarp = TILE_N / 2;
  constexpr bool kSplitK = (EPI == kEpiSplitKF32);
  constexpr bool kF32Out = (EPI == BT_EPI_BIAS_RESIDUAL_F32OUT) || kSplitK;
  constexpr bool kHasResidual = (EPI == BT_EPI_BIAS_RESIDUAL || EPI == BT_EPI_BIAS_RESIDUAL_F32OUT) || kSplitK;
  static_assert(!(kSplitK && TMA_STORE), "split-K partials are stored by the threads");
  // 128 bytes of output per row and chunk: 32 fp32 or 64 fp16 columns.
  constexpr int kChunk = kF32Out ? 32 : (kColsPerWarp >= 64 ? 64 : 32);
  constexpr int kNChunks = kColsPerWarp / kChunk;
  constexpr int kHalves = kChunk / 32;  // tcgen05.ld x32 per chunk
  const int row0 = m0 + quarter * 32;
  const int row = row0 + lane;
  const bool row_ok = row < M;
  const bool slab_full = TMA_STORE && (row0 + 32 <= M);  // all 32 rows valid: bulk store, else predicated stores
  const uint32_t t_row = tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + col_half * kColsPerWarp;
  uint32_t raw[2][kHalves][32];
#pragma unroll
  for (int h = 0; h < kHalves; ++h) tmem_ld_32x32(t_row + h * 32, raw[0][h]);
  tmem_ld_wait();
#pragma unroll
  for (int ci = 0; ci < kNChunks; ++ci) {
    const int c = ci * kChunk;
    const int col = col_half * kColsPerWarp + c;  // column inside the tile
    const int gcol = n0 + col;
    if (ci + 1 < kNChunks) {
#pragma unroll
      for (int h = 0; h < kHalves; ++h) tmem_ld_32x32(t_row + c + kChunk + h * 32, raw[(ci + 1) & 1][h]);
    }
    float v[kChunk];
#pragma unroll
    for (int h = 0; h < kHalves; ++h)
#pragma unroll
      for (int i = 0; i < 32; ++i) v[h * 32 + i] = __uint_as_float(raw[ci & 1][h][i]);
    if (EPI != BT_EPI_NONE && (!kSplitK || split == 0)) {
      const uint4* bp = reinterpret_cast<const uint4*>(args.bias + gcol);
#pragma unroll
      for (int q = 0; q < kChunk / 8; ++q) {
        const uint4 b4 = __ldg(bp + q);
        const __half2* bh = reinterpret_cast<const __half2*>(&b4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(bh[j]);
          v[q * 8 + 2 * j] += f.x;
          v[q * 8 + 2 * j + 1] += f.y;
        }
      }
    }
    if (EPI == BT_EPI_BIAS_GELU) {
      if (args.gelu_kind == BT_GELU_TANH) {
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[i] = gelu_tanh(v[i]);
      } else {
#pragma unroll
        for (int i = 0; i < kChunk; i += 2) gelu_erf_fast_pair(v[i], v[i + 1]);
      }
    }
    const size_t off = static_cast<size_t>(row) * args.N + gcol +
                       (kSplitK ? static_cast<size_t>(split) * static_cast<size_t>(args.split_stride) : 0);
    if (kHasResidual) {
#pragma unroll
      for (int q = 0; q < kChunk / 8; ++q) {
        const uint4 r4 = resv[c / 8 + q];
        const __half2* rh = reinterpret_cast<const __half2*>(&r4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(rh[j]);
          v[q * 8 + 2 * j] += f.x;
          v[q * 8 + 2 * j + 1] += f.y;
        }
      }
    }
    // 8 (or 4) units of 16 bytes per row
    constexpr int kUnits = kF32Out ? 8 : kChunk / 8;
    uint4 units[kUnits];
    if (kF32Out) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        units[q] = make_uint4(__float_as_uint(v[q * 4]), __float_as_uint(v[q * 4 + 1]), __float_as_uint(v[q * 4 + 2]),
                              __float_as_uint(v[q * 4 + 3]));
    } else {
#pragma unroll
      for (int q = 0; q < kChunk / 8; ++q) {
        units[q].x = pack_half2(v[q * 8 + 0], v[q * 8 + 1]);
        units[q].y = pack_half2(v[q * 8 + 2], v[q * 8 + 3]);
        units[q].z = pack_half2(v[q * 8 + 4], v[q * 8 + 5]);
        units[q].w = pack_half2(v[q * 8 + 6], v[q * 8 + 7]);
      }
    }
    if (slab_full) {
      // the bulk store that last used this staging buffer must have finished reading it
      if (lane == 0) tma_store_wait_read_n<STG_BUFS - 1>();
      __syncwarp();
      uint8_t* sbuf = stg + (STG_BUFS == 2 ? (ci & 1) * kStagingBytesPerWarp : 0);
      uint8_t* srow = sbuf + lane * 128;
#pragma unroll
      for (int q = 0; q < kUnits; ++q) *reinterpret_cast<uint4*>(srow + ((q ^ (lane & 7)) << 4)) = units[q];
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(tm_out, sbuf, gcol, row0);
        tma_store_commit();
      }
    } else if (row_ok) {
      uint4* op = kF32Out ? reinterpret_cast<uint4*>(reinterpret_cast<float*>(args.out) + off)
                          : reinterpret_cast<uint4*>(args.out + off);
#pragma unroll
      for (int q = 0; q < kUnits; ++q) op[q] = units[q];
    }
    if (ci + 1 < kNChunks) tmem_ld_wait();
  }
}

// The residual slice of a thread's row, fetched before the accumulator is waited for so that
// its latency hides behind the main loop of the tile.
template <int TILE_N, int EPI>
__device__ __forceinline__ void prefetch_residual(const GemmArgs& args, int m0, int n0, int M, int quarter,
                                                  int col_half, int lane, uint4* resv, int split = 0) {
  constexpr int kColsPerWarp = TILE_N / 2;
  constexpr bool kHasResidual = (EPI == BT_EPI_BIAS_RESIDUAL || EPI == BT_EPI_BIAS_RESIDUAL_F32OUT ||
                                 EPI == BT_EPI_BIAS_RESIDUAL_LAYERNORM || EPI == kEpiSplitKF32);
  if (kHasResidual) {
    const int row = m0 + quarter * 32 + lane;
    const bool row_ok = row < M && split == 0;  // only the first K range carries the residual
    const uint4* rp = reinterpret_cast<const uint4*>(args.residual + static_cast<size_t>(row) * args.N + n0 +
                                                     col_half * kColsPerWarp);
#pragma unroll
    for (int q = 0; q < kColsPerWarp / 8; ++q) resv[q] = row_ok ? __ldg(rp + q) : make_uint4(0u, 0u, 0u, 0u);
  }
}

// ------------------------------------------------------------------------------------------
// One CTA per SM, tile 128 x BLOCK_N.
// ------------------------------------------------------------------------------------------
template <int BLOCK_N, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_out, const GemmArgs args) {
  using Cfg = GemmCfg<BLOCK_N>;
  constexpr int kStages = Cfg::kStages;
  constexpr bool kSplitK = (EPI == kEpiSplitKF32);
  constexpr bool kHasResidual = (EPI == BT_EPI_BIAS_RESIDUAL || EPI == BT_EPI_BIAS_RESIDUAL_F32OUT) || kSplitK;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kStagingBytes);
  uint64_t* full_bar = bars;                    // [kStages]
  uint64_t* empty_bar = bars + kStages;         // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;      // [2]
  uint64_t* acc_empty = bars + 2 * kStages + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_out);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_tiles = args.N / BLOCK_N;
  const int splits = kSplitK ? args.split_k : 1;
  const int num_kb = args.K / kBlockK / splits;  // K blocks per tile (per K range with split-K)
  // Tile number -> (K range, column block, row block).  The K range and the column block come from
  // the low part of the number, so those of a CTA's first tile (number blockIdx.x) are known before
  // the row count is.
  auto tile_cols = [&](int tile, int& n0, int& sp) -> int {
    sp = 0;
    if (kSplitK) {
      sp = tile % splits;
      tile /= splits;
    }
    n0 = (tile % n_tiles) * BLOCK_N;
    return tile / n_tiles;
  };
  // The weights are written by no kernel of the chain, so the W blocks of the first tile are
  // requested before the wait for the kernel before (whose tail they then overlap): the first
  // `pre_kb` stages get their full byte count armed and their W part requested here, their A
  // part after the wait.
  const int pre_kb = args.early_w ? (num_kb < kStages ? num_kb : kStages) : 0;
  if (warp == 0 && lane == 0) {
    int n0 = 0, sp = 0;
    tile_cols(static_cast<int>(blockIdx.x), n0, sp);
    for (int kb = 0; kb < pre_kb; ++kb) {
      uint8_t* sb = smem + kb * Cfg::kStageBytes + kABytes;
      mbar_arrive_expect_tx(&full_bar[kb], Cfg::kStageBytes);
#pragma unroll
      for (int c = 0; c < BLOCK_N / 64; ++c)
        tma_load_2d(sb + c * (64 * kBlockK * 2), &tm_b, &full_bar[kb], n0 + c * 64, (sp * num_kb + kb) * kBlockK);
    }
  } else if (warp >= 2 && EPI != BT_EPI_NONE && args.early_w && args.bias != nullptr) {
    // the bias slice of the first tile, for the same reason
    int n0 = 0, sp = 0;
    tile_cols(static_cast<int>(blockIdx.x), n0, sp);
    const __half* bp = args.bias + n0 + ((warp - 2) >> 2) * (BLOCK_N / 2);
    if (lane * 64 < BLOCK_N / 2) prefetch_l1(bp + lane * 64);
  }

  // Everything above touched only this CTA's own resources and the weights; from here on global
  // memory written by earlier kernels is read.  The A blocks of the armed stages go first, before
  // the row count is known: the first tile's rows lie inside the allocation whether or not they
  // are valid, and a CTA that turns out to have no tile only has to wait for them.
  pdl_wait();
  if (warp == 0 && lane == 0 && pre_kb > 0) {
    int n0 = 0, sp = 0;
    const int m0 = tile_cols(static_cast<int>(blockIdx.x), n0, sp) * kBlockM;
    for (int kb = 0; kb < pre_kb; ++kb)
      tma_load_2d(smem + kb * Cfg::kStageBytes, &tm_a, &full_bar[kb], (sp * num_kb + kb) * kBlockK, m0);
  }
  int M = args.m_rows;
  if (args.m_dev != nullptr) {
    const int md = __ldg(args.m_dev);
    M = md < M ? md : M;
  }
  const int m_tiles = (M + kBlockM - 1) / kBlockM;
  const int total_tiles = m_tiles * n_tiles * splits;
  // The li-th tile of this CTA: tiles go round-robin over the CTAs.  With split-K a tile is an
  // (output tile, K range) pair; `sp` is the range.
  auto tile_at = [&](int li, int& m0, int& n0, int& sp) -> bool {
    const int tile = static_cast<int>(blockIdx.x) + li * static_cast<int>(gridDim.x);
    if (tile >= total_tiles) return false;
    m0 = tile_cols(tile, n0, sp) * kBlockM;
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int m0 = 0, n0 = 0, sp = 0;
      if (!tile_at(0, m0, n0, sp)) {
        // No tile for this CTA after all (fewer valid rows than allocated): wait for the armed
        // stages, so that no copy is in flight at exit.
        for (int kb = 0; kb < pre_kb; ++kb)
          if (!mbar_wait_bounded(&full_bar[kb], 0u, abort_flag, args.status, kStatusGemmProducerTimeout)) break;
      }
      for (int li = 0; ok && tile_at(li, m0, n0, sp); ++li) {
        for (int i = 0; i < num_kb; ++i) {
          const int kb = sp * num_kb + i;
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + kABytes;
          if (li == 0 && i < pre_kb) {
            // armed and requested above (stage == i here)
          } else {
            if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, args.status,
                                   kStatusGemmProducerTimeout)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
            tma_load_2d(sa, &tm_a, &full_bar[stage], kb * kBlockK, m0);
#pragma unroll
            for (int c = 0; c < BLOCK_N / 64; ++c)
              tma_load_2d(sb + c * (64 * kBlockK * 2), &tm_b, &full_bar[stage], n0 + c * 64, kb * kBlockK);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int m0 = 0, n0 = 0, sp = 0;
      for (int it = 0; ok && tile_at(it, m0, n0, sp); ++it) {
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aphase ^ 1u, abort_flag, args.status, kStatusGemmMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        gstamp(args.timing, it, 0);
        const uint32_t d_tmem = tmem_base + as * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, args.status, kStatusGemmMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint64_t adesc = smem_desc(args.a_desc_hi, sa + k * args.a_kstep_bytes);
            const uint64_t bdesc = smem_desc(args.b_desc_hi, sb + k * args.b_kstep_bytes);
            umma_f16_ss(d_tmem, adesc, bdesc, args.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
        gstamp(args.timing, it, 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int e = warp - 2;
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    const int col_half = e >> 2;   // which half of the tile's columns
    uint8_t* stg = smem + kStages * Cfg::kStageBytes + e * kStagingBytesPerWarp;  // 32 rows x 128 B, swizzled
    int m0 = 0, n0 = 0, sp = 0;
    for (int it = 0; tile_at(it, m0, n0, sp); ++it) {
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      uint4 resv[kHasResidual ? BLOCK_N / 16 : 1];
      prefetch_residual<BLOCK_N, EPI>(args, m0, n0, M, quarter, col_half, lane, resv, sp);
      if (!mbar_wait_bounded(&acc_full[as], aphase, abort_flag, args.status, kStatusGemmEpilogueTimeout)) break;
      tc_fence_after();
      if (warp == 2 && lane == 0) gstamp(args.timing, it, 2);
      epilogue_tile<BLOCK_N, EPI, Cfg::kTmaStore, 1>(args, &tm_out, stg, tmem_base + as * BLOCK_N, m0, n0, M, quarter,
                                                  col_half, lane, resv, sp);
      if (warp == 2 && lane == 0) gstamp(args.timing, it, 3);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
    }
    if (Cfg::kTmaStore && lane == 0) tma_store_wait_all();  // staging rows must outlive the last bulk store
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag != 0) {
    // A wait ran out somewhere: give copies that may still be in flight time to
    // land before the CTA's shared memory is handed to another block.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// Two CTAs per cluster (an SM pair), tile 256 x 256, tcgen05.mma.cta_group::2.
// CTA rank r of the pair owns rows m0 + r*128 .. +127 (its own accumulator in its own tensor
// memory) and stages W columns n0 + r*128 .. +127.  Barriers:
//   full[s]      leader's copy only: 1 arrival (leader's expect_tx of BOTH CTAs' bytes); the
//                peer's TMA completes its bytes on the leader's barrier.
//   empty[s]     one per CTA, arrived by the leader's commit multicast to both CTAs.
//   acc_full[a]  one per CTA, same multicast commit.
//   acc_empty[a] leader's copy only: 16 arrivals (8 epilogue warps of each CTA).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion is counted on a barrier that may live in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once every
// tcgen05 operation issued so far has retired.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_f16_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ CUtensorMap tm_out, const GemmArgs args) {
  using Cfg = PairCfg;
  constexpr int kStages = Cfg::kStages;
  constexpr int kTileN = Cfg::kTileN;
  constexpr bool kHasResidual = (EPI == BT_EPI_BIAS_RESIDUAL || EPI == BT_EPI_BIAS_RESIDUAL_F32OUT);

  extern __shared__ uint8_t smem_raw[];
  // Both CTAs of the pair must use identical shared-memory offsets (the MMA and the multicast
  // commit address the peer by offset); dynamic shared memory starts at the same offset in
  // every CTA of a launch, so the same round-up applies to both.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kStagingBytes);
  uint64_t* full_bar = bars;                    // [kStages]  (leader's copy is the live one)
  uint64_t* empty_bar = bars + kStages;         // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;      // [2]
  uint64_t* acc_empty = bars + 2 * kStages + 2; // [2]        (leader's copy is the live one)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
  const bool leader = cta_rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 2 * kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();  // see gemm_f16_kernel
  int M = args.m_rows;
  if (args.m_dev != nullptr) {
    const int md = __ldg(args.m_dev);
    M = md < M ? md : M;
  }
  const int n_tiles = args.N / kTileN;
  const int m_tiles = (M + 2 * kBlockM - 1) / (2 * kBlockM);
  const int total_tiles = m_tiles * n_tiles;
  const int num_kb = args.K / kBlockK;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_a);
      tma_prefetch_desc(&tm_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters) {
        const int m0 = (tile / n_tiles) * (2 * kBlockM) + static_cast<int>(cta_rank) * kBlockM;
        const int n0 = (tile % n_tiles) * kTileN + static_cast<int>(cta_rank) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, args.status,
                                 kStatusGemmProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + kABytes;
          // the leader announces the bytes of both CTAs; all copies complete on its barrier
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &tm_a, bar, kb * kBlockK, m0);
          tma_load_2d_pair(sb, &tm_b, bar, n0, kb * kBlockK);
          tma_load_2d_pair(sb + 64 * kBlockK * 2, &tm_b, bar, n0 + 64, kb * kBlockK);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters, ++it) {
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aphase ^ 1u, abort_flag, args.status, kStatusGemmMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        gstamp(args.timing, it, 0);
        const uint32_t d_tmem = tmem_base + as * kTileN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, args.status, kStatusGemmMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint64_t adesc = smem_desc(args.a_desc_hi, sa + k * args.a_kstep_bytes);
            const uint64_t bdesc = smem_desc(args.b_desc_hi, sb + k * args.b_kstep_bytes);
            umma_f16_ss_pair(d_tmem, adesc, bdesc, args.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);  // frees the stage in both CTAs
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit_pair(&acc_full[as]);
        gstamp(args.timing, it, 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int e = warp - 2;
    const int quarter = warp & 3;
    const int col_half = e >> 2;
    uint8_t* stg = smem + kStages * Cfg::kStageBytes + e * (Cfg::kStagingBufs * kStagingBytesPerWarp);
    int it = 0;
    for (int tile = cluster_id; tile < total_tiles; tile += num_clusters, ++it) {
      const int m0 = (tile / n_tiles) * (2 * kBlockM) + static_cast<int>(cta_rank) * kBlockM;
      const int n0 = (tile % n_tiles) * kTileN;
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      uint4 resv[kHasResidual ? kTileN / 16 : 1];
      prefetch_residual<kTileN, EPI>(args, m0, n0, M, quarter, col_half, lane, resv);
      if (!mbar_wait_bounded(&acc_full[as], aphase, abort_flag, args.status, kStatusGemmEpilogueTimeout)) break;
      tc_fence_after();
      if (warp == 2 && lane == 0) gstamp(args.timing, it, 2);
      epilogue_tile<kTileN, EPI, true, Cfg::kStagingBufs>(args, &tm_out, stg, tmem_base + as * kTileN, m0, n0, M,
                                                          quarter, col_half, lane, resv);
      if (warp == 2 && lane == 0) gstamp(args.timing, it, 3);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[as]), 0));
    }
    if (lane == 0) tma_store_wait_all();
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------
// GEMM + bias + residual + LayerNorm in one kernel:  y = LN(A*W + bias + residual)*gamma + beta.
// Same tiles, schedule and main loop as gemm_f16_kernel<256, .>: tile t = (row tile t / C,
// column tile t % C), C = N/256, tiles round-robin over the CTAs, so the C column tiles of a
// row tile are worked on by C neighbouring CTAs at about the same time.  The fp32 sums stay
// in tensor memory; the pre-normalisation tensor never goes to HBM.  Every epilogue thread
// owns one row and 128 of its columns:
//   1. v = accumulator + bias + residual, written back to tensor memory, with the sum and
//      sum of squares of v - s (s = the thread's first value: shifted one-pass statistics);
//   2. the partial (mean_i, M2_i) goes to a global scratch row (it stays in L2) as two 64-bit
//      words, each (value bits << 32 | epoch of this launch): an aligned 64-bit store is
//      single-copy atomic, so the tag validates the value and no fence or counter is needed;
//   3. the thread polls (bounded) the 2 * 2*C words of its row until all carry the epoch and
//      merges the 2*C partials (equal counts):
//         mean = avg(mean_i),  M2 = sum(M2_i) + 128 * sum((mean_i - mean)^2);
//   4. second read of tensor memory: normalise, gamma / beta, fp16, staging, TMA store.
// Accumulators are double buffered, so 1-4 of a tile overlap the main loop of the CTA's next
// tile.  A CTA only ever waits for the C CTAs working on the same row tile, and those wait for
// nothing but that row tile in turn, so the waits are never circular.  Progress does need those
// C = N/256 neighbouring CTAs to be resident together: the grid never exceeds the SM count and a CTA
// takes a whole SM, so they are as soon as the kernels before have left; should something else hold
// SMs for long (another process, a hung kernel on another stream), the wait, bounded like every
// other wait of the library, gives up and reports kStatusGemmEpilogueTimeout instead of spinning.
// The scratch (16 * N/128 bytes per row) must not hold this launch's epoch in the low half of any
// word beforehand: the caller zeroes it once and numbers the launches that share it 1, 2, 3, ...
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_relaxed_gpu_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// The epilogue warps' loop of the GEMM + LayerNorm kernels (one-CTA and pair form share it): steps 1-4
// of the description above for every tile that `tile_at(it, m0, n0)` yields (m0 = first of this CTA's 128
// rows, n0 = first of the tile's 256 columns); `release_acc(as)` hands accumulator buffer `as` back to the
// MMA issuer.  `stg_base`: 8 staging buffers of 4 KB; `res_bar`: 8 barriers, one per epilogue warp.
template <class TileAt, class ReleaseAcc>
__device__ __forceinline__ void ln_epilogue_loop(const GemmArgs& args, const CUtensorMap* tm_out,
                                                 const CUtensorMap* tm_res, uint8_t* stg_base, uint64_t* acc_full,
                                                 uint64_t* vec_full, uint64_t* vec_empty, uint64_t* res_bar,
                                                 uint4* vec_s, volatile int* abort_flag, uint32_t tmem_base, int M,
                                                 int n_tiles, int warp, int lane, TileAt tile_at,
                                                 ReleaseAcc release_acc) {
  constexpr int kTileN = 256;
  constexpr int kColsPerThread = kTileN / 2;  // 128
  const int e = warp - 2;
  const int quarter = warp & 3;
  const int col_half = e >> 2;
  uint8_t* stg = stg_base + e * kStagingBytesPerWarp;
  const int parts = 2 * n_tiles;                        // partials per row
  const float inv_n = 1.0f / static_cast<float>(args.N);
  int m0 = 0, n0 = 0;
  for (int it = 0; tile_at(it, m0, n0); ++it) {
    const int as = it & 1;
    const uint32_t aphase = (it >> 1) & 1;
    const int row0 = m0 + quarter * 32;
    const int row = row0 + lane;
    const bool row_ok = row < M;
    const int gcol0 = n0 + col_half * kColsPerThread;  // first of this thread's 128 columns
    const int part = 2 * (n0 / kTileN) + col_half;
    // The first epilogue warp brings the tile's bias / gamma / beta slices into shared memory (every
    // thread re-reads them, and the residual loads below keep evicting them from L1).
    if (e == 0) {
      uint4 vb = __ldg(reinterpret_cast<const uint4*>(args.bias + n0) + lane);
      uint4 vg = make_uint4(0u, 0u, 0u, 0u), vt = vg;
      if (!args.gb_fp32) {
        vg = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(args.gamma) + n0) + lane);
        vt = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(args.beta) + n0) + lane);
      }
      if (!mbar_wait_bounded(vec_empty, (it & 1u) ^ 1u, abort_flag, args.status, kStatusGemmEpilogueTimeout)) break;
      vec_s[lane] = vb;
      vec_s[32 + lane] = vg;
      vec_s[64 + lane] = vt;
      __syncwarp();
      if (lane == 0) mbar_arrive(vec_full);
    }
    // Residual rows of this warp (32 rows x 128 columns) come through its staging buffer in two
    // TMA boxes of 64 columns: row-strided 16-byte loads from the threads would cost one L1 tag
    // look-up per lane and load (4096 per tile), which alone took longer than the main loop.
    // The first box is requested now, the second when the first has been read.
    if (lane == 0) {
      tma_store_wait_read_n<0>();  // the bulk stores of the previous tile have read the buffer
      mbar_arrive_expect_tx(&res_bar[e], kStagingBytesPerWarp);
      tma_load_2d(stg, tm_res, &res_bar[e], gcol0, row0);
    }
    if (!mbar_wait_bounded(&acc_full[as], aphase, abort_flag, args.status, kStatusGemmEpilogueTimeout)) break;
    tc_fence_after();
    if (!mbar_wait_bounded(vec_full, it & 1u, abort_flag, args.status, kStatusGemmEpilogueTimeout)) break;
    if (warp == 2 && lane == 0) gstamp(args.timing, it, 2);
    const uint4* sbias = vec_s + col_half * (kColsPerThread / 8);
    const uint4* sgamma = vec_s + 32 + col_half * (kColsPerThread / 8);
    const uint4* sbeta = vec_s + 64 + col_half * (kColsPerThread / 8);
    const uint32_t t_row = tmem_base + as * kTileN + (static_cast<uint32_t>(quarter * 32) << 16) +
                           col_half * kColsPerThread;
    // ---- 1. v = acc + bias + residual -> tensor memory; shifted sums
    float sd = 0.f, sdd = 0.f, shift0 = 0.f;
    unsigned long long sd2 = pack_f32x2(0.f, 0.f), sdd2 = sd2, nshift2 = sd2;
    {
      uint32_t raw[2][32];
      tmem_ld_32x32(t_row, raw[0]);
      bool res_ok = true;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        // this thread's 64 residual values of box hh: row `lane` of the swizzled buffer
        if (!mbar_wait_bounded(&res_bar[e], (static_cast<uint32_t>(it) * 2u + hh) & 1u, abort_flag, args.status,
                               kStatusGemmEpilogueTimeout)) {
          res_ok = false;
          break;
        }
        uint4 rres[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
          rres[q] = *reinterpret_cast<const uint4*>(stg + lane * 128 + ((q ^ (lane & 7)) << 4));
        if (hh == 0) {
          fence_proxy_async_smem();  // the reads above precede the next bulk write into the buffer
          __syncwarp();
          if (lane == 0) {
            mbar_arrive_expect_tx(&res_bar[e], kStagingBytesPerWarp);
            tma_load_2d(stg, tm_res, &res_bar[e], gcol0 + 64, row0);
          }
        }
#pragma unroll
        for (int cj = 0; cj < 2; ++cj) {
          const int ci = hh * 2 + cj;
          const int c = ci * 32;
          tmem_ld_wait();
          if (ci + 1 < kColsPerThread / 32) tmem_ld_32x32(t_row + c + 32, raw[(ci + 1) & 1]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 b4 = sbias[c / 8 + q];
            const __half2* bh = reinterpret_cast<const __half2*>(&b4);
            const __half2* rh = reinterpret_cast<const __half2*>(&rres[cj * 4 + q]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 fb = __half22float2(bh[j]);
              const float2 fr = __half22float2(rh[j]);
              const unsigned long long br2 = add_f32x2(pack_f32x2(fb.x, fb.y), pack_f32x2(fr.x, fr.y));
              const unsigned long long v2 = add_f32x2(
                  pack_f32x2(__uint_as_float(raw[ci & 1][q * 8 + 2 * j]), __uint_as_float(raw[ci & 1][q * 8 + 2 * j + 1])), br2);
              float v0, v1;
              unpack_f32x2(v2, v0, v1);
              if (ci == 0 && q == 0 && j == 0) {
                shift0 = v0;
                nshift2 = pack_f32x2(-v0, -v0);
              }
              const unsigned long long d2 = add_f32x2(v2, nshift2);
              sd2 = add_f32x2(sd2, d2);
              sdd2 = fma_f32x2(d2, d2, sdd2);
              raw[ci & 1][q * 8 + 2 * j] = __float_as_uint(v0);
              raw[ci & 1][q * 8 + 2 * j + 1] = __float_as_uint(v1);
            }
          }
          tmem_st_32x32(t_row + c, raw[ci & 1]);
        }
      }
      if (!res_ok) break;
      float s0, s1, q0, q1;
      unpack_f32x2(sd2, s0, s1);
      unpack_f32x2(sdd2, q0, q1);
      sd = s0 + s1;
      sdd = q0 + q1;
    }
    const float lmean = shift0 + sd * (1.0f / kColsPerThread);
    const float m2 = fmaxf(sdd - sd * sd * (1.0f / kColsPerThread), 0.f);
    if (warp == 2 && lane == 0) gstamp(args.timing, it, 4);
    // ---- 2. publish the partial: two 64-bit words, each (value bits << 32 | epoch).  A naturally
    // aligned 64-bit store is single-copy atomic, so a reader that finds this launch's epoch in a word
    // also has its value: no fence, no counter, no second round trip.
    const uint32_t epoch = args.ln_epoch;
    unsigned long long* words = reinterpret_cast<unsigned long long*>(args.out);
    if (row_ok) {
      unsigned long long* wp = words + (static_cast<size_t>(row) * parts + part) * 2;
      st_relaxed_gpu_u64(wp, (static_cast<unsigned long long>(__float_as_uint(lmean)) << 32) | epoch);
      st_relaxed_gpu_u64(wp + 1, (static_cast<unsigned long long>(__float_as_uint(m2)) << 32) | epoch);
    }
    if (warp == 2 && lane == 0) gstamp(args.timing, it, 5);
    // ---- 3. wait until the row's 2 * parts words all carry this epoch (bounded), then merge.
    // The partials of the 32 rows of this slab come from the same 2*C warps, so one lane probes its
    // own row (2 * parts loads per probe, not 64 * parts: letting every lane poll its row was measured
    // and cost 15 % of the kernel, a pause between probes changed nothing) and only then does every
    // lane read and validate its row; a lane whose words are not all there yet sends the warp round
    // again.
    float mean = 0.f, rstd = 0.f;
    float pm[8], pq[8];  // N <= 1024: at most 8 partials per row
    const unsigned long long* rp64 = words + static_cast<size_t>(row_ok ? row : 0) * parts * 2;
    const long long t0 = clock64();
    bool give_up = false;
    while (true) {
      if (lane == 0 && row_ok) {
        uint32_t probes = 0;
        while (true) {
          // all loads are issued before any tag is looked at (no short-circuit: one round trip, not 2*parts)
          uint32_t bad = 0;
#pragma unroll
          for (int p = 0; p < 8; ++p)
            if (p < parts) {
              const unsigned long long w0 = ld_relaxed_gpu_u64(rp64 + 2 * p);
              const unsigned long long w1 = ld_relaxed_gpu_u64(rp64 + 2 * p + 1);
              bad |= (static_cast<uint32_t>(w0) ^ epoch) | (static_cast<uint32_t>(w1) ^ epoch);
            }
          if (bad == 0) break;
          if ((++probes & 15u) == 0u && (*abort_flag != 0 || clock64() - t0 > (1ll << 31))) break;
        }
      }
      __syncwarp();
      uint32_t bad = 0;
      if (row_ok) {
#pragma unroll
        for (int p = 0; p < 8; ++p)
          if (p < parts) {
            const unsigned long long w0 = ld_relaxed_gpu_u64(rp64 + 2 * p);
            const unsigned long long w1 = ld_relaxed_gpu_u64(rp64 + 2 * p + 1);
            bad |= (static_cast<uint32_t>(w0) ^ epoch) | (static_cast<uint32_t>(w1) ^ epoch);
            pm[p] = __uint_as_float(static_cast<uint32_t>(w0 >> 32));
            pq[p] = __uint_as_float(static_cast<uint32_t>(w1 >> 32));
          }
      }
      if (__all_sync(0xffffffffu, bad == 0)) break;
      if (*abort_flag != 0 || clock64() - t0 > (1ll << 31)) {
        give_up = true;
        break;
      }
      __nanosleep(100);
    }
    if (__any_sync(0xffffffffu, give_up)) {
      if (lane == 0) {
        *abort_flag = 1;
        if (args.status != nullptr) atomicCAS(args.status, 0, kStatusGemmEpilogueTimeout);
      }
      break;
    }
    if (row_ok) {
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if (p < parts) mean += pm[p];
      mean *= 1.0f / static_cast<float>(parts);
      float M2 = 0.f;
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if (p < parts) {
          const float d = pm[p] - mean;
          M2 += pq[p] + static_cast<float>(kColsPerThread) * d * d;
        }
      rstd = rsqrtf(M2 * inv_n + args.eps);
    }
    if (warp == 2 && lane == 0) gstamp(args.timing, it, 6);
    const float shift = -mean * rstd;
    const unsigned long long rstd2 = pack_f32x2(rstd, rstd), shift2 = pack_f32x2(shift, shift);
    tmem_st_wait();  // the write-back of step 1 is complete before tensor memory is read again
    // ---- 4. normalise, gamma / beta, fp16, store (64 columns = 128 B per row at a time)
    const bool slab_full = row0 + 32 <= M;
    {
      uint32_t raw[2][32];
      tmem_ld_32x32(t_row, raw[0]);
#pragma unroll
      for (int ci = 0; ci < kColsPerThread / 32; ++ci) {
        const int c = ci * 32;
        const int hh = ci & 1;  // which half of the current 64-column store chunk
        uint8_t* srow = stg + lane * 128;
        if (hh == 0 && slab_full) {
          if (lane == 0) tma_store_wait_read_n<0>();  // the previous bulk store has read the staging rows
          __syncwarp();
        }
        tmem_ld_wait();
        if (ci + 1 < kColsPerThread / 32) tmem_ld_32x32(t_row + c + 32, raw[(ci + 1) & 1]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int col8 = gcol0 + c + q * 8;  // first of these 8 columns
          float g[8], b[8];
          if (args.gb_fp32) {
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(args.gamma) + (col8 >> 2));
            const float4 g1 = __ldg(reinterpret_cast<const float4*>(args.gamma) + (col8 >> 2) + 1);
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(args.beta) + (col8 >> 2));
            const float4 b1 = __ldg(reinterpret_cast<const float4*>(args.beta) + (col8 >> 2) + 1);
            g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
            b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
          } else {
            const uint4 g4 = sgamma[c / 8 + q];
            const uint4 b4 = sbeta[c / 8 + q];
            const __half2* gh = reinterpret_cast<const __half2*>(&g4);
            const __half2* bh = reinterpret_cast<const __half2*>(&b4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 fg = __half22float2(gh[j]);
              const float2 fb = __half22float2(bh[j]);
              g[2 * j] = fg.x; g[2 * j + 1] = fg.y;
              b[2 * j] = fb.x; b[2 * j + 1] = fb.y;
            }
          }
          float y[8];
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            const unsigned long long n2 = fma_f32x2(
                pack_f32x2(__uint_as_float(raw[ci & 1][q * 8 + i]), __uint_as_float(raw[ci & 1][q * 8 + i + 1])), rstd2, shift2);
            unpack_f32x2(fma_f32x2(n2, pack_f32x2(g[i], g[i + 1]), pack_f32x2(b[i], b[i + 1])), y[i], y[i + 1]);
          }
          uint4 u;
          u.x = pack_half2(y[0], y[1]);
          u.y = pack_half2(y[2], y[3]);
          u.z = pack_half2(y[4], y[5]);
          u.w = pack_half2(y[6], y[7]);
          const int unit = hh * 4 + q;  // 16-byte unit inside the 128-byte row
          if (slab_full)
            *reinterpret_cast<uint4*>(srow + ((unit ^ (lane & 7)) << 4)) = u;
          else if (row_ok)
            *reinterpret_cast<uint4*>(args.out_ln + static_cast<size_t>(row) * args.N + col8) = u;
        }
        if (hh == 1 && slab_full) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(tm_out, stg, gcol0 + c - 32, row0);
            tma_store_commit();
          }
        }
      }
    }
    if (warp == 2 && lane == 0) gstamp(args.timing, it, 3);
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      release_acc(as);
      mbar_arrive(vec_empty);
    }
  }
  if (lane == 0) tma_store_wait_all();
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_f16_ln_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_res,
                   const GemmArgs args) {
  constexpr int kTileN = 256;
  using Cfg = GemmCfg<kTileN>;
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kStagingBytes);
  uint64_t* full_bar = bars;                    // [kStages]
  uint64_t* empty_bar = bars + kStages;         // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;      // [2]
  uint64_t* acc_empty = bars + 2 * kStages + 2; // [2]
  uint64_t* vec_full = bars + 2 * kStages + 4;   // bias / gamma / beta of the tile's columns are in shared memory
  uint64_t* vec_empty = bars + 2 * kStages + 5;  // all epilogue warps are done with them
  uint64_t* res_bar = bars + 2 * kStages + 6;    // [kEpiWarps] a warp's residual rows have landed in its staging buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 6 + kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // fp16 vectors of the current tile's 256 columns: bias | gamma | beta (gamma / beta only when they are fp16)
  uint4* vec_s = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], kEpiWarps);
    }
    mbar_init(vec_full, 1);
    mbar_init(vec_empty, kEpiWarps);
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(&res_bar[w], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_out);
    tma_prefetch_desc(&tm_res);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();  // see gemm_f16_kernel
  int M = args.m_rows;
  if (args.m_dev != nullptr) {
    const int md = __ldg(args.m_dev);
    M = md < M ? md : M;
  }
  const int n_tiles = args.N / kTileN;
  const int m_tiles = (M + kBlockM - 1) / kBlockM;
  const int total_tiles = m_tiles * n_tiles;
  const int num_kb = args.K / kBlockK;
  auto tile_at = [&](int li, int& m0, int& n0) -> bool {
    const int tile = static_cast<int>(blockIdx.x) + li * static_cast<int>(gridDim.x);
    if (tile >= total_tiles) return false;
    m0 = (tile / n_tiles) * kBlockM;
    n0 = (tile % n_tiles) * kTileN;
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int m0 = 0, n0 = 0;
      for (int li = 0; ok && tile_at(li, m0, n0); ++li) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, args.status,
                                 kStatusGemmProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d(sa, &tm_a, &full_bar[stage], kb * kBlockK, m0);
#pragma unroll
          for (int c = 0; c < kTileN / 64; ++c)
            tma_load_2d(sb + c * (64 * kBlockK * 2), &tm_b, &full_bar[stage], n0 + c * 64, kb * kBlockK);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int m0 = 0, n0 = 0;
      for (int it = 0; ok && tile_at(it, m0, n0); ++it) {
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aphase ^ 1u, abort_flag, args.status, kStatusGemmMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        gstamp(args.timing, it, 0);
        const uint32_t d_tmem = tmem_base + as * kTileN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, args.status, kStatusGemmMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint64_t adesc = smem_desc(args.a_desc_hi, sa + k * args.a_kstep_bytes);
            const uint64_t bdesc = smem_desc(args.b_desc_hi, sb + k * args.b_kstep_bytes);
            umma_f16_ss(d_tmem, adesc, bdesc, args.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
        gstamp(args.timing, it, 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    ln_epilogue_loop(args, &tm_out, &tm_res, smem + kStages * Cfg::kStageBytes, acc_full, vec_full, vec_empty, res_bar,
                     vec_s, abort_flag, tmem_base, M, n_tiles, warp, lane, tile_at,
                     [&](int as) { mbar_arrive(&acc_empty[as]); });
  }

  // ------------------------------------------------------------------ teardown
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
// GEMM + bias + residual + LayerNorm on SM pairs: the main loop of gemm_f16_pair_kernel (256 x 256
// tiles, cta_group::2, half of the W tile per SM) with the epilogue of gemm_f16_ln_kernel.  Each CTA
// of a pair holds the accumulator of its own 128 rows, so its epilogue warps do exactly what those of
// the one-CTA kernel do; the partials of a row come from the N/256 clusters working on that row tile.
// Tiles go round-robin over the clusters (all resident: the launch asks for no more clusters than fit),
// and a cluster only waits for clusters working on earlier or the same row tiles: no circular wait.
// ------------------------------------------------------------------------------------------
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_f16_pair_ln_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                        const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_res,
                        const GemmArgs args) {
  using Cfg = PairCfg;
  constexpr int kStages = Cfg::kStages;
  constexpr int kTileN = Cfg::kTileN;

  extern __shared__ uint8_t smem_raw[];
  // Both CTAs of the pair must use identical shared-memory offsets (the MMA and the multicast
  // commit address the peer by offset); dynamic shared memory starts at the same offset in
  // every CTA of a launch, so the same round-up applies to both.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kStagingBytes);
  uint64_t* full_bar = bars;                    // [kStages]  (leader's copy is the live one)
  uint64_t* empty_bar = bars + kStages;         // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;      // [2]
  uint64_t* acc_empty = bars + 2 * kStages + 2; // [2]        (leader's copy is the live one)
  uint64_t* vec_full = bars + 2 * kStages + 4;   // as in gemm_f16_ln_kernel
  uint64_t* vec_empty = bars + 2 * kStages + 5;
  uint64_t* res_bar = bars + 2 * kStages + 6;    // [kEpiWarps]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 6 + kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint4* vec_s = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
  const bool leader = cta_rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 2 * kEpiWarps);
    }
    mbar_init(vec_full, 1);
    mbar_init(vec_empty, kEpiWarps);
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(&res_bar[w], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();  // see gemm_f16_kernel
  int M = args.m_rows;
  if (args.m_dev != nullptr) {
    const int md = __ldg(args.m_dev);
    M = md < M ? md : M;
  }
  const int n_tiles = args.N / kTileN;
  const int m_tiles = (M + 2 * kBlockM - 1) / (2 * kBlockM);
  const int total_tiles = m_tiles * n_tiles;
  const int num_kb = args.K / kBlockK;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_a);
      tma_prefetch_desc(&tm_b);
      tma_prefetch_desc(&tm_out);
      tma_prefetch_desc(&tm_res);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters) {
        const int m0 = (tile / n_tiles) * (2 * kBlockM) + static_cast<int>(cta_rank) * kBlockM;
        const int n0 = (tile % n_tiles) * kTileN + static_cast<int>(cta_rank) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, args.status,
                                 kStatusGemmProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + kABytes;
          // the leader announces the bytes of both CTAs; all copies complete on its barrier
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &tm_a, bar, kb * kBlockK, m0);
          tma_load_2d_pair(sb, &tm_b, bar, n0, kb * kBlockK);
          tma_load_2d_pair(sb + 64 * kBlockK * 2, &tm_b, bar, n0 + 64, kb * kBlockK);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters, ++it) {
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aphase ^ 1u, abort_flag, args.status, kStatusGemmMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        gstamp(args.timing, it, 0);
        const uint32_t d_tmem = tmem_base + as * kTileN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, args.status, kStatusGemmMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint64_t adesc = smem_desc(args.a_desc_hi, sa + k * args.a_kstep_bytes);
            const uint64_t bdesc = smem_desc(args.b_desc_hi, sb + k * args.b_kstep_bytes);
            umma_f16_ss_pair(d_tmem, adesc, bdesc, args.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);  // frees the stage in both CTAs
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit_pair(&acc_full[as]);
        gstamp(args.timing, it, 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    auto tile_at = [&](int it, int& m0, int& n0) -> bool {
      const int tile = cluster_id + it * num_clusters;
      if (tile >= total_tiles) return false;
      m0 = (tile / n_tiles) * (2 * kBlockM) + static_cast<int>(cta_rank) * kBlockM;
      n0 = (tile % n_tiles) * kTileN;
      return true;
    };
    ln_epilogue_loop(args, &tm_out, &tm_res, smem + kStages * Cfg::kStageBytes, acc_full, vec_full, vec_empty, res_bar,
                     vec_s, abort_flag, tmem_base, M, n_tiles, warp, lane, tile_at,
                     [&](int as) { mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[as]), 0)); });
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
  }
}


// ------------------------------------------------------------------------------------------ launch
template <int BLOCK_N, int EPI>
cudaError_t launch_one(const GemmLaunch& g, const GemmArgs& a, cudaStream_t stream) {
  using Cfg = GemmCfg<BLOCK_N>;
  static bool attr_set[64] = {};  // per template instance and device
  auto kern = gemm_f16_kernel<BLOCK_N, EPI>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const int n_tiles = g.N / BLOCK_N;
  const int m_tiles = (g.m_rows + kBlockM - 1) / kBlockM;
  long long tiles = static_cast<long long>(n_tiles) * m_tiles * (EPI == kEpiSplitKF32 ? a.split_k : 1);
  int grid = static_cast<int>(tiles < g.num_sms ? tiles : g.num_sms);
  if (grid < 1) grid = 1;
  return launch_pdl(kern, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, stream, g.tm_a, g.tm_b, g.tm_out, a);
}

template <int BLOCK_N>
cudaError_t launch_epi(const GemmLaunch& g, const GemmArgs& a, cudaStream_t stream) {
  switch (g.epilogue) {
    case BT_EPI_NONE: return launch_one<BLOCK_N, BT_EPI_NONE>(g, a, stream);
    case BT_EPI_BIAS: return launch_one<BLOCK_N, BT_EPI_BIAS>(g, a, stream);
    case BT_EPI_BIAS_GELU: return launch_one<BLOCK_N, BT_EPI_BIAS_GELU>(g, a, stream);
    case BT_EPI_BIAS_RESIDUAL: return launch_one<BLOCK_N, BT_EPI_BIAS_RESIDUAL>(g, a, stream);
    case BT_EPI_BIAS_RESIDUAL_F32OUT: return launch_one<BLOCK_N, BT_EPI_BIAS_RESIDUAL_F32OUT>(g, a, stream);
    default: return cudaErrorInvalidValue;
  }
}

// Clusters of two that can be co-resident on a device (one CTA per SM); 0 = not yet asked.
int g_pair_clusters[64] = {};

template <int EPI>
cudaError_t launch_pair(const GemmLaunch& g, const GemmArgs& a, cudaStream_t stream) {
  using Cfg = PairCfg;
  static bool attr_set[64] = {};
  auto kern = gemm_f16_pair_kernel<EPI>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  if (g_pair_clusters[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (g.num_sms / 2));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = g.num_sms / 2;
    }
    g_pair_clusters[dev] = n;
  }
  const int n_tiles = g.N / Cfg::kTileN;
  const int m_tiles = (g.m_rows + 2 * kBlockM - 1) / (2 * kBlockM);
  long long tiles = static_cast<long long>(n_tiles) * m_tiles;
  int clusters = static_cast<int>(tiles < g_pair_clusters[dev] ? tiles : g_pair_clusters[dev]);
  if (clusters < 1) clusters = 1;
  return launch_pdl(kern, dim3(2 * clusters), dim3(kGemmThreads), Cfg::kSmemBytes, stream, g.tm_a, g.tm_b, g.tm_out, a);
}

cudaError_t launch_pair_epi(const GemmLaunch& g, const GemmArgs& a, cudaStream_t stream) {
  switch (g.epilogue) {
    case BT_EPI_NONE: return launch_pair<BT_EPI_NONE>(g, a, stream);
    case BT_EPI_BIAS: return launch_pair<BT_EPI_BIAS>(g, a, stream);
    case BT_EPI_BIAS_GELU: return launch_pair<BT_EPI_BIAS_GELU>(g, a, stream);
    case BT_EPI_BIAS_RESIDUAL: return launch_pair<BT_EPI_BIAS_RESIDUAL>(g, a, stream);
    case BT_EPI_BIAS_RESIDUAL_F32OUT: return launch_pair<BT_EPI_BIAS_RESIDUAL_F32OUT>(g, a, stream);
    default: return cudaErrorInvalidValue;
  }
}

struct LnGemmCfg {
  static constexpr int kSmemBytes = GemmCfg<256>::kSmemBytes + 1536;  // + bias / gamma / beta slices of a tile
};
static_assert(LnGemmCfg::kSmemBytes <= 227 * 1024, "shared memory of the GEMM + LayerNorm kernel");

struct PairLnGemmCfg {
  static constexpr int kSmemBytes = PairCfg::kSmemBytes + 1536;
};
static_assert(PairLnGemmCfg::kSmemBytes <= 227 * 1024, "shared memory of the pair GEMM + LayerNorm kernel");
int g_pair_ln_clusters[64] = {};

// The pair form of the GEMM + LayerNorm kernel.  `a.idesc` must describe M = 256.
cudaError_t launch_pair_ln_gemm(const GemmLaunch& g, const GemmArgs& a, cudaStream_t stream) {
  using Cfg = PairLnGemmCfg;
  static bool attr_set[64] = {};
  auto kern = gemm_f16_pair_ln_kernel;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  if (g_pair_ln_clusters[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (g.num_sms / 2));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    int n = 0;
    // every cluster must be resident (clusters wait for one another's row statistics): without an
    // answer from the occupancy query the pair form is not used
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = -1;
    }
    g_pair_ln_clusters[dev] = n;
  }
  if (g_pair_ln_clusters[dev] <= 0) return cudaErrorNotSupported;
  const int n_tiles = g.N / 256;
  const int m_tiles = (g.m_rows + 2 * kBlockM - 1) / (2 * kBlockM);
  long long tiles = static_cast<long long>(n_tiles) * m_tiles;
  int clusters = static_cast<int>(tiles < g_pair_ln_clusters[dev] ? tiles : g_pair_ln_clusters[dev]);
  if (clusters < 1) clusters = 1;
  return launch_pdl(kern, dim3(2 * clusters), dim3(kGemmThreads), Cfg::kSmemBytes, stream, g.tm_a, g.tm_b, g.tm_out,
                    g.tm_res, a);
}

cudaError_t launch_ln_gemm(const GemmLaunch& g, const GemmArgs& a_in, cudaStream_t stream) {
  using Cfg = LnGemmCfg;
  static bool attr_set[64] = {};
  auto kern = gemm_f16_ln_kernel;
  if (g.N % 256 != 0 || g.N > 1024 || !g.out_ln || !g.gamma || !g.beta || !g.residual || !g.bias || g.ln_epoch == 0)
    return cudaErrorInvalidValue;
  // The pair form (main loop on SM pairs, half of the W tile per SM) is used where the main loop is the longer
  // leg of a tile, i.e. for a long K (FFN2, K = 4 x hidden): measured in situ on 69.6k-row launches, 79.5 against
  // 85 ms of FFN2 kernel time per three steps and +1.3 % on the whole forward.  For a short K (attention output)
  // the epilogue is the longer leg, and a buffer of the pair's accumulator is only released when the epilogue
  // warps of BOTH CTAs are done with it: 11 % slower there.  (On 18.9k-row launches, 1800 per step, the gain
  // on FFN2 was 5 % of its kernel time and the forward did not move.)  Debug key 9: 1 = always, 2 = never.
  const bool want_pair = g_dbg_ln_pair == 1 || (g_dbg_ln_pair == 0 && g.K >= 2048);
  if (want_pair) {
    GemmArgs ap = a_in;
    ap.idesc = make_idesc_f16(256, 256, 0, 1);
    const cudaError_t e = launch_pair_ln_gemm(g, ap, stream);
    if (e != cudaErrorNotSupported) return e;
  }
  const GemmArgs& a = a_in;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const int m_tiles = (g.m_rows + kBlockM - 1) / kBlockM;
  const long long tiles = static_cast<long long>(m_tiles) * (g.N / 256);
  int grid = static_cast<int>(tiles < g.num_sms ? tiles : g.num_sms);
  if (grid < 1) grid = 1;
  return launch_pdl(kern, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, stream, g.tm_a, g.tm_b, g.tm_out, g.tm_res, a);
}

// The pair kernel needs N % 256 == 0 and pays off once every SM pair gets at least two
// 256 x 256 tiles (below that the narrower one-CTA tiles fill the machine better).
bool use_pair_kernel(const GemmLaunch& g) {
  if (g.epilogue == BT_EPI_BIAS_RESIDUAL_LAYERNORM) return false;
  if (g_dbg_pair_mode == 1) return g.N % 256 == 0;
  if (g_dbg_pair_mode == 2 || g_dbg_force_block_n != 0 || g.block_n != 0) return false;
  if (g.N % 256 != 0) return false;
  // Measured at 18.9k rows: with a short main loop (K = 768) the fp32 + residual epilogue bounds
  // the tile time and the one-CTA kernel is a few percent faster.  (The GELU epilogue used to be
  // on that list; with the present epilogue the pair kernel gains 1.6 % on the whole forward.)
  if ((g.epilogue == BT_EPI_BIAS_RESIDUAL || g.epilogue == BT_EPI_BIAS_RESIDUAL_F32OUT) && g.K < 2048) return false;
  const long long tiles = static_cast<long long>((g.m_rows + 255) / 256) * (g.N / 256);
  return tiles >= 2LL * (g.num_sms / 2);
}

}  // namespace

// Few rows and a long K leave most SMs idle while a handful stream the weights one K block
// after the other; cutting K spreads that stream.  The widest cut whose (tile, range) pairs number at
// most one and a half times the SMs (the row count is an upper bound: padded rows make no tiles), with
// at least three K blocks per range.
int gemm_pick_split_k(int m_rows, int N, int K, int num_sms) {
  if (N % 64 != 0 || K % kBlockK != 0) return 1;
  if (g_dbg_split_k != 0)
    return (g_dbg_split_k > 0 && (K / kBlockK) % g_dbg_split_k == 0) ? static_cast<int>(g_dbg_split_k) : 1;
  const long long tiles = static_cast<long long>((m_rows + kBlockM - 1) / kBlockM) * (N / 64);
  const int num_kb = K / kBlockK;
  const int cands[3] = {8, 4, 2};
  for (int i = 0; i < 3; ++i) {
    const int s = cands[i];
    if (num_kb % s != 0 || num_kb / s < 3) continue;
    if (tiles * s <= num_sms + num_sms / 2) return s;
  }
  return 1;
}

int gemm_pick_block_n(int m_rows, int N, int num_sms) {
  if (g_dbg_force_block_n != 0) return static_cast<int>(g_dbg_force_block_n);
  const int m_tiles = (m_rows + kBlockM - 1) / kBlockM;
  // Prefer the widest tile that still gives every SM at least one tile.
  const int cands[3] = {256, 128, 64};
  for (int i = 0; i < 3; ++i) {
    const int bn = cands[i];
    if (N % bn != 0) continue;
    if (static_cast<long long>(m_tiles) * (N / bn) >= num_sms) return bn;
  }
  for (int i = 2; i >= 0; --i)
    if (N % cands[i] == 0) return cands[i];
  return 0;
}

cudaError_t launch_gemm(const GemmLaunch& g, cudaStream_t stream) {
  if (g.K % kBlockK != 0 || g.m_rows <= 0) return cudaErrorInvalidValue;
  GemmArgs a;
  a.out = g.out;
  a.bias = g.bias;
  a.residual = g.residual;
  a.m_dev = g.m_dev;
  a.m_rows = g.m_rows;
  a.N = g.N;
  a.K = g.K;
  a.gelu_kind = g.gelu_kind;
  a.status = g.status;
  a.out_ln = g.out_ln;
  a.gamma = g.gamma;
  a.beta = g.beta;
  a.gb_fp32 = g.gb_fp32 ? 1 : 0;
  a.eps = g.eps;
  a.ln_epoch = g.ln_epoch;
  a.timing = g_dbg_gemm_timing;
  // A: K-major, 128B swizzle, 8-row groups 1024 B apart; 16 K-elements = 32 B.
  a.a_desc_hi = make_smem_desc_hi(16, 1024);
  a.a_kstep_bytes = 32;
  // W: MN-major, 128B swizzle; 64-column chunks 8 KiB apart (LBO), 8-k groups
  // 1024 B apart (SBO); 16 K-rows = 2048 B.
  const uint32_t lbo = g_dbg_b_lbo ? static_cast<uint32_t>(g_dbg_b_lbo) : 64u * kBlockK * 2u;
  const uint32_t sbo = g_dbg_b_sbo ? static_cast<uint32_t>(g_dbg_b_sbo) : 1024u;
  a.b_desc_hi = make_smem_desc_hi(lbo, sbo);
  a.b_kstep_bytes = g_dbg_b_kstep ? static_cast<uint32_t>(g_dbg_b_kstep) : 2048u;
  a.split_k = 1;
  a.split_stride = 0;
  a.early_w = g_dbg_early_w != 0 ? 1 : 0;
  if (g.split_k > 1) {
    if (g.epilogue != BT_EPI_BIAS_RESIDUAL_F32OUT || g.N % 64 != 0 || (g.K / kBlockK) % g.split_k != 0)
      return cudaErrorInvalidValue;
    a.split_k = g.split_k;
    a.split_stride = static_cast<long long>(g.m_rows) * g.N;
    a.idesc = make_idesc_f16(kBlockM, 64, 0, 1);
    return launch_one<64, kEpiSplitKF32>(g, a, stream);
  }
  if (use_pair_kernel(g)) {
    a.idesc = make_idesc_f16(256, 256, 0, 1);  // M = 256 across the pair
    return launch_pair_epi(g, a, stream);
  }
  if (g.epilogue == BT_EPI_BIAS_RESIDUAL_LAYERNORM) {
    a.idesc = make_idesc_f16(kBlockM, 256, 0, 1);
    return launch_ln_gemm(g, a, stream);
  }
  int bn = g.block_n != 0 ? g.block_n : gemm_pick_block_n(g.m_rows, g.N, g.num_sms);
  if (bn == 0 || g.N % bn != 0) return cudaErrorInvalidValue;
  a.idesc = make_idesc_f16(kBlockM, bn, 0, 1);
  switch (bn) {
    case 256: return launch_epi<256>(g, a, stream);
    case 128: return launch_epi<128>(g, a, stream);
    case 64: return launch_epi<64>(g, a, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace bt

// Diagnostics hook (not part of the stable ABI): overrides descriptor fields of
// the W operand / the tile width so that encodings can be compared on a device
// without rebuilding.  key: 1 = LBO bytes, 2 = SBO bytes, 3 = K-step bytes,
// 4 = forced BLOCK_N of the one-CTA kernel, 5 = pair kernel (0 auto, 1 always when
// N % 256 == 0, 2 never), 6 = programmatic dependent launch on (1, default) / off (0),
// 7 = split-K of the fp32-sum GEMMs (0 policy, < 0 never, > 0 that many K ranges),
// 8 = W blocks of a CTA's first tile requested before the dependency wait (1, default) or after (0),
// 9 = GEMM + LayerNorm on SM pairs (0, the default: for K >= 2048; 1 always; 2 never).
// value 0 restores the default for keys 1-5 and 7.
// Device buffer of 148 x 16 x 8 long long for clock64 stamps of the GEMM kernels (null = off):
// slots 0/1 MMA warp (accumulator free, last commit), 2/3 epilogue warp 2 (accumulator ready, tile
// done), 4..6 LayerNorm kernel only (sums written back, partial published, partials of all peers seen).
extern "C" int bt_debug_set_gemm_timing(long long* device_buffer) {
  bt::g_dbg_gemm_timing = device_buffer;
  return 0;
}
// Host-side shape policies, callable without a device (tests): what 0 = tile width of the one-CTA
// kernel, 1 = K ranges of an fp32-sum GEMM, 2 = 1 if the pair kernel would take a bias-only GEMM.
extern "C" int bt_debug_policy(int what, int m_rows, int N, int K, int num_sms) {
  switch (what) {
    case 0: return bt::gemm_pick_block_n(m_rows, N, num_sms);
    case 1: return bt::gemm_pick_split_k(m_rows, N, K, num_sms);
    case 2: {
      bt::GemmLaunch g = {};
      g.m_rows = m_rows;
      g.N = N;
      g.K = K;
      g.epilogue = BT_EPI_BIAS;
      g.block_n = 0;
      g.num_sms = num_sms;
      return bt::use_pair_kernel(g) ? 1 : 0;
    }
    default: return -1;
  }
}
extern "C" int bt_debug_set(int key, long long value) {
  switch (key) {
    case 1: bt::g_dbg_b_lbo = value; return 0;
    case 2: bt::g_dbg_b_sbo = value; return 0;
    case 3: bt::g_dbg_b_kstep = value; return 0;
    case 4: bt::g_dbg_force_block_n = value; return 0;
    case 7: bt::g_dbg_split_k = value; return 0;
    case 8: bt::g_dbg_early_w = value; return 0;
    case 9: bt::g_dbg_ln_pair = value; return 0;
    case 5: bt::g_dbg_pair_mode = value; return 0;
    case 6: bt::set_pdl_enabled(value != 0); return 0;
    default: return 1;
  }
}
