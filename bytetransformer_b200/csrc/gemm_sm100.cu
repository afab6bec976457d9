// Dense fp16 GEMM for sm_100a:  out[M,N] = epilogue(A[M,K] * W[K,N]),  fp32 accumulation.
//
// Replaces the reference's cuBLAS / CUTLASS-2.x calls on the encoder path
// (bytetransformer/src/gemm.cu:32-39, bytetransformer/src/gemm_bias_act.cu:76-148).
//
// Design (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer: A tile [128 x 64] (K-major) and W tile [64 x BLOCK_N]
//               (N contiguous = MN-major for UMMA, so the reference's [in,out]
//               weight layout is consumed as is, no transposed copy) into a
//               128B-swizzled shared-memory ring.
//   warp 1      allocates tensor memory and issues tcgen05.mma (128 x BLOCK_N x 16,
//               kind::f16) from one elected lane; accumulators are double buffered
//               in tensor memory (2 x BLOCK_N columns) so the epilogue of tile i
//               overlaps the main loop of tile i+1.
//   warps 2..9  epilogue: tcgen05.ld -> +bias -> GELU / +residual -> fp16 (or fp32)
//               -> 128B-swizzled staging rows in shared memory -> TMA bulk store
//               (full 128-byte lines); a 32-row slab that crosses M falls back to
//               row-predicated 16-byte stores, so rows >= M are never written.
// M is read from device memory (the packed token count is only known on the
// device), so the host never blocks; the grid is sized from the allocated rows.
// Every mbarrier wait is bounded: on expiry the CTA records a code in the status
// word and all roles drain to a common exit that frees tensor memory.
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
  uint64_t a_desc_hi;
  uint64_t b_desc_hi;
  uint32_t a_kstep_bytes;
  uint32_t b_kstep_bytes;
  uint32_t idesc;
};

// Debug overrides of the shared-memory descriptor fields (0 = use the default).
long long g_dbg_b_lbo = 0, g_dbg_b_sbo = 0, g_dbg_b_kstep = 0, g_dbg_force_block_n = 0;

template <int BLOCK_N, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_out, const GemmArgs args) {
  using Cfg = GemmCfg<BLOCK_N>;
  constexpr int kStages = Cfg::kStages;

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

  int M = args.m_rows;
  if (args.m_dev != nullptr) {
    const int md = __ldg(args.m_dev);
    M = md < M ? md : M;
  }
  const int n_tiles = args.N / BLOCK_N;
  const int m_tiles = (M + kBlockM - 1) / kBlockM;
  const int total_tiles = m_tiles * n_tiles;
  const int num_kb = args.K / kBlockK;

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
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_a);
      tma_prefetch_desc(&tm_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / n_tiles) * kBlockM;
        const int n0 = (tile % n_tiles) * BLOCK_N;
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
          for (int c = 0; c < BLOCK_N / 64; ++c)
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
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aphase ^ 1u, abort_flag, args.status, kStatusGemmMmaTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
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
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int e = warp - 2;
    const int quarter = warp & 3;            // TMEM lane quarter this warp may read
    const int col_half = e >> 2;             // which half of the tile's columns
    constexpr int kColsPerWarp = BLOCK_N / 2;
    constexpr bool kF32Out = (EPI == BT_EPI_BIAS_RESIDUAL_F32OUT);
    constexpr bool kHasResidual = (EPI == BT_EPI_BIAS_RESIDUAL || EPI == BT_EPI_BIAS_RESIDUAL_F32OUT);
    // 128 bytes of output per row and chunk: 32 fp32 or 64 fp16 columns.
    constexpr int kChunk = kF32Out ? 32 : (kColsPerWarp >= 64 ? 64 : 32);
    constexpr bool kTmaStore = Cfg::kTmaStore;
    uint8_t* stg = smem + kStages * Cfg::kStageBytes + e * kStagingBytesPerWarp;  // 32 rows x 128 B, swizzled
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const int m0 = (tile / n_tiles) * kBlockM;
      const int n0 = (tile % n_tiles) * BLOCK_N;
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      const int row0 = m0 + quarter * 32;
      const int row = row0 + lane;
      const bool row_ok = row < M;
      // The residual slice of this thread's row is fetched before waiting for the
      // accumulator, so its latency hides behind the main loop of the tile.
      uint4 resv[kHasResidual ? kColsPerWarp / 8 : 1];
      if (kHasResidual) {
        const uint4* rp = reinterpret_cast<const uint4*>(args.residual + static_cast<size_t>(row) * args.N + n0 +
                                                         col_half * kColsPerWarp);
#pragma unroll
        for (int q = 0; q < kColsPerWarp / 8; ++q) resv[q] = row_ok ? __ldg(rp + q) : make_uint4(0u, 0u, 0u, 0u);
      }
      if (!mbar_wait_bounded(&acc_full[as], aphase, abort_flag, args.status, kStatusGemmEpilogueTimeout)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool slab_full = kTmaStore && (row0 + 32 <= M);  // all 32 rows valid: bulk store, else predicated stores
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * BLOCK_N;
#pragma unroll
      for (int c = 0; c < kColsPerWarp; c += kChunk) {
        const int col = col_half * kColsPerWarp + c;  // column inside the tile
        const int gcol = n0 + col;
        float v[kChunk];
        {
          uint32_t r[32];
          tmem_ld_32x32(t_row + col, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (kChunk == 64) {
            tmem_ld_32x32(t_row + col + 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[(kChunk == 64 ? 32 : 0) + i] = __uint_as_float(r[i]);
          }
        }
        if (EPI != BT_EPI_NONE) {
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
            for (int i = 0; i < kChunk; ++i) v[i] = gelu_erf_fast(v[i]);
          }
        }
        const size_t off = static_cast<size_t>(row) * args.N + gcol;
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
        // 8 units of 16 bytes per row
        uint4 units[8];
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
        constexpr int kUnits = kF32Out ? 8 : kChunk / 8;
        if (slab_full) {
          // the previous bulk store of this warp must have finished reading the staging rows
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
          uint8_t* srow = stg + lane * 128;
#pragma unroll
          for (int q = 0; q < kUnits; ++q) *reinterpret_cast<uint4*>(srow + ((q ^ (lane & 7)) << 4)) = units[q];
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tm_out, stg, gcol, row0);
            tma_store_commit();
          }
        } else if (row_ok) {
          uint4* op = kF32Out ? reinterpret_cast<uint4*>(reinterpret_cast<float*>(args.out) + off)
                              : reinterpret_cast<uint4*>(args.out + off);
#pragma unroll
          for (int q = 0; q < kUnits; ++q) op[q] = units[q];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
    }
    if (kTmaStore && lane == 0) tma_store_wait_all();  // staging rows must outlive the last bulk store
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
  long long tiles = static_cast<long long>(n_tiles) * m_tiles;
  int grid = static_cast<int>(tiles < g.num_sms ? tiles : g.num_sms);
  if (grid < 1) grid = 1;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(g.tm_a, g.tm_b, g.tm_out, a);
  return cudaGetLastError();
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

}  // namespace

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
  int bn = g.block_n != 0 ? g.block_n : gemm_pick_block_n(g.m_rows, g.N, g.num_sms);
  if (bn == 0 || g.N % bn != 0 || g.K % kBlockK != 0 || g.m_rows <= 0) return cudaErrorInvalidValue;
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
  // A: K-major, 128B swizzle, 8-row groups 1024 B apart; 16 K-elements = 32 B.
  a.a_desc_hi = make_smem_desc_hi(16, 1024);
  a.a_kstep_bytes = 32;
  // W: MN-major, 128B swizzle; 64-column chunks 8 KiB apart (LBO), 8-k groups
  // 1024 B apart (SBO); 16 K-rows = 2048 B.
  const uint32_t lbo = g_dbg_b_lbo ? static_cast<uint32_t>(g_dbg_b_lbo) : 64u * kBlockK * 2u;
  const uint32_t sbo = g_dbg_b_sbo ? static_cast<uint32_t>(g_dbg_b_sbo) : 1024u;
  a.b_desc_hi = make_smem_desc_hi(lbo, sbo);
  a.b_kstep_bytes = g_dbg_b_kstep ? static_cast<uint32_t>(g_dbg_b_kstep) : 2048u;
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
// 4 = forced BLOCK_N.  value 0 restores the default.
extern "C" int bt_debug_set(int key, long long value) {
  switch (key) {
    case 1: bt::g_dbg_b_lbo = value; return 0;
    case 2: bt::g_dbg_b_sbo = value; return 0;
    case 3: bt::g_dbg_b_kstep = value; return 0;
    case 4: bt::g_dbg_force_block_n = value; return 0;
    default: return 1;
  }
}
