// Device-side building blocks shared by the sm_100a kernels: mbarrier, TMA,
// tcgen05 (UMMA + tensor memory) wrappers, shared-memory matrix descriptors and
// bounded waits.  Everything here is inline PTX; there is no CUTLASS dependency.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bt {

// ---------------------------------------------------------------------------
// Device status word codes (written by kernels, read by bt_device_status()).
// A non-zero code means a bounded wait gave up or a bounds check tripped; the
// kernel that saw it returned early and its output is not valid.
// ---------------------------------------------------------------------------
enum StatusCode : int {
  kStatusOk = 0,
  kStatusGemmProducerTimeout = 0x101,
  kStatusGemmMmaTimeout = 0x102,
  kStatusGemmEpilogueTimeout = 0x103,
  kStatusMhaLoadTimeout = 0x201,
  kStatusMhaMmaTimeout = 0x202,
  kStatusMhaSoftmaxTimeout = 0x203,
  kStatusBadOffsets = 0x301,
  kStatusSelfTestTimeout = 0x7F1,  // bt_selftest_bounded_wait(): the wait that nothing satisfies ran out, as intended
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------- programmatic dependent launch
// Every kernel of the library starts with pdl_launch_dependents() (the next kernel of the
// stream may be launched as soon as all CTAs of this one have started) and calls
// pdl_wait() before its first access to global memory that an earlier kernel may have
// written or may still read: the wait returns once the preceding kernel has completed
// and its writes are visible.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Hint: bring the 128-byte line at `p` into L1 (constants such as bias, gamma and beta, asked for
// while the kernel still waits for its predecessor).
__device__ __forceinline__ void prefetch_l1(const void* p) {
  asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking test of a phase (try_wait may suspend the thread for a while before it answers).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wait for a phase with an upper bound.  Returns false when the bound ran out
// or another role of this CTA already gave up (`*abort_flag` non-zero); the
// caller must then leave its loop and fall through to the common teardown.
// The bound is ~2^31 SM cycles (about a second) unless the caller gives another,
// checked every 256 polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag, int* status, int code,
                                                  long long max_cycles = (1ll << 31)) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > max_cycles) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
// `x` is the innermost (contiguous) coordinate and must keep x*elem_size a
// multiple of 16 bytes.  No cluster multicast is used anywhere in this library.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// 2-D tiled store shared -> global (bulk async group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest 0 bulk groups of this thread have finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Makes generic-proxy shared-memory writes visible to the async proxy (UMMA/TMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, fp32 accumulate; issued by ONE thread.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane
// (base_lane + i), columns [col, col+32).  A warp may only touch the lane
// quarter (warp_id % 4) * 32.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// tcgen05.ld 32x32b.x32 into elements [B, B + 32) of a 128-element register array (no address of the array
// is formed, so it stays in registers).
template <int B>
__device__ __forceinline__ void tmem_ld_32x32_at(uint32_t taddr, uint32_t (&r)[128]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[B + 0]), "=r"(r[B + 1]), "=r"(r[B + 2]), "=r"(r[B + 3]), "=r"(r[B + 4]), "=r"(r[B + 5]), "=r"(r[B + 6]),
        "=r"(r[B + 7]), "=r"(r[B + 8]), "=r"(r[B + 9]), "=r"(r[B + 10]), "=r"(r[B + 11]), "=r"(r[B + 12]), "=r"(r[B + 13]),
        "=r"(r[B + 14]), "=r"(r[B + 15]), "=r"(r[B + 16]), "=r"(r[B + 17]), "=r"(r[B + 18]), "=r"(r[B + 19]), "=r"(r[B + 20]),
        "=r"(r[B + 21]), "=r"(r[B + 22]), "=r"(r[B + 23]), "=r"(r[B + 24]), "=r"(r[B + 25]), "=r"(r[B + 26]), "=r"(r[B + 27]),
        "=r"(r[B + 28]), "=r"(r[B + 29]), "=r"(r[B + 30]), "=r"(r[B + 31])
      : "r"(taddr)
      : "memory");
}
// Register -> tensor memory, same lane / column mapping as the loads above.
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
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------------------------- UMMA descriptors (sm_100)
// Shared-memory matrix descriptor, 64 bit:
//   [ 0,14) start address >> 4      [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4 [46,48) version = 1
//   [49,52) base offset = 0         [61,64) layout: 0 none, 2 = 128-byte swizzle
// K-major, 128B swizzle  (rows of 64 fp16 = 128 B, 8-row groups of 1024 B):
//   SBO = distance between 8-row groups; LBO unused.
// MN-major, 128B swizzle (64 contiguous MN elements per k row, 8 k rows = 1024 B):
//   LBO = distance between 64-element chunks along MN; SBO = distance between
//   8-k groups.
__host__ __device__ constexpr uint64_t make_smem_desc_hi(uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t smem_desc(uint64_t hi_template, uint32_t smem_addr) {
  return hi_template | static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
}
// Instruction descriptor for kind::f16, fp16 A/B, fp32 D.
//   [4,6) D format 1 = f32; [7,10) A fmt 0 = f16; [10,13) B fmt 0 = f16;
//   bit 15 A major (0 K / 1 MN); bit 16 B major; [17,23) N>>3; [24,29) M>>4.
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// -------------------------------------------------------------------- maths
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
// Exact-form GELU, x * Phi(x), with one special-function op:
//   gelu(x) = max(x, 0) - 0.5 * |x| * erfc(|x| / sqrt(2)),   erfc(z) = 2^p(z),
// p = degree-5 polynomial fit of log2(erfc(z)) on [0, 4.3] (z is clamped there; beyond,
// erfc < 2e-9).  Maximum absolute error of the result against 0.5*x*(1+erf(x/sqrt 2)) in
// fp32 arithmetic: 6.4e-7 over x in [-8, 8] — far below fp16 resolution of the output.
__device__ __forceinline__ float gelu_erf_fast(float x) {
  const float ax = fabsf(x);
  const float z = fminf(ax * 0.70710678118654752f, 4.3f);
  float p = fmaf(-0.002677350537851453f, z, 0.02833780087530613f);
  p = fmaf(p, z, -0.1465892493724823f);
  p = fmaf(p, z, -0.9199854135513306f);
  p = fmaf(p, z, -1.6274596452713013f);
  p = fmaf(p, z, -3.764020948437974e-05f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(p));
  return fmaf(-0.5f * ax, e, fmaxf(x, 0.f));
}
// Two values at once with the packed fp32 instructions of sm_100 (fma.rn.f32x2: one issue slot for two
// lanes of a 64-bit register pair): the polynomial and the final multiply-add, which are most of the
// instructions of gelu_erf_fast, take half the issue slots.  Same arithmetic, same results.
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ void gelu_erf_fast_pair(float& x0, float& x1) {
  const float a0 = fabsf(x0), a1 = fabsf(x1);
  const unsigned long long z = pack_f32x2(fminf(a0 * 0.70710678118654752f, 4.3f), fminf(a1 * 0.70710678118654752f, 4.3f));
  unsigned long long p = fma_f32x2(pack_f32x2(-0.002677350537851453f, -0.002677350537851453f), z,
                                   pack_f32x2(0.02833780087530613f, 0.02833780087530613f));
  p = fma_f32x2(p, z, pack_f32x2(-0.1465892493724823f, -0.1465892493724823f));
  p = fma_f32x2(p, z, pack_f32x2(-0.9199854135513306f, -0.9199854135513306f));
  p = fma_f32x2(p, z, pack_f32x2(-1.6274596452713013f, -1.6274596452713013f));
  p = fma_f32x2(p, z, pack_f32x2(-3.764020948437974e-05f, -3.764020948437974e-05f));
  float p0, p1, e0, e1;
  unpack_f32x2(p, p0, p1);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(p0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(p1));
  const unsigned long long r = fma_f32x2(pack_f32x2(-0.5f * a0, -0.5f * a1), pack_f32x2(e0, e1),
                                         pack_f32x2(fmaxf(x0, 0.f), fmaxf(x1, 0.f)));
  unpack_f32x2(r, x0, x1);
}
__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh( sqrt(2/pi) (x + 0.044715 x^3) ))
  const float u = 0.7978845608028654f * x * (1.0f + 0.044715f * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace bt
