// Diagnostic: how fast can the warps of a CTA read tensor memory when they do nothing else?
// Every warp reads its 32 lanes x 256 columns over and over with tcgen05.ld of one shape, waits
// for each load and XORs the words together.  The figure (bytes per clock and SM) is the ceiling
// against which the rate of an epilogue or a softmax can be judged: if they consume tensor memory
// far below it, tensor memory is not what bounds them.  Not part of the stable ABI.
#include "common.cuh"
#include "kernels.h"

namespace bt {
namespace {

__device__ __forceinline__ void probe_ld_x64(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void probe_ld_x128(uint32_t taddr, uint32_t (&r)[128]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x128.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63, %64, %65, %66, %67, %68, %69, %70, %71, %72, %73, %74, %75, %76, %77, %78, %79, %80, %81, %82, %83, %84, %85, %86, %87, %88, %89, %90, %91, %92, %93, %94, %95, %96, %97, %98, %99, %100, %101, %102, %103, %104, %105, %106, %107, %108, %109, %110, %111, %112, %113, %114, %115, %116, %117, %118, %119, %120, %121, %122, %123, %124, %125, %126, %127}, [%128];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]), "=r"(r[64]), "=r"(r[65]), "=r"(r[66]), "=r"(r[67]), "=r"(r[68]), "=r"(r[69]), "=r"(r[70]), "=r"(r[71]), "=r"(r[72]), "=r"(r[73]), "=r"(r[74]), "=r"(r[75]), "=r"(r[76]), "=r"(r[77]), "=r"(r[78]), "=r"(r[79]), "=r"(r[80]), "=r"(r[81]), "=r"(r[82]), "=r"(r[83]), "=r"(r[84]), "=r"(r[85]), "=r"(r[86]), "=r"(r[87]), "=r"(r[88]), "=r"(r[89]), "=r"(r[90]), "=r"(r[91]), "=r"(r[92]), "=r"(r[93]), "=r"(r[94]), "=r"(r[95]), "=r"(r[96]), "=r"(r[97]), "=r"(r[98]), "=r"(r[99]), "=r"(r[100]), "=r"(r[101]), "=r"(r[102]), "=r"(r[103]), "=r"(r[104]), "=r"(r[105]), "=r"(r[106]), "=r"(r[107]), "=r"(r[108]), "=r"(r[109]), "=r"(r[110]), "=r"(r[111]), "=r"(r[112]), "=r"(r[113]), "=r"(r[114]), "=r"(r[115]), "=r"(r[116]), "=r"(r[117]), "=r"(r[118]), "=r"(r[119]), "=r"(r[120]), "=r"(r[121]), "=r"(r[122]), "=r"(r[123]), "=r"(r[124]), "=r"(r[125]), "=r"(r[126]), "=r"(r[127])
               : "r"(taddr)
               : "memory");
}

// MODE 0: .x32, 1: .x64, 2: .x128; a wait after every load.
template <int MODE>
__global__ void __launch_bounds__(256) tmem_read_probe_kernel(int reps, long long* clocks, uint32_t* sink) {
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    tmem_alloc(&slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t base = slot;
  // warps 0-3 read columns 0..255 of their lane quarter, warps 4-7 columns 256..511
  const uint32_t t0 = base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + (warp >> 2) * 256;
  uint32_t acc = 0;
  __syncthreads();
  const long long c0 = clock64();
  for (int r = 0; r < reps; ++r) {
    if (MODE == 0) {
      for (int c = 0; c < 256; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t0 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc ^= v[i];
      }
    } else if (MODE == 1) {
      for (int c = 0; c < 256; c += 64) {
        uint32_t v[64];
        probe_ld_x64(t0 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 64; ++i) acc ^= v[i];
      }
    } else {
      for (int c = 0; c < 256; c += 128) {
        uint32_t v[128];
        probe_ld_x128(t0 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 128; ++i) acc ^= v[i];
      }
    }
  }
  const long long c1 = clock64();
  __syncthreads();
  if (threadIdx.x == 0) clocks[blockIdx.x] = c1 - c0;
  sink[blockIdx.x * blockDim.x + threadIdx.x] = acc;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(base, 512);
  }
}

}  // namespace
}  // namespace bt

// mode 0/1/2 = tcgen05.ld .x32/.x64/.x128, warps = 4 or 8 per CTA, one CTA per SM (`ctas` of them).
// `clocks_dev`: `ctas` long long, `sink_dev`: ctas * 256 uint32 (device).  Each CTA reads
// reps * warps * 32 lanes * 256 columns * 4 bytes in clocks_dev[cta] clocks.
extern "C" int bt_debug_tmem_read_probe(int mode, int warps, int ctas, int reps, long long* clocks_dev,
                                         unsigned int* sink_dev, void* stream_v) {
  if ((warps != 4 && warps != 8) || ctas <= 0 || reps <= 0 || !clocks_dev || !sink_dev) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const dim3 grid(ctas), block(warps * 32);
  switch (mode) {
    case 0: bt::tmem_read_probe_kernel<0><<<grid, block, 0, stream>>>(reps, clocks_dev, sink_dev); break;
    case 1: bt::tmem_read_probe_kernel<1><<<grid, block, 0, stream>>>(reps, clocks_dev, sink_dev); break;
    case 2: bt::tmem_read_probe_kernel<2><<<grid, block, 0, stream>>>(reps, clocks_dev, sink_dev); break;
    default: return -1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
