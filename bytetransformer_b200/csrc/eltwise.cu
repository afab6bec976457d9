// HBM-bound row kernels: (add bias + residual +) LayerNorm, the same fused with
// the packed -> padded scatter, add-bias + GELU, and masked softmax.
//
// All of them use 16-byte global accesses and warp-shuffle reductions; one warp
// owns one row, so no shared memory or block barrier is needed.
//
// Reference counterparts (paths relative to the ByteTransformer root):
//   layernorm_rows_kernel<false>  add_bias_input_layernorm{,_v2}
//                                 (bytetransformer/include/layernorm.h:273-296, src/layernorm.cu:89-102)
//   layernorm_rows_kernel<true>   add_bias_input_layernorm_restore_output{,_v2}
//                                 (layernorm.h:334-373, layernorm.cu:126-148)
//   add_bias_gelu_kernel          add_bias_gelu (bytetransformer/src/gemm_bias_act.cu:32-47)
//   masked_softmax_kernel         softmax_kernel_warp_half2* (bytetransformer/include/softmax.h:25-297)
// Differences kept on purpose: the sums x + bias + residual are formed in fp32
// (the reference adds in fp16 first, layernorm.h:289-290); statistics are
// two-pass (mean, then centred variance) in fp32 as in the reference.
//
// Algorithmic bytes per row of H halves: LayerNorm reads x (+ residual) and
// writes out: 6*H bytes with residual, 4*H without; the restore variant writes
// every padded row (2*H bytes each, zeros for padding).
#include "common.cuh"
#include "kernels.h"
#include "../../include/bt_b200.h"

namespace bt {

namespace {

constexpr int kLnWarps = 4;
constexpr int kLnMaxVec = 4;  // register-resident rows up to 4*32*8 = 1024 halves
constexpr int kLnMaxSplit = 8;  // most fp32 partial sums a row may arrive in

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  q.x = pack_half2(f[0], f[1]);
  q.y = pack_half2(f[2], f[3]);
  q.z = pack_half2(f[4], f[5]);
  q.w = pack_half2(f[6], f[7]);
  return q;
}

template <bool GB_FP32>
__device__ __forceinline__ void load_gb8(const void* p, int vec, float (&f)[8]) {
  if (GB_FP32) {
    const float4* fp = reinterpret_cast<const float4*>(p) + 2 * vec;
    const float4 a = __ldg(fp), b = __ldg(fp + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + vec);
    unpack8(q, f);
  }
}

// RESTORE = false: rows [0, M) of x -> rows [0, M) of out.
// RESTORE = true : grid covers the B*S padded rows; row (b,i) reads packed row
//                  batch_idx[b]+i when i < len_b, else writes zeros.
template <bool RESTORE, bool GB_FP32, bool X_FP32, int NVEC, bool SPLIT>
__global__ void __launch_bounds__(kLnWarps * 32)
layernorm_rows_kernel(const void* __restrict__ x_v, const __half* __restrict__ bias,
                      const __half* __restrict__ residual, const void* __restrict__ gamma,
                      const void* __restrict__ beta, __half* __restrict__ out, const int* __restrict__ m_dev,
                      int m_rows, const int* __restrict__ batch_idx, int S, int hidden, float eps, LnSplit split) {
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = hidden / 8;
  {
    // gamma and beta are written by no kernel of the chain: ask for their lines while waiting
    const int gb_bytes = hidden * (GB_FP32 ? 4 : 2);
    const int off = static_cast<int>(threadIdx.x) * 128;
    if (off < gb_bytes) {
      prefetch_l1(reinterpret_cast<const uint8_t*>(gamma) + off);
      prefetch_l1(reinterpret_cast<const uint8_t*>(beta) + off);
    }
  }
  pdl_wait();
  // Rows are walked with a grid stride (the grid is capped at a few waves of the machine), so
  // a warp keeps streaming instead of paying a block launch per row.
  long long row_limit = m_rows;
  if (!RESTORE && m_dev != nullptr) {
    const int md = __ldg(m_dev);
    row_limit = md < m_rows ? md : m_rows;
  }
  for (long long row = static_cast<long long>(blockIdx.x) * kLnWarps + warp; row < row_limit;
       row += static_cast<long long>(gridDim.x) * kLnWarps) {
  long long src_row = row;
  if (RESTORE) {
    const int b = static_cast<int>(row / S);
    const int i = static_cast<int>(row - static_cast<long long>(b) * S);
    const int off = __ldg(batch_idx + b);
    const int len = __ldg(batch_idx + b + 1) - off;
    if (i >= len) {
      uint4* o4 = reinterpret_cast<uint4*>(out + row * hidden);
      for (int v = lane; v < nvec; v += 32) o4[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    src_row = off + i;
  }

  const uint4* x4 = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(x_v) + src_row * hidden);
  const float4* xf = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x_v) + src_row * hidden);
  const uint4* r4 = residual ? reinterpret_cast<const uint4*>(residual + src_row * hidden) : nullptr;
  const uint4* b4 = bias ? reinterpret_cast<const uint4*>(bias) : nullptr;

  float val[NVEC][8];
  float sum = 0.f;
#pragma unroll
  for (int it = 0; it < NVEC; ++it) {
    const int v = it * 32 + lane;
    if (v < nvec) {
      if (X_FP32) {
        const float4 a = __ldg(xf + 2 * v), b = __ldg(xf + 2 * v + 1);
        val[it][0] = a.x; val[it][1] = a.y; val[it][2] = a.z; val[it][3] = a.w;
        val[it][4] = b.x; val[it][5] = b.y; val[it][6] = b.z; val[it][7] = b.w;
        // the sum arrives in `split.n` <= kLnMaxSplit fp32 parts (K ranges of the GEMM before); the loads of
        // all parts are independent and issued together
        if (SPLIT) {
          float4 c[kLnMaxSplit - 1], d[kLnMaxSplit - 1];
#pragma unroll
          for (int sp = 1; sp < kLnMaxSplit; ++sp) {
            const float4* xs = xf + sp * (split.stride / 4);
            c[sp - 1] = sp < split.n ? __ldg(xs + 2 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
            d[sp - 1] = sp < split.n ? __ldg(xs + 2 * v + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int sp = 0; sp < kLnMaxSplit - 1; ++sp) {
            val[it][0] += c[sp].x; val[it][1] += c[sp].y; val[it][2] += c[sp].z; val[it][3] += c[sp].w;
            val[it][4] += d[sp].x; val[it][5] += d[sp].y; val[it][6] += d[sp].z; val[it][7] += d[sp].w;
          }
        }
      } else {
        unpack8(__ldg(x4 + v), val[it]);
      }
      if (r4) {
        float t[8];
        unpack8(__ldg(r4 + v), t);
#pragma unroll
        for (int k = 0; k < 8; ++k) val[it][k] += t[k];
      }
      if (b4) {
        float t[8];
        unpack8(__ldg(b4 + v), t);
#pragma unroll
        for (int k = 0; k < 8; ++k) val[it][k] += t[k];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) sum += val[it][k];
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) val[it][k] = 0.f;
    }
  }
  const float mean = warp_sum(sum) / static_cast<float>(hidden);
  float sq = 0.f;
#pragma unroll
  for (int it = 0; it < NVEC; ++it) {
    if (it * 32 + lane < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float d = val[it][k] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / static_cast<float>(hidden) + eps);

  uint4* o4 = reinterpret_cast<uint4*>(out + row * hidden);
#pragma unroll
  for (int it = 0; it < NVEC; ++it) {
    const int v = it * 32 + lane;
    if (v < nvec) {
      float g[8], bt_[8], o[8];
      load_gb8<GB_FP32>(gamma, v, g);
      load_gb8<GB_FP32>(beta, v, bt_);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = fmaf((val[it][k] - mean) * rstd, g[k], bt_[k]);
      o4[v] = pack8(o);
    }
  }
  }  // row loop
}

template <bool RESTORE, bool GB_FP32, bool X_FP32, bool SPLIT>
cudaError_t launch_ln_nvec(int nvec_needed, dim3 grid, cudaStream_t stream, const void* x, const __half* bias,
                           const __half* residual, const void* gamma, const void* beta, __half* out,
                           const int* m_dev, int m_rows, const int* batch_idx, int S, int hidden, float eps,
                           LnSplit split) {
#define BT_LN_CASE(NV)                                                                                        \
  case NV:                                                                                                    \
    return launch_pdl(layernorm_rows_kernel<RESTORE, GB_FP32, X_FP32, NV, SPLIT>, grid, dim3(kLnWarps * 32), 0, stream,  \
                      x, bias, residual, gamma, beta, out, m_dev, m_rows, batch_idx, S, hidden, eps, split);
  switch (nvec_needed) {
    BT_LN_CASE(1)
    BT_LN_CASE(2)
    BT_LN_CASE(3)
    BT_LN_CASE(4)
    default: return cudaErrorInvalidValue;
  }
#undef BT_LN_CASE
  return cudaGetLastError();
}

// x[row, :] = gelu(x[row, :] + bias), in place.  A thread owns one 16-byte column vector (its bias slice
// is read once) and walks down the rows, four rows per trip so that four loads are in flight; the exact-form
// GELU costs one special-function op per element (gelu_erf_fast).  blockIdx.x selects the column block,
// blockIdx.y the first row.
__global__ void __launch_bounds__(128)
add_bias_gelu_kernel(uint4* __restrict__ x, const uint4* __restrict__ bias, const int* __restrict__ m_dev,
                     int m_rows, int nvec, int gelu_kind) {
  pdl_launch_dependents();
  pdl_wait();
  int M = m_rows;
  if (m_dev != nullptr) {
    const int md = __ldg(m_dev);
    M = md < M ? md : M;
  }
  const int v = static_cast<int>(blockIdx.x * blockDim.x + threadIdx.x);
  if (v >= nvec) return;
  float b[8];
  unpack8(__ldg(bias + v), b);
  const int stride = static_cast<int>(gridDim.y);
  for (int r0 = static_cast<int>(blockIdx.y); r0 < M; r0 += 4 * stride) {
    uint4 in[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int r = r0 + u * stride;
      if (r < M) in[u] = x[static_cast<size_t>(r) * nvec + v];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int r = r0 + u * stride;
      if (r < M) {
        float f[8];
        unpack8(in[u], f);
        if (gelu_kind == BT_GELU_TANH) {
#pragma unroll
          for (int k = 0; k < 8; ++k) f[k] = gelu_tanh(f[k] + b[k]);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) f[k] = gelu_erf_fast(f[k] + b[k]);
        }
        x[static_cast<size_t>(r) * nvec + v] = pack8(f);
      }
    }
  }
}

__device__ __forceinline__ float exp2f_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Logits are laid out [nh, B, S, S] as in the reference (softmax.h:33: ((head*B + b)*S + i)*S); S <= 1024.
// VEC path (S % 8 == 0): a warp owns one (b, i) row of the mask and walks the nh heads' logits rows that
// share it, so the additive term (1 - mask) * -10000 is read and converted once per nh rows; the next
// head's row is requested before the current one is worked on.  Everything is in units of log2
// (exp(x) = 2^(x log2 e)): one special-function op per element.  The other path: one warp per logits row.
template <bool VEC, int NIT>
__global__ void __launch_bounds__(128)
masked_softmax_kernel(__half* __restrict__ logits, const __half* __restrict__ mask, int B, int nh, int S,
                      float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * 4 + warp;
  if (VEC) {
    const long long mask_rows = static_cast<long long>(B) * S;
    if (row >= mask_rows) return;
    const int nvec = S / 8;
    const float scale_l2 = scale * 1.4426950408889634f;
    const long long head_stride = mask_rows * S;  // halves between the same (b, i) row of two heads
    __half* lp = logits + row * S;
    float add[NIT][8];
    uint4 raw[2][NIT];  // the rows of the next two heads, in flight
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int v = it * 32 + lane;
      if (v < nvec) {
        raw[0][it] = *(reinterpret_cast<const uint4*>(lp) + v);
        if (nh > 1) raw[1][it] = *(reinterpret_cast<const uint4*>(lp + head_stride) + v);
        float m[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(mask + row * S) + v), m);
#pragma unroll
        for (int k = 0; k < 8; ++k) add[it][k] = fmaf(m[k], 14426.950408889634f, -14426.950408889634f);
      }
    }
    for (int h = 0; h < nh; ++h, lp += head_stride) {
      float val[NIT][8];
      float mx = -INFINITY;
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int v = it * 32 + lane;
        if (v < nvec) {
          unpack8(raw[0][it], val[it]);
          raw[0][it] = raw[1][it];
          if (h + 2 < nh) raw[1][it] = *(reinterpret_cast<const uint4*>(lp + 2 * head_stride) + v);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            val[it][k] = fmaf(val[it][k], scale_l2, add[it][k]);
            mx = fmaxf(mx, val[it][k]);
          }
        }
      }
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        if (it * 32 + lane < nvec) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            val[it][k] = exp2f_fast(val[it][k] - mx);
            sum += val[it][k];
          }
        }
      }
      const float inv = 1.0f / (warp_sum(sum) + 1e-6f);
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int v = it * 32 + lane;
        if (v < nvec) {
#pragma unroll
          for (int k = 0; k < 8; ++k) val[it][k] *= inv;
          *(reinterpret_cast<uint4*>(lp) + v) = pack8(val[it]);
        }
      }
    }
  } else {
    const long long rows = static_cast<long long>(B) * nh * S;
    if (row >= rows) return;
    const int i = static_cast<int>(row % S);
    const int b = static_cast<int>((row / S) % B);
    __half* lp = logits + row * S;
    const __half* mp = mask + (static_cast<long long>(b) * S + i) * S;
    float val[32];
    float mx = -INFINITY;
#pragma unroll
    for (int it = 0; it < 32; ++it) {
      const int j = it * 32 + lane;
      if (j < S) {
        val[it] = fmaf(__half2float(lp[j]), scale, (1.0f - __half2float(mp[j])) * -10000.0f);
        mx = fmaxf(mx, val[it]);
      }
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < 32; ++it) {
      if (it * 32 + lane < S) {
        val[it] = __expf(val[it] - mx);
        sum += val[it];
      }
    }
    const float inv = 1.0f / (warp_sum(sum) + 1e-6f);
#pragma unroll
    for (int it = 0; it < 32; ++it) {
      const int j = it * 32 + lane;
      if (j < S) lp[j] = __float2half_rn(val[it] * inv);
    }
  }
}

}  // namespace

// at most 16 resident blocks (64 warps) per SM on 148 SMs
static unsigned ln_grid(long long blocks_needed) {
  const long long cap = 148LL * 16;
  return static_cast<unsigned>(blocks_needed < cap ? (blocks_needed < 1 ? 1 : blocks_needed) : cap);
}

template <bool RESTORE>
static cudaError_t launch_ln_dispatch(bool gb_fp32, bool x_fp32, int nv, dim3 grid, cudaStream_t stream, const void* x,
                                      const __half* bias, const __half* residual, const void* gamma, const void* beta,
                                      __half* out, const int* m_dev, int m_rows, const int* batch_idx, int S,
                                      int hidden, float eps, LnSplit split) {
#define BT_LN_ARGS nv, grid, stream, x, bias, residual, gamma, beta, out, m_dev, m_rows, batch_idx, S, hidden, eps, split
  if (split.n > 1) {  // fp32 partial sums (checked by the callers)
    if (gb_fp32) return launch_ln_nvec<RESTORE, true, true, true>(BT_LN_ARGS);
    return launch_ln_nvec<RESTORE, false, true, true>(BT_LN_ARGS);
  }
  if (gb_fp32) {
    if (x_fp32) return launch_ln_nvec<RESTORE, true, true, false>(BT_LN_ARGS);
    return launch_ln_nvec<RESTORE, true, false, false>(BT_LN_ARGS);
  }
  if (x_fp32) return launch_ln_nvec<RESTORE, false, true, false>(BT_LN_ARGS);
  return launch_ln_nvec<RESTORE, false, false, false>(BT_LN_ARGS);
#undef BT_LN_ARGS
}

cudaError_t launch_layernorm(const void* x, bool x_fp32, const __half* bias, const __half* residual,
                             const void* gamma, const void* beta, bool gb_fp32, __half* out, const int* m_dev,
                             int m_rows, int hidden, float eps, cudaStream_t stream, LnSplit split) {
  if (hidden % 8 != 0 || hidden > kLnMaxVec * 256 || m_rows <= 0) return cudaErrorInvalidValue;
  if (split.n > 1 && (!x_fp32 || split.stride % 4 != 0 || split.n > kLnMaxSplit)) return cudaErrorInvalidValue;
  const int nv = (hidden / 8 + 31) / 32;
  dim3 grid(ln_grid((m_rows + kLnWarps - 1) / kLnWarps));
  return launch_ln_dispatch<false>(gb_fp32, x_fp32, nv, grid, stream, x, bias, residual, gamma, beta, out, m_dev,
                                   m_rows, nullptr, 0, hidden, eps, split);
}

cudaError_t launch_layernorm_restore(const void* x, bool x_fp32, const __half* bias, const __half* residual,
                                     const void* gamma, const void* beta, bool gb_fp32, __half* out_padded,
                                     const int* batch_idx, int B, int S, int hidden, float eps,
                                     cudaStream_t stream, LnSplit split) {
  if (hidden % 8 != 0 || hidden > kLnMaxVec * 256 || B <= 0 || S <= 0) return cudaErrorInvalidValue;
  if (split.n > 1 && (!x_fp32 || split.stride % 4 != 0 || split.n > kLnMaxSplit)) return cudaErrorInvalidValue;
  const int nv = (hidden / 8 + 31) / 32;
  const long long rows = static_cast<long long>(B) * S;
  dim3 grid(ln_grid((rows + kLnWarps - 1) / kLnWarps));
  return launch_ln_dispatch<true>(gb_fp32, x_fp32, nv, grid, stream, x, bias, residual, gamma, beta, out_padded,
                                  nullptr, static_cast<int>(rows), batch_idx, S, hidden, eps, split);
}

cudaError_t launch_add_bias_gelu(__half* x, const __half* bias, const int* m_dev, int m_rows, int n, int gelu_kind,
                                 cudaStream_t stream) {
  if (n % 8 != 0 || m_rows <= 0) return cudaErrorInvalidValue;
  const int nvec = n / 8;
  const unsigned gx = static_cast<unsigned>((nvec + 127) / 128);
  // enough row groups for ~16 CTAs per SM, never more than rows
  long long gy = (148LL * 16 + gx - 1) / gx;
  if (gy > m_rows) gy = m_rows;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  return launch_pdl(add_bias_gelu_kernel, dim3(gx, static_cast<unsigned>(gy)), dim3(128), 0, stream,
                    reinterpret_cast<uint4*>(x), reinterpret_cast<const uint4*>(bias), m_dev, m_rows, nvec, gelu_kind);
}

cudaError_t launch_masked_softmax(__half* logits, const __half* mask, int B, int nh, int S, float scale,
                                  cudaStream_t stream) {
  if (S <= 0 || S > 1024 || B <= 0 || nh <= 0) return cudaErrorInvalidValue;
  const long long rows = static_cast<long long>(B) * nh * S;
  if (S % 8 == 0) {  // a warp per mask row, looping over the heads
    dim3 grid_v(static_cast<unsigned>((static_cast<long long>(B) * S + 3) / 4));
    if (S <= 256) return launch_pdl(masked_softmax_kernel<true, 1>, grid_v, dim3(128), 0, stream, logits, mask, B, nh, S, scale);
    if (S <= 512) return launch_pdl(masked_softmax_kernel<true, 2>, grid_v, dim3(128), 0, stream, logits, mask, B, nh, S, scale);
    return launch_pdl(masked_softmax_kernel<true, 4>, grid_v, dim3(128), 0, stream, logits, mask, B, nh, S, scale);
  }
  dim3 grid(static_cast<unsigned>((rows + 3) / 4));
  return launch_pdl(masked_softmax_kernel<false, 4>, grid, dim3(128), 0, stream, logits, mask, B, nh, S, scale);
}

// ---------------------------------------------------------------------------------------
// Self-test of the bounded wait every pipeline of the library relies on: one CTA waits on an
// mbarrier that nothing will ever arrive on.  The wait must give up after `max_cycles`, record
// kStatusSelfTestTimeout in the status word and let the kernel return normally, leaving the
// context usable.  Nothing faults, traps or spins without a limit.
// ---------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(int* status, long long max_cycles, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag_s;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag_s = 0;
    fence_mbar_init();
  }
  __syncthreads();
  volatile int* abort_flag = &abort_flag_s;
  if (threadIdx.x == 0) {
    // phase 0 never completes: no thread arrives on `bar`
    const bool got = mbar_wait_bounded(&bar, 0u, abort_flag, status, kStatusSelfTestTimeout, max_cycles);
    if (gave_up != nullptr) *gave_up = got ? 0 : 1;
  } else if (threadIdx.x == 32) {
    // a second role that sees the first one give up through the CTA's abort flag
    long long spins = 0;
    while (*abort_flag == 0 && spins < max_cycles) spins += 64, __nanosleep(64);
  }
  __syncthreads();
}
}  // namespace

cudaError_t launch_bounded_wait_selftest(int* status, long long max_cycles, int* gave_up, cudaStream_t stream) {
  if (max_cycles < 1024) max_cycles = 1024;
  if (max_cycles > (1ll << 31)) max_cycles = (1ll << 31);
  return launch_pdl(bounded_wait_selftest_kernel, dim3(1), dim3(64), 0, stream, status, max_cycles, gave_up);
}

}  // namespace bt
