// Padding removal bookkeeping: mask -> lengths -> prefix-sum offsets, and the
// pack (padded -> packed) / restore (packed -> padded, zero fill) row copies.
//
// Integer results are bit-exact with the reference's
// `parallel_prefix` (bytetransformer/include/remove_padding.h:36-86):
//   len_b        = #{ j : mask[b,0,j] >= 0.5 }          (only mask row 0 is read)
//   batch_idx[0] = 0, batch_idx[b+1] = batch_idx[b] + len_b   (batch_idx[B] = T)
//   word_idx[batch_idx[b] + i] = b*S + i  for i < len_b
// Unlike the reference there is no device-to-host copy of T: the consumers read
// batch_idx[B] on the device.
//
// Both are HBM-bound.  Algorithmic bytes: offsets 2*B*S (mask row 0) + 4*(B+1) +
// 4*T; pack 4*T*H (read + write fp16); restore 2*T*H + 2*B*S*H.
#include "common.cuh"
#include "kernels.h"

namespace bt {

namespace {

constexpr int kOffThreads = 1024;

__global__ void __launch_bounds__(kOffThreads, 1)
build_offsets_kernel(const __half* __restrict__ mask, int B, int S, int* __restrict__ batch_idx,
                     int* __restrict__ word_idx) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_warps = kOffThreads / 32;
  const __half half_thr = __float2half(0.5f);

  // 1. lengths: one warp per sequence; len goes to batch_idx[b+1] for now
  const bool vec_ok = (S % 8) == 0;
  for (int b = warp; b < B; b += n_warps) {
    const __half* row = mask + static_cast<size_t>(b) * S * S;
    int cnt = 0;
    if (vec_ok) {
      const uint4* row4 = reinterpret_cast<const uint4*>(row);
      for (int v = lane; v < S / 8; v += 32) {
        const uint4 q = __ldg(row4 + v);
        const __half* hp = reinterpret_cast<const __half*>(&q);
#pragma unroll
        for (int i = 0; i < 8; ++i) cnt += __hge(hp[i], half_thr) ? 1 : 0;
      }
    } else {
      for (int j = lane; j < S; j += 32) cnt += __hge(row[j], half_thr) ? 1 : 0;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) batch_idx[b + 1] = cnt;
  }
  if (tid == 0) {
    batch_idx[0] = 0;
    carry_s = 0;
  }
  __syncthreads();

  // 2. inclusive scan of batch_idx[1..B] in chunks of 1024 (any B)
  for (int base = 0; base < B; base += kOffThreads) {
    const int i = base + tid;
    const int len = i < B ? batch_idx[i + 1] : 0;
    int x = len;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int carry = carry_s;
    const int incl = x + (warp > 0 ? warp_sums[warp - 1] : 0) + carry;
    if (i < B) batch_idx[i + 1] = incl;
    __syncthreads();
    if (tid == kOffThreads - 1) carry_s = incl;
    __syncthreads();
  }

  // 3. packed row -> padded row map
  for (int b = warp; b < B; b += n_warps) {
    const int off = batch_idx[b];
    const int len = batch_idx[b + 1] - off;
    for (int i = lane; i < len; i += 32) word_idx[off + i] = b * S + i;
  }
}

// With right padding the valid rows of sequence b are one contiguous run of
// len_b*H halves in both layouts, so pack / restore are B segment copies done
// with 16-byte accesses (the reference gathers row by row through word_idx,
// remove_padding.h:104-121).
__global__ void __launch_bounds__(256)
pack_rows_kernel(const uint4* __restrict__ padded, uint4* __restrict__ packed, const int* __restrict__ batch_idx,
                 int S, int vec_per_row) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  const int off = __ldg(batch_idx + b);
  const int len = __ldg(batch_idx + b + 1) - off;
  const long long n = static_cast<long long>(len) * vec_per_row;
  const uint4* src = padded + static_cast<size_t>(b) * S * vec_per_row;
  uint4* dst = packed + static_cast<size_t>(off) * vec_per_row;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < n;
       v += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[v] = __ldg(src + v);
}

__global__ void __launch_bounds__(256)
restore_rows_kernel(const uint4* __restrict__ packed, uint4* __restrict__ padded, const int* __restrict__ batch_idx,
                    int S, int vec_per_row) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  const int off = __ldg(batch_idx + b);
  const int len = __ldg(batch_idx + b + 1) - off;
  const long long n = static_cast<long long>(len) * vec_per_row;
  const long long total = static_cast<long long>(S) * vec_per_row;
  const uint4* src = packed + static_cast<size_t>(off) * vec_per_row;
  uint4* dst = padded + static_cast<size_t>(b) * S * vec_per_row;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[v] = v < n ? __ldg(src + v) : make_uint4(0u, 0u, 0u, 0u);
}

__global__ void __launch_bounds__(256) uniform_offsets_kernel(int* __restrict__ batch_idx, int B, int S,
                                                              int* __restrict__ clear_flag) {
  pdl_launch_dependents();
  pdl_wait();
  if (clear_flag != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *clear_flag = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i <= B; i += gridDim.x * blockDim.x) batch_idx[i] = i * S;
}

// One CTA per sequence.  len = number of entries >= 0.5 in row 0 (the definition of the packed path);
// the mask is a right-padding mask iff each of the first len rows allows exactly the first len keys
// and no later row allows a key from len on (padding rows may allow the same prefix, as when the key
// mask is broadcast over the rows, or nothing, as in an outer product of the length mask).  The second
// condition is what tells a causal mask (row 0 = one key) from a sequence of length one.
__global__ void __launch_bounds__(256)
mask_is_right_padded_kernel(const __half* __restrict__ mask, int B, int S, int* __restrict__ flag) {
  __shared__ int s_len;
  __shared__ int s_bad;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const __half* m = mask + static_cast<size_t>(b) * S * S;
  const __half half_thr = __float2half(0.5f);
  if (threadIdx.x == 0) {
    s_len = 0;
    s_bad = 0;
  }
  __syncthreads();
  int cnt = 0;
  for (int j = threadIdx.x; j < S; j += blockDim.x) cnt += __hge(m[j], half_thr) ? 1 : 0;
  if (cnt) atomicAdd(&s_len, cnt);
  __syncthreads();
  const int len = s_len;
  bool bad = false;
  const long long n = static_cast<long long>(S) * S;
  for (long long e = threadIdx.x; e < n && !bad; e += blockDim.x) {
    const int i = static_cast<int>(e / S);
    const int j = static_cast<int>(e % S);
    const bool allowed = __hge(m[e], half_thr);
    bad = (i < len) ? (allowed != (j < len)) : (allowed && j >= len);
  }
  if (bad) s_bad = 1;
  __syncthreads();
  if (threadIdx.x == 0 && s_bad) atomicExch(flag, 0);
}

// General-mask attention: for every (sequence, tile of 128 query rows) the number of leading keys that
// matter.  A key whose mask value is exactly 0 gets -10000 added to its score and an exponential of 0,
// so the key tiles behind the last non-zero mask entry of every row of the query tile can be left out -
// unless a row has no non-zero entry at all: then all its scores are shifted alike, its softmax runs
// over ALL keys, and the bound of its tile is the full length.  Thread = one query row, scanned from
// the end; CTA = one query tile.
__global__ void __launch_bounds__(128)
mask_key_bound_kernel(const __half* __restrict__ mask, int S, int* __restrict__ bound) {
  __shared__ int s_bound;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) s_bound = 0;
  __syncthreads();
  const int b = blockIdx.y;
  const int row = blockIdx.x * 128 + threadIdx.x;
  if (row < S) {
    const __half* m = mask + (static_cast<size_t>(b) * S + row) * S;
    const __half zero = __float2half(0.f);
    int last = -1;
    int j = S - 1;
    if ((S & 7) == 0) {
      // 16-byte steps while the vector is all zero
      for (; j >= 7 && last < 0; j -= 8) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(m + j - 7));
        if ((v.x | v.y | v.z | v.w) & 0x7FFF7FFFu) {  // some half is not +-0
          for (int k = j; k > j - 8; --k)
            if (__hne(m[k], zero)) {
              last = k;
              break;
            }
        }
      }
    } else {
      for (; j >= 0 && last < 0; --j)
        if (__hne(m[j], zero)) last = j;
    }
    atomicMax(&s_bound, last < 0 ? S : last + 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) bound[b * gridDim.x + blockIdx.x] = s_bound;
}

// The mask of the general path as one bit per (query, key): bit k of a row's word k/32 is set iff
// mask[row, k] == 1.  `flag` (zero beforehand) is raised when some entry is neither 0 nor 1: the attention
// kernel then keeps adding the fp16 mask itself.  Warp per mask row; a row's words are `stride_words`
// apart (a multiple of 4, so that the 128 bits of a key tile are one aligned 16-byte load).
__global__ void __launch_bounds__(256)
mask_bits_kernel(const __half* __restrict__ mask, int S, long long rows, uint32_t* __restrict__ bits,
                 int stride_words, int* __restrict__ flag) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const unsigned short* m = reinterpret_cast<const unsigned short*>(mask) + row * S;
  uint32_t* out = bits + row * stride_words;
  bool odd = false;  // an entry that is neither +-0 nor 1
  if ((S & 7) == 0) {
    const int nvec = S >> 3;
    for (int v0 = 0; v0 < nvec; v0 += 32) {
      const int v = v0 + lane;
      uint32_t byte = 0;
      if (v < nvec) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(m) + v);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t lo = w[i] & 0xffffu, hi = w[i] >> 16;
          byte |= (lo == 0x3c00u ? 1u : 0u) << (2 * i);
          byte |= (hi == 0x3c00u ? 1u : 0u) << (2 * i + 1);
          odd = odd || (lo != 0x3c00u && (lo & 0x7fffu) != 0u) || (hi != 0x3c00u && (hi & 0x7fffu) != 0u);
        }
      }
      uint32_t part = byte << ((lane & 3) * 8);
      part |= __shfl_xor_sync(0xffffffffu, part, 1);
      part |= __shfl_xor_sync(0xffffffffu, part, 2);
      if ((lane & 3) == 0 && v < nvec) out[v >> 2] = part;
    }
  } else {
    for (int k0 = 0; k0 < S; k0 += 32) {
      const int k = k0 + lane;
      const uint32_t h = k < S ? m[k] : 0u;
      odd = odd || (h != 0x3c00u && (h & 0x7fffu) != 0u);
      const uint32_t word = __ballot_sync(0xffffffffu, h == 0x3c00u);
      if (lane == 0) out[k0 >> 5] = word;
    }
  }
  if (__any_sync(0xffffffffu, odd) && lane == 0) atomicOr(flag, 1);
}

__global__ void set_flag_kernel(int* flag, int v) {
  pdl_launch_dependents();
  pdl_wait();
  *flag = v;
}

inline int copy_grid_x(int S, int vec_per_row) {
  const long long total = static_cast<long long>(S) * vec_per_row;
  long long g = (total + 256 * 4 - 1) / (256 * 4);  // ~4 vectors (64 B) per thread
  if (g < 1) g = 1;
  if (g > 1024) g = 1024;
  return static_cast<int>(g);
}

}  // namespace

cudaError_t launch_build_offsets(const __half* mask, int B, int S, int* batch_idx, int* word_idx,
                                 cudaStream_t stream) {
  return launch_pdl(build_offsets_kernel, dim3(1), dim3(kOffThreads), 0, stream, mask, B, S, batch_idx, word_idx);
}

cudaError_t launch_uniform_offsets(int* batch_idx, int B, int S, cudaStream_t stream, int* clear_flag) {
  const int grid = (B + 1 + 255) / 256;
  return launch_pdl(uniform_offsets_kernel, dim3(grid), dim3(256), 0, stream, batch_idx, B, S, clear_flag);
}

int mask_bits_stride_words(int S) { return ((S + 127) / 128) * 4; }

cudaError_t launch_mask_bits(const __half* mask, int B, int S, uint32_t* bits, int* flag_dev, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return cudaErrorInvalidValue;
  const long long rows = static_cast<long long>(B) * S;
  return launch_pdl(mask_bits_kernel, dim3(static_cast<unsigned>((rows + 7) / 8)), dim3(256), 0, stream, mask, S, rows,
                    bits, mask_bits_stride_words(S), flag_dev);
}

cudaError_t launch_mask_is_right_padded(const __half* mask, int B, int S, int* flag_dev, cudaStream_t stream) {
  cudaError_t e = launch_pdl(set_flag_kernel, dim3(1), dim3(1), 0, stream, flag_dev, 1);
  if (e != cudaSuccess) return e;
  return launch_pdl(mask_is_right_padded_kernel, dim3(B), dim3(256), 0, stream, mask, B, S, flag_dev);
}

cudaError_t launch_mask_key_bound(const __half* mask, int B, int S, int* bound_dev, cudaStream_t stream) {
  if (B <= 0 || B > 65535 || S <= 0) return cudaErrorInvalidValue;
  return launch_pdl(mask_key_bound_kernel, dim3((S + 127) / 128, B), dim3(128), 0, stream, mask, S, bound_dev);
}

cudaError_t launch_pack_rows(const __half* padded, __half* packed, const int* batch_idx, int B, int S, int hidden,
                             cudaStream_t stream) {
  const int vec = hidden / 8;
  dim3 grid(copy_grid_x(S, vec), B);
  return launch_pdl(pack_rows_kernel, grid, dim3(256), 0, stream, reinterpret_cast<const uint4*>(padded),
                    reinterpret_cast<uint4*>(packed), batch_idx, S, vec);
}

cudaError_t launch_restore_rows(const __half* packed, __half* padded, const int* batch_idx, int B, int S,
                                int hidden, cudaStream_t stream) {
  const int vec = hidden / 8;
  dim3 grid(copy_grid_x(S, vec), B);
  return launch_pdl(restore_rows_kernel, grid, dim3(256), 0, stream, reinterpret_cast<const uint4*>(packed),
                    reinterpret_cast<uint4*>(padded), batch_idx, S, vec);
}

}  // namespace bt
