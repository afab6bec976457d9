// The two steps either side of the encoder stack in a BERT model:
//
//   embedding front end:  x[b,s,:] = LayerNorm(word[token_ids[b,s]] + pos[position] + type[type_ids[b,s]])
//   pooler back end:      pooled[b,:] = tanh(y[b,0,:] * W + bias)
//
// The reference stops short of both: its infer parameters carry `position_ids` /
// `token_type_ids` that nothing reads (bytetransformer/include/bert_transformer.h:93-95) and
// an unused kernel shows the intended fusion of the embedding LayerNorm with packing
// (bytetransformer/include/layernorm.h:219-240).  Both kernels are HBM/latency-bound row
// kernels: a warp per token (16-byte gathers, fp32 two-pass statistics) and a CTA per
// (sequence, 64 output columns) for the B x H x H pooler product.
//
// Algorithmic bytes: embedding 3*2*H read + 2*H written per token (table rows mostly come
// from L2); pooler 2*H*H of weights per launch (re-read by the B sequences from L2).
#include "common.cuh"
#include "kernels.h"

namespace bt {

namespace {

constexpr int kEmbWarps = 8;

// NVEC = 16-byte vectors (8 halves) per lane: hidden <= NVEC * 256.
template <bool GB_FP32, int NVEC>
__global__ void __launch_bounds__(kEmbWarps * 32)
embedding_layernorm_kernel(const __half* __restrict__ word_emb, const __half* __restrict__ pos_emb,
                           const __half* __restrict__ type_emb, const void* __restrict__ gamma,
                           const void* __restrict__ beta, const int* __restrict__ token_ids,
                           const int* __restrict__ type_ids, const int* __restrict__ position_ids,
                           __half* __restrict__ out, int rows, int seq_len, int hidden, int vocab, int max_pos,
                           int n_types, float eps, const int* __restrict__ word_idx, const int* __restrict__ t_dev) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = hidden >> 3;
  const float inv_h = 1.0f / static_cast<float>(hidden);
  // Packed output (word_idx != null): output row r is the r-th valid token, whose ids sit at padded
  // position word_idx[r]; rows from *t_dev (the packed token count) on do not exist.  The padded
  // [B,S,H] tensor is then never written nor read again by a pack step.
  if (word_idx != nullptr) {
    const int t = __ldg(t_dev);
    rows = t < rows ? t : rows;
  }
  for (int row = blockIdx.x * kEmbWarps + warp; row < rows; row += gridDim.x * kEmbWarps) {
    const int src = word_idx != nullptr ? __ldg(word_idx + row) : row;
    // ids outside their table are clamped (the tables are the caller's; no fault on bad input)
    int tok = __ldg(token_ids + src);
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    int pos = position_ids != nullptr ? __ldg(position_ids + src) : src % seq_len;
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    int typ = type_ids != nullptr ? __ldg(type_ids + src) : 0;
    typ = typ < 0 ? 0 : (typ >= n_types ? n_types - 1 : typ);
    const uint4* w4 = reinterpret_cast<const uint4*>(word_emb + static_cast<size_t>(tok) * hidden);
    const uint4* p4 = reinterpret_cast<const uint4*>(pos_emb + static_cast<size_t>(pos) * hidden);
    const uint4* t4 = reinterpret_cast<const uint4*>(type_emb + static_cast<size_t>(typ) * hidden);
    float v[NVEC][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        const uint4 a = __ldg(w4 + vi), b = __ldg(p4 + vi), c = __ldg(t4 + vi);
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        const __half2* bh = reinterpret_cast<const __half2*>(&b);
        const __half2* ch = reinterpret_cast<const __half2*>(&c);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __half22float2(ah[j]), fb = __half22float2(bh[j]), fc = __half22float2(ch[j]);
          v[i][2 * j] = fa.x + fb.x + fc.x;
          v[i][2 * j + 1] = fa.y + fb.y + fc.y;
          sum += v[i][2 * j] + v[i][2 * j + 1];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum * inv_h;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      if (i * 32 + lane < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[i][j] - mean;
          sq = fmaf(d, d, sq);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq * inv_h + eps);
    uint4* o4 = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * hidden);
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        float g[8], bt_[8];
        if (GB_FP32) {
          const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * vi);
          const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * vi + 1);
          const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * vi);
          const float4 b1 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * vi + 1);
          g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
          bt_[0] = b0.x; bt_[1] = b0.y; bt_[2] = b0.z; bt_[3] = b0.w; bt_[4] = b1.x; bt_[5] = b1.y; bt_[6] = b1.z; bt_[7] = b1.w;
        } else {
          const uint4 g4 = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
          const uint4 b4 = __ldg(reinterpret_cast<const uint4*>(beta) + vi);
          const __half2* gh = reinterpret_cast<const __half2*>(&g4);
          const __half2* bh = reinterpret_cast<const __half2*>(&b4);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 fg = __half22float2(gh[j]), fb = __half22float2(bh[j]);
            g[2 * j] = fg.x; g[2 * j + 1] = fg.y;
            bt_[2 * j] = fb.x; bt_[2 * j + 1] = fb.y;
          }
        }
        uint4 o;
        o.x = pack_half2(fmaf((v[i][0] - mean) * rstd, g[0], bt_[0]), fmaf((v[i][1] - mean) * rstd, g[1], bt_[1]));
        o.y = pack_half2(fmaf((v[i][2] - mean) * rstd, g[2], bt_[2]), fmaf((v[i][3] - mean) * rstd, g[3], bt_[3]));
        o.z = pack_half2(fmaf((v[i][4] - mean) * rstd, g[4], bt_[4]), fmaf((v[i][5] - mean) * rstd, g[5], bt_[5]));
        o.w = pack_half2(fmaf((v[i][6] - mean) * rstd, g[6], bt_[6]), fmaf((v[i][7] - mean) * rstd, g[7], bt_[7]));
        o4[vi] = o;
      }
    }
  }
}

// pooled[b, n] = tanh(sum_k y[b, 0, k] * W[k, n] + bias[n]).  CTA = (64 output columns, one sequence),
// 256 threads: thread (kg, cp) sums every 8th k (k = kg mod 8) for the column pair cp, so a warp reads
// one 128-byte line of W per k and up to 32 loads are in flight per thread; the eight groups meet in shared
// memory.  The work is tiny (B x H x H): what matters is that no thread walks a long chain of loads.
__global__ void __launch_bounds__(256)
pooler_kernel(const __half* __restrict__ y, const __half* __restrict__ W, const __half* __restrict__ bias,
              __half* __restrict__ pooled, int seq_len, int hidden) {
  extern __shared__ float xs[];  // hidden floats: the first token's row, then 8 x 64 partial sums
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  const int n0 = blockIdx.x * 64;
  const __half* row = y + static_cast<size_t>(b) * seq_len * hidden;
  for (int k = threadIdx.x; k < hidden; k += blockDim.x) xs[k] = __half2float(__ldg(row + k));
  __syncthreads();
  const int cp = threadIdx.x & 31;   // column pair
  const int kg = threadIdx.x >> 5;   // k group (the warp)
  const int n = n0 + 2 * cp;
  float acc0 = 0.f, acc1 = 0.f;
  if (n + 1 < hidden) {  // hidden is even (checked by the launcher)
    const __half2* wp = reinterpret_cast<const __half2*>(W + n);
    const size_t ld2 = static_cast<size_t>(hidden) / 2;  // row stride in half2
#pragma unroll 32
    for (int k = kg; k < hidden; k += 8) {
      const float2 w = __half22float2(__ldg(wp + static_cast<size_t>(k) * ld2));
      acc0 = fmaf(xs[k], w.x, acc0);
      acc1 = fmaf(xs[k], w.y, acc1);
    }
  }
  float* part = xs + hidden;
  part[kg * 64 + 2 * cp] = acc0;
  part[kg * 64 + 2 * cp + 1] = acc1;
  __syncthreads();
  const int c = threadIdx.x;
  if (c < 64 && n0 + c < hidden) {
    float sum = __half2float(__ldg(bias + n0 + c));
#pragma unroll
    for (int g = 0; g < 8; ++g) sum += part[g * 64 + c];
    pooled[static_cast<size_t>(b) * hidden + n0 + c] = __float2half(tanhf(sum));
  }
}

template <bool GB_FP32>
cudaError_t launch_emb(int nvec_per_lane, dim3 grid, cudaStream_t stream, const __half* word_emb, const __half* pos_emb,
                       const __half* type_emb, const void* gamma, const void* beta, const int* token_ids,
                       const int* type_ids, const int* position_ids, __half* out, int rows, int seq_len, int hidden,
                       int vocab, int max_pos, int n_types, float eps, const int* word_idx, const int* t_dev) {
  dim3 block(kEmbWarps * 32);
  switch (nvec_per_lane) {
    case 1: return launch_pdl(embedding_layernorm_kernel<GB_FP32, 1>, grid, block, 0, stream, word_emb, pos_emb, type_emb, gamma, beta, token_ids, type_ids, position_ids, out, rows, seq_len, hidden, vocab, max_pos, n_types, eps, word_idx, t_dev);
    case 2: return launch_pdl(embedding_layernorm_kernel<GB_FP32, 2>, grid, block, 0, stream, word_emb, pos_emb, type_emb, gamma, beta, token_ids, type_ids, position_ids, out, rows, seq_len, hidden, vocab, max_pos, n_types, eps, word_idx, t_dev);
    case 3: return launch_pdl(embedding_layernorm_kernel<GB_FP32, 3>, grid, block, 0, stream, word_emb, pos_emb, type_emb, gamma, beta, token_ids, type_ids, position_ids, out, rows, seq_len, hidden, vocab, max_pos, n_types, eps, word_idx, t_dev);
    case 4: return launch_pdl(embedding_layernorm_kernel<GB_FP32, 4>, grid, block, 0, stream, word_emb, pos_emb, type_emb, gamma, beta, token_ids, type_ids, position_ids, out, rows, seq_len, hidden, vocab, max_pos, n_types, eps, word_idx, t_dev);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_embedding_layernorm(const __half* word_emb, const __half* pos_emb, const __half* type_emb,
                                       const void* gamma, const void* beta, bool gb_fp32, const int* token_ids,
                                       const int* type_ids, const int* position_ids, __half* out, int rows, int seq_len,
                                       int hidden, int vocab, int max_pos, int n_types, float eps, cudaStream_t stream,
                                       const int* word_idx, const int* t_dev) {
  if (rows <= 0 || hidden <= 0 || hidden % 8 != 0 || hidden > 1024 || seq_len <= 0) return cudaErrorInvalidValue;
  if ((word_idx == nullptr) != (t_dev == nullptr)) return cudaErrorInvalidValue;
  const int nvec_per_lane = (hidden / 8 + 31) / 32;
  long long g = (static_cast<long long>(rows) + kEmbWarps - 1) / kEmbWarps;
  if (g > 148 * 16) g = 148 * 16;
  dim3 grid(static_cast<unsigned>(g));
  return gb_fp32 ? launch_emb<true>(nvec_per_lane, grid, stream, word_emb, pos_emb, type_emb, gamma, beta, token_ids, type_ids, position_ids, out, rows, seq_len, hidden, vocab, max_pos, n_types, eps, word_idx, t_dev)
                 : launch_emb<false>(nvec_per_lane, grid, stream, word_emb, pos_emb, type_emb, gamma, beta, token_ids, type_ids, position_ids, out, rows, seq_len, hidden, vocab, max_pos, n_types, eps, word_idx, t_dev);
}

cudaError_t launch_pooler(const __half* y, const __half* W, const __half* bias, __half* pooled, int B, int seq_len,
                          int hidden, cudaStream_t stream) {
  if (B <= 0 || B > 65535 || seq_len <= 0 || hidden <= 0 || hidden > 8192 || hidden % 2 != 0) return cudaErrorInvalidValue;
  dim3 grid((hidden + 63) / 64, B);
  const size_t smem = (static_cast<size_t>(hidden) + 512) * sizeof(float);
  return launch_pdl(pooler_kernel, grid, dim3(256), smem, stream, y, W, bias, pooled, seq_len, hidden);
}

}  // namespace bt
