// Host-side launchers of the sm_100a kernels (internal to the library; the
// public surface is the C ABI in include/bt_b200.h).  Every launcher enqueues on
// `stream` and returns the cudaError_t of the launch; none synchronises.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

namespace bt {

// Launch with the programmatic-stream-serialization attribute (see pdl_wait() in
// common.cuh); `pdl_enabled()` can be switched off for A/B measurements.
bool pdl_enabled();
void set_pdl_enabled(bool on);
// The calling thread's next launch is serialised the ordinary way (it starts when everything before it
// on the stream has completed and is visible).  The entry points whose GEMMs read their weights ahead
// of `griddepcontrol.wait` ask for this for their first kernel: a later kernel of the call can only start
// once that one has, so nothing a caller's own kernel wrote before the call (the weights, say) can still
// be in flight when a weight block is requested early.
void pdl_next_launch_plain();
bool pdl_take_attr();  // whether the launch being made gets the attribute (consumes a pending request)
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_take_attr() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

// ---- tensor maps -----------------------------------------------------------
// Encodes a 2-D fp16 (elem_bytes 2) or fp32 (elem_bytes 4) row-major tensor [rows, cols] (row stride `ld` elements)
// with a {box_cols, box_rows} box and 128-byte swizzle.  Returns false when the
// driver entry point is unavailable or the encode fails.
bool make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t box_cols, uint32_t box_rows, int elem_bytes = 2);

// ---- offsets / pack / restore ----------------------------------------------
cudaError_t launch_build_offsets(const __half* mask, int B, int S, int* batch_idx, int* word_idx,
                                 cudaStream_t stream);
cudaError_t launch_pack_rows(const __half* padded, __half* packed, const int* batch_idx, int B, int S,
                             int hidden, cudaStream_t stream);
// batch_idx[i] = i * S for i = 0..B (every sequence keeps all S rows: the general-mask path)
// (`clear_flag`: a word the kernel also sets to zero, or null)
cudaError_t launch_uniform_offsets(int* batch_idx, int B, int S, cudaStream_t stream, int* clear_flag = nullptr);
// One bit per (query, key) of a [B,S,S] mask: bit k of word k/32 of row (b*S + q) is set iff mask[b,q,k] == 1;
// a row's words are mask_bits_stride_words(S) apart.  *flag_dev (zero beforehand) becomes 1 if some entry
// is neither 0 nor 1, in which case the bits do not stand for the mask.
int mask_bits_stride_words(int S);
cudaError_t launch_mask_bits(const __half* mask, int B, int S, uint32_t* bits, int* flag_dev, cudaStream_t stream);
// *flag_dev = 1 if every mask[b] is a right-padding mask (exactly the first len_b keys allowed in each of
// the first len_b rows, no key from len_b on allowed in any later row; len_b = number of entries >= 0.5
// in row 0), else 0.
cudaError_t launch_mask_is_right_padded(const __half* mask, int B, int S, int* flag_dev, cudaStream_t stream);
// bound_dev[b * ceil(S/128) + t] = number of leading keys that query tile t of sequence b needs (see offsets.cu)
cudaError_t launch_mask_key_bound(const __half* mask, int B, int S, int* bound_dev, cudaStream_t stream);
cudaError_t launch_restore_rows(const __half* packed, __half* padded, const int* batch_idx, int B, int S,
                                int hidden, cudaStream_t stream);

// ---- GEMM ---------------------------------------------------------------------
// Epilogue of the split-K form of BT_EPI_BIAS_RESIDUAL_F32OUT (internal: chosen through GemmLaunch::split_k).
constexpr int kEpiSplitKF32 = 64;
// Ranges to cut K into for an fp32-sum GEMM of `m_rows` x N over K; 1 = no split.
int gemm_pick_split_k(int m_rows, int N, int K, int num_sms);
struct GemmLaunch {
  CUtensorMap tm_a;  // A [m_rows, K], box {64, 128}
  CUtensorMap tm_b;  // W [K, N],     box {64, 64}
  CUtensorMap tm_out;  // out [m_rows, N]: fp16 box {64, 32} or fp32 box {32, 32} (128-byte rows)
  __half* out;
  const __half* bias;
  const __half* residual;
  const int* m_dev;  // device int with the number of valid rows, or null
  int m_rows;        // rows allocated in A / out / residual (upper bound of M)
  int N;
  int K;
  // fused LayerNorm (BT_EPI_BIAS_RESIDUAL_LAYERNORM): `out` is a scratch of 16 * N/128 bytes per row for the
  // tagged row-statistics partials (zeroed once by the caller), `ln_epoch` >= 1 the tag of this launch,
  // different from that of every earlier launch on the same scratch since it was zeroed
  __half* out_ln = nullptr;
  uint32_t ln_epoch = 0;
  CUtensorMap tm_res;  // residual [m_rows, N] fp16, box {64, 32} (fused LayerNorm only)
  const void* gamma = nullptr;
  const void* beta = nullptr;
  bool gb_fp32 = false;
  float eps = 1e-6f;
  int epilogue;      // BT_EPI_*
  int gelu_kind;     // BT_GELU_*
  int block_n;       // 64, 128 or 256; 0 = choose from the shape
  // BT_EPI_BIAS_RESIDUAL_F32OUT only: > 1 cuts K into that many ranges, each handled by its own CTA
  // (few rows, long K: more SMs stream the weights).  Range s writes an fp32 partial sum to
  // out + s * m_rows * N floats, range 0 with bias and residual; the consumer adds the ranges up.
  int split_k = 1;
  int* status;       // device status word
  int num_sms;
};
int gemm_pick_block_n(int m_rows, int N, int num_sms);
cudaError_t launch_gemm(const GemmLaunch& g, cudaStream_t stream);

// ---- fused multi-head attention -----------------------------------------------
struct MhaLaunch {
  CUtensorMap tm_qkv;  // qkv [rows, 3H], box {64, 128}
  CUtensorMap tm_ctx;  // ctx [rows, H], box {64, 32}: bulk stores of whole 32-row output slabs (has_tm_ctx)
  bool has_tm_ctx = false;
  __half* ctx;         // [rows, H]
  const int* batch_idx;
  int batch;
  int max_len;         // upper bound of every sequence length
  int rows = 0;        // rows allocated in qkv / ctx
  int head_num;
  int hidden;          // H = head_num * 64
  float scale_log2e;   // log2(e) / sqrt(64) / tao
  int* status;
  // general-mask variant: all sequences have max_len rows, scores get bias - 10000 * (1 - mask) added
  const __half* gen_mask = nullptr;  // [batch, max_len, max_len], null = lengths from batch_idx only
  const __half* gen_bias = nullptr;  // [head_num, max_len, max_len] or null
  float gen_inv_scale = 8.0f;        // sqrt(64) * tao
  const int* gen_kv_bound = nullptr; // [batch, ceil(max_len/128)] keys that matter per query tile (launch_mask_key_bound) or null
  // the mask as bits (launch_mask_bits) and the word that says whether they may be used (0 = yes); null = no bits
  const uint32_t* gen_bits = nullptr;
  const int* gen_bits_flag = nullptr;
};
cudaError_t launch_mha(const MhaLaunch& a, cudaStream_t stream);

// ---- element-wise / normalisation -------------------------------------------
// An fp32 input may arrive as `n` partial sums `stride` floats apart (the K ranges of a split-K GEMM).
struct LnSplit {
  int n = 1;
  long long stride = 0;
};
cudaError_t launch_layernorm(const void* x, bool x_fp32, const __half* bias, const __half* residual, const void* gamma,
                             const void* beta, bool gb_fp32, __half* out, const int* m_dev, int m_rows,
                             int hidden, float eps, cudaStream_t stream, LnSplit split = LnSplit());
cudaError_t launch_layernorm_restore(const void* x, bool x_fp32, const __half* bias, const __half* residual,
                                     const void* gamma, const void* beta, bool gb_fp32, __half* out_padded,
                                     const int* batch_idx, int B, int S, int hidden, float eps,
                                     cudaStream_t stream, LnSplit split = LnSplit());
cudaError_t launch_add_bias_gelu(__half* x, const __half* bias, const int* m_dev, int m_rows, int n,
                                 int gelu_kind, cudaStream_t stream);
cudaError_t launch_masked_softmax(__half* logits, const __half* mask, int B, int nh, int S, float scale,
                                  cudaStream_t stream);

// Address of the per-device status word (a __device__ variable of the library).
int* device_status_word();

// ---- embedding front end / pooler back end -------------------------------------
// out[row,:] = LayerNorm(word[token] + pos[position] + type[type]) * gamma + beta; position = row % seq_len
// when position_ids is null, type 0 when type_ids is null; ids are clamped into their tables.
// With `word_idx` / `t_dev` (both or neither): packed output - row r is the r-th valid token, its ids at
// padded position word_idx[r], rows from *t_dev on are not written.
cudaError_t launch_embedding_layernorm(const __half* word_emb, const __half* pos_emb, const __half* type_emb,
                                       const void* gamma, const void* beta, bool gb_fp32, const int* token_ids,
                                       const int* type_ids, const int* position_ids, __half* out, int rows, int seq_len,
                                       int hidden, int vocab, int max_pos, int n_types, float eps, cudaStream_t stream,
                                       const int* word_idx = nullptr, const int* t_dev = nullptr);
// pooled[b,:] = tanh(y[b,0,:] * W + bias), W [hidden, hidden] row-major [in,out]
cudaError_t launch_pooler(const __half* y, const __half* W, const __half* bias, __half* pooled, int B, int seq_len,
                          int hidden, cudaStream_t stream);

// ---- self-test --------------------------------------------------------------
// One CTA waits (bounded by max_cycles, clamped to [2^10, 2^31]) on a barrier nothing arrives on;
// writes kStatusSelfTestTimeout to *status and 1 to *gave_up (device int, may be null).
cudaError_t launch_bounded_wait_selftest(int* status, long long max_cycles, int* gave_up, cudaStream_t stream);

}  // namespace bt
