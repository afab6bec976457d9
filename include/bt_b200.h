/*
 * bt_b200 — C ABI of the B200 (sm_100a) padding-free BERT encoder library.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an
 * int status (0 = BT_OK) and never throws, exits or synchronises the host.  All
 * data pointers are DEVICE pointers owned by the caller; `stream` is a
 * `cudaStream_t` passed as `void*`.  The library allocates no device memory:
 * scratch is the caller's `workspace` (size from bt_workspace_bytes()).
 *
 * Concurrency: a handle may be used by one host thread at a time (it caches tensor maps and
 * counts launches); different handles may be used from different threads and streams at once.
 * Calls on one handle are ordered by the stream they are given; a handle's kernels on two
 * streams at once must not share a workspace.  The first kernel of every forward call is
 * serialised behind all earlier work of its stream the ordinary way; the others use programmatic
 * dependent launch among themselves.
 *
 * Device: a handle belongs to the device it was created for (bt_config.device), and that device must
 * be the calling thread's current CUDA device in every call that takes the handle: the library does
 * not switch devices.  A call made with another device current returns BT_ERR_INVALID_ARG
 * ("handle belongs to device X, current device is Y") before anything is launched.  Data pointers
 * that the kernels read by tensor map or 16-byte accesses (activations, weights, masks, workspace)
 * must be 16-byte aligned; a misaligned one is refused with BT_ERR_INVALID_ARG.
 *
 * Symbols named bt_debug_* (and bt_profile_*) are not part of this interface: they exist for the
 * repository's own tests and timing scripts, set PROCESS-WIDE state that every handle of the process
 * sees (kernel selection, tile shapes), are not thread-safe and may change or vanish.  A production
 * host never calls them; bt_version() reports the library build.
 *
 * Each declaration names the reference interface it stands in for
 * (paths relative to the ByteTransformer project root).
 *
 * Data layout conventions (identical to the reference):
 *   - fp16 everywhere (`__half`), GEMM weights row-major [in_features, out_features]
 *   - qkv_kernel [H,3H] with column thirds Q|K|V, head h = columns h*64..h*64+63 of a third
 *   - padded activations [B,S,H]; packed activations [T,H], T = number of valid tokens
 *   - attention mask [B,S,S] fp16, 1 = attend, 0 = masked, right padded
 *   - batch_idx int32[B+1] (exclusive prefix sum of lengths, batch_idx[B] = T),
 *     word_idx int32[T] (packed row -> padded row b*S+i)
 */
#ifndef BT_B200_H_
#define BT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define BT_OK 0
#define BT_ERR_INVALID_ARG 1   /* null pointer, bad shape, unsupported size       */
#define BT_ERR_WORKSPACE 2     /* workspace too small                             */
#define BT_ERR_CUDA 3          /* a CUDA runtime / driver call failed             */
#define BT_ERR_UNSUPPORTED 4   /* e.g. head size != 64, device is not sm_100      */
#define BT_ERR_DEVICE_STATUS 5 /* a kernel reported a bounded-wait / bounds error */

#define BT_GELU_ERF 0  /* exact GELU: what the reference's PyTorch encoder computes */
#define BT_GELU_TANH 1 /* tanh approximation: what the reference's CUDA kernels compute */

/* epilogue selector of bt_gemm() */
#define BT_EPI_NONE 0          /* out = A*W                         */
#define BT_EPI_BIAS 1          /* out = A*W + bias                  */
#define BT_EPI_BIAS_GELU 2     /* out = gelu(A*W + bias)            */
#define BT_EPI_BIAS_RESIDUAL 3 /* out = A*W + bias + residual       */
#define BT_EPI_BIAS_RESIDUAL_F32OUT 4 /* same, but `out` is float[M,N]: the pre-LayerNorm sum keeps fp32 */
#define BT_EPI_BIAS_RESIDUAL_LAYERNORM 5 /* LN(A*W + bias + residual): only through bt_gemm_layernorm() */

typedef struct bt_encoder_s* bt_handle;

/* Replaces the constructor arguments of `BertTransformer<OpType>`
 * (bytetransformer/include/bert_transformer.h:120-131) and the numeric
 * constants the reference hard-codes in its kernels. */
typedef struct {
  int head_num;
  int size_per_head;   /* must be 64 (as for every fused path of the reference) */
  int max_batch_size;
  int max_seq_len;     /* <= 1024, as th_op/util.h:40 */
  int intermediate_mult; /* FFN width = mult * hidden; the reference fixes 4 (bert_transformer.h:74) */
  float ln_eps;        /* reference kernels: 1e-6 (layernorm.h:133) */
  int gelu_kind;       /* BT_GELU_ERF or BT_GELU_TANH */
  float tao;           /* softmax temperature (attention.h:33-39); 1.0 = standard */
  int gamma_beta_fp32; /* LayerNorm gamma/beta are float (1) or half (0): `use_fp32` of the reference */
  int device;          /* CUDA device ordinal; -1 = current device */
} bt_config;

/* Replaces `BertTransformerParam<OpType>` + `AttentionParam::attr_bias_QKV`
 * (bert_transformer.h:31-82, attention.h:25-39): the 12 weight tensors of one layer. */
typedef struct {
  const void* qkv_kernel;                  /* [H,3H] half */
  const void* qkv_bias;                    /* [3H]   half */
  const void* attr_output_kernel;          /* [H,H]  half */
  const void* attr_output_bias;            /* [H]    half */
  const void* attr_output_layernorm_gamma; /* [H] half or float */
  const void* attr_output_layernorm_beta;  /* [H] half or float */
  const void* inter_kernel;                /* [H,4H] half */
  const void* inter_bias;                  /* [4H]   half */
  const void* output_kernel;               /* [4H,H] half */
  const void* output_bias;                 /* [H]    half */
  const void* output_layernorm_gamma;      /* [H] half or float */
  const void* output_layernorm_beta;       /* [H] half or float */
} bt_layer_weights;

/* ---- object life cycle -------------------------------------------------- */

/* `new BertTransformer<HALF>(max_batch, heads, 64, max_seq, ...)`
 * (bert_transformer.h:120-185).  Host-only; fails with BT_ERR_UNSUPPORTED on a
 * device that is not compute capability 10.x. */
int bt_create(const bt_config* cfg, bt_handle* out);
int bt_destroy(bt_handle h);

/* `BertTransformer::initialize(param)` (bert_transformer.h:187-191), for layer
 * `layer` of a stack (the reference object holds one layer).  Stores raw
 * pointers only. */
int bt_set_layer_weights(bt_handle h, int layer, const bt_layer_weights* w);

/* `BertTransformer::cal_bufsize()` (bert_transformer.h:193-213). */
int bt_workspace_bytes(bt_handle h, int batch_size, int seq_len, size_t* bytes);

/* Human-readable text of the last host-side error of this handle. */
const char* bt_last_error(bt_handle h);
/* Reads (and clears) the device status word that kernels write when a bounded
 * wait ran out.  Synchronises `stream`.  0 = no device-side error. */
int bt_device_status(bt_handle h, void* stream, int* status);

#define BT_STATUS_SELFTEST_TIMEOUT 0x7F1
/* Self-test of the failure path (no counterpart in the reference, whose kernels have no
 * device-side waits): enqueues a one-CTA kernel that waits, with the same bounded wait as
 * every pipeline of the library, on a barrier that nothing arrives on.  After about
 * `max_cycles` SM cycles (clamped to [2^10, 2^31]) the wait gives up, the kernel writes
 * BT_STATUS_SELFTEST_TIMEOUT to the status word (read it with bt_device_status) and 1 to
 * `*gave_up_dev` (device int, may be NULL) and returns normally; the CUDA context stays
 * usable.  Nothing faults or traps. */
int bt_selftest_bounded_wait(bt_handle h, long long max_cycles, int* gave_up_dev, void* stream);

/* ---- forward passes ----------------------------------------------------- */

/* `BertTransformer::infer(param)` (bert_transformer.h:215-222 ->
 * src/bert_transformer.cu:28-130): one encoder layer on a padded batch;
 * padding rows of `out` are written as zeros.  `input` and `out` must not alias. */
int bt_layer_forward_padded(bt_handle h, int layer, const void* input /*[B,S,H]*/,
                            const void* attr_mask /*[B,S,S]*/, void* out /*[B,S,H]*/,
                            void* workspace, size_t workspace_bytes, int batch_size, int seq_len,
                            void* stream);

/* No counterpart in the reference.  Same result as bt_layer_forward_padded(), for
 * callers that have no workspace to hand over and may not allocate one: code that
 * runs inside another framework's execution callback, under a memory plan that was
 * fixed beforehand, or in a process whose device-memory budget is frozen once it
 * is serving.  The scratch is an array of BT_STATIC_SCRATCH_BYTES built into the
 * library's device image (each GPU that loads the library holds it until the
 * process ends), so the call performs no cudaMalloc / cudaFree and uses no
 * allocating helper.
 *   - Limit: bt_workspace_bytes(batch_size, seq_len) must not exceed
 *     BT_STATIC_SCRATCH_BYTES (hidden 768: batch_size*seq_len <= 2400 tokens,
 *     hidden 1024: <= 1800); larger shapes return BT_ERR_WORKSPACE and run nothing.
 *   - The first call on a device looks the array's device address up
 *     (cudaGetSymbolAddress); make that first call outside any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels may
 *     overlap on the GPU (different streams) race on it; serialise them.  The array
 *     keeps the previous call's bytes; nothing in it has to start at zero, every
 *     region is written by this call before it is read. */
#define BT_STATIC_SCRATCH_BYTES (48u * 1024u * 1024u)
int bt_layer_forward_padded_static(bt_handle h, int layer, const void* input /*[B,S,H]*/,
                                   const void* attr_mask /*[B,S,S]*/, void* out /*[B,S,H]*/,
                                   int batch_size, int seq_len, void* stream);

/* The reference's `for layer in range(n_layers)` loop
 * (unit_test/python_scripts/bert_transformer_test.py:191-200) as ONE call:
 * offsets + pack once, `n_layers` layers on the packed batch, one scatter. */
int bt_stack_forward_padded(bt_handle h, int n_layers, const void* input, const void* attr_mask,
                            void* out, void* workspace, size_t workspace_bytes, int batch_size,
                            int seq_len, void* stream);

/* The reference's padded / unfused attention semantics (`is_remove_padding = false`,
 * `attention_bias`): nothing is packed, every one of the batch_size*seq_len output rows is
 * computed, and the score of (query q, key k) of sequence b and head h is
 *   q.k * scale + attention_bias[h,q,k] + (1 - attr_mask[b,q,k]) * -10000
 * before the softmax (bytetransformer/include/softmax.h:41-45,
 * bytetransformer/src/attention_nofused.cu:78-95, th_op/bert_transformer_ext.h:83-107).  Any
 * [B,S,S] mask is honoured element by element (prefix-LM, block-diagonal, ...), not only row 0.
 * `attention_bias` is fp16 [head_num, seq_len, seq_len] or NULL.  Workspace: bt_workspace_bytes().
 * A key whose mask value is exactly 0 contributes an exponential of 0, so key tiles behind the last
 * non-zero mask entry of a tile of 128 query rows are not computed; a query row whose mask is all
 * zero has every score shifted alike and therefore attends to ALL keys, as the formula says (this
 * assumes |attention_bias| far below 10000).
 * Rows that a right-padding mask would have dropped hold finite but meaningless values, as in
 * the reference's padded path; use bt_mask_is_right_padded() to route such masks to the packed
 * entry points instead. */
int bt_layer_forward_padded_general(bt_handle h, int layer, const void* input, const void* attr_mask,
                                    const void* attention_bias, void* out, void* workspace,
                                    size_t workspace_bytes, int batch_size, int seq_len, void* stream);
int bt_stack_forward_padded_general(bt_handle h, int n_layers, const void* input, const void* attr_mask,
                                    const void* attention_bias, void* out, void* workspace,
                                    size_t workspace_bytes, int batch_size, int seq_len, void* stream);

/* Checks on the device whether every attr_mask[b] is a right-padding mask, i.e. whether the
 * packed entry points (which, like the reference's `parallel_prefix`, look at row 0 only:
 * remove_padding.h:51-54,81-85) would honour it: with len_b = number of entries >= 0.5 in row
 * 0, each of the first len_b rows must allow exactly the first len_b keys and no later row may
 * allow a key from len_b on (so a causal mask is not taken for length 1).  `scratch_dev` is
 * one device int; `*result` (host) receives 1 or 0.  Synchronises `stream`.  The reference has
 * no such check and silently mis-packs other masks. */
int bt_mask_is_right_padded(const void* attr_mask, int batch_size, int seq_len, int* scratch_dev,
                            int* result, void* stream);

/* Same stack on an already packed batch: x_packed [T,H], cu_seqlens int32[B+1]
 * on the DEVICE (same meaning as batch_idx), `total_tokens` = T known to the
 * host (rows allocated in x_packed / out_packed), `max_len` >= every length.
 * The reference has no packed entry; its packed state lives between
 * src/bert_transformer.cu:68 and :124. */
int bt_stack_forward_packed(bt_handle h, int n_layers, const void* x_packed, const int* cu_seqlens,
                            int batch_size, int max_len, int total_tokens, void* out_packed,
                            void* workspace, size_t workspace_bytes, void* stream);
/* Workspace for bt_stack_forward_packed(). */
int bt_workspace_bytes_packed(bt_handle h, int batch_size, int total_tokens, size_t* bytes);

/* ---- the individual steps of the path (each usable on its own) ---------- */

/* `build_sequence_length_padding_offset_kernelLauncher`
 * (bytetransformer/include/remove_padding.h:88-101) without its blocking D2H
 * copy: T stays on the device in batch_idx[B]. */
int bt_build_offsets(const void* attr_mask /*[B,S,S] half*/, int batch_size, int seq_len,
                     int* batch_idx /*[B+1]*/, int* word_idx /*[B*S], first T used*/, void* stream);

/* `compressBertInput_kernelLauncher` (remove_padding.h:104-121): packed[t,:] =
 * padded[word_idx[t],:].  Rows are `hidden` halves, hidden % 8 == 0. */
int bt_pack_rows(const void* padded /*[B*S,hidden]*/, void* packed /*[T,hidden]*/,
                 const int* batch_idx, const int* word_idx, int batch_size, int seq_len, int hidden,
                 void* stream);

/* Inverse of bt_pack_rows with zero fill of padding rows (the scatter half of
 * `add_bias_input_layernorm_restore_output_kernel_launcher`, layernorm.h:430-446). */
int bt_restore_rows(const void* packed, void* padded, const int* batch_idx, int batch_size,
                    int seq_len, int hidden, void* stream);

/* `dense_layer_kernel_launcher` (bytetransformer/src/gemm.cu:32-39) and
 * `gemm_bias_gelu` (src/gemm_bias_act.cu:76-148): out[M,N] = epi(A[M,K] * W[K,N]).
 * A row-major with row stride K, W row-major [K,N], out/residual row stride N.
 * The number of valid rows is min(*m_dev, m_rows) when m_dev != NULL (device
 * int, e.g. batch_idx + B), else m_rows; A/out/residual must have m_rows rows
 * allocated.  K % 64 == 0 and N % 64 == 0.  fp32 accumulation in tensor memory. */
int bt_gemm(bt_handle h, const void* A, const void* W, void* out, const void* bias,
            const void* residual, const int* m_dev, int m_rows, int N, int K, int epilogue,
            int gelu_kind, void* stream);

/* The attention-output / FFN-output step as ONE kernel: `dense_layer_kernel_launcher`
 * followed by `add_bias_input_layernorm_kernel_launcher`
 * (bytetransformer/src/bert_transformer.cu:102-109 and :115-129):
 * out[M,N] = LayerNorm(A[M,K] * W[K,N] + bias + residual) * gamma + beta.
 * The pre-normalisation sums stay in tensor memory; the N/256 CTAs that share a 128-row tile
 * exchange row statistics through `scratch_f32`, a device buffer of m_rows*N*4 bytes whose
 * contents are undefined afterwards (used: 16*N/128 bytes per row, which this call zeroes
 * itself with a memset on `stream`).  N % 256 == 0, N <= 1024, K % 64 == 0.  The waits
 * between CTAs are bounded like every other wait (bt_device_status). */
int bt_gemm_layernorm(bt_handle h, const void* A, const void* W, const void* bias, const void* residual,
                      const void* gamma, const void* beta, int gamma_beta_fp32, float eps,
                      void* scratch_f32, void* out, const int* m_dev, int m_rows, int N, int K,
                      void* stream);

/* `Attention<HALF>::infer` (bytetransformer/include/attention.h:124-139; packed
 * kernels src/attention_fused.cu:295-414, src/attention_fused_long.cu:171-312):
 * ctx[T,H] = per sequence, per head softmax(Q K^T / sqrt(64) / tao) V over the
 * sequence's own valid tokens.  qkv [rows,3H] already holds Q|K|V + bias. */
int bt_attention(bt_handle h, const void* qkv, void* ctx, const int* batch_idx, int batch_size,
                 int max_len, int rows_allocated, void* stream);

/* `add_bias_input_layernorm_kernel_launcher` (layernorm.h:410-428):
 * out = LN(x + bias + residual) * gamma + beta over rows [0, min(*m_dev, m_rows)).
 * bias and residual may be NULL (treated as zero).  x is half[rows,hidden], or
 * float[rows,hidden] when x_fp32 != 0 (the output of a BT_EPI_BIAS_RESIDUAL_F32OUT
 * GEMM).  hidden % 8 == 0, <= 1024. */
int bt_add_bias_residual_layernorm(const void* x, int x_fp32, const void* bias, const void* residual,
                                   const void* gamma, const void* beta, int gamma_beta_fp32,
                                   void* out, const int* m_dev, int m_rows, int hidden, float eps,
                                   void* stream);

/* `add_bias_input_layernorm_restore_output_kernel_launcher` (layernorm.h:430-446):
 * same LayerNorm, but row (b,i) of the padded output takes packed row
 * batch_idx[b]+i, and rows i >= len_b are written as zeros. */
int bt_add_bias_residual_layernorm_restore(const void* x, int x_fp32, const void* bias, const void* residual,
                                           const void* gamma, const void* beta,
                                           int gamma_beta_fp32, void* out_padded,
                                           const int* batch_idx, int batch_size, int seq_len,
                                           int hidden, float eps, void* stream);

/* `add_bias_gelu` (bytetransformer/src/gemm_bias_act.cu:32-66): x = gelu(x + bias) in place
 * over [rows, n]. */
int bt_add_bias_gelu(void* x, const void* bias, const int* m_dev, int m_rows, int n, int gelu_kind,
                     void* stream);

/* `softmax_kernelLauncher` (bytetransformer/include/softmax.h:318-475): in-place
 * masked softmax over logits laid out [nh,B,S,S] (softmax.h:33):
 * p = softmax(scale*x + (1-mask)*-10000) with 1/(sum+1e-6) normalisation;
 * mask [B,S,S].  The reference applies the scale in the preceding GEMM; pass 1.0
 * for identical behaviour. */
int bt_masked_softmax(void* logits, const void* attr_mask, int batch_size, int head_num, int seq_len,
                      float scale, void* stream);

/* ---- launch accounting and per-kernel timing ------------------------------ */
/* Kernel kinds of the arrays below (one slot per kind, BT_PROF_KINDS slots). */
#define BT_PROF_OFFSETS 0
#define BT_PROF_PACK 1
#define BT_PROF_GEMM_QKV 2
#define BT_PROF_MHA 3
#define BT_PROF_GEMM_ATTN_OUT 4
#define BT_PROF_LAYERNORM 5
#define BT_PROF_GEMM_FFN1 6
#define BT_PROF_GEMM_FFN2 7
#define BT_PROF_GEMM_OTHER 8
#define BT_PROF_KINDS 9
/* The steps either side of the encoder stack (no counterpart in the reference: its infer
 * parameters only carry unused `position_ids` / `token_type_ids`,
 * bytetransformer/include/bert_transformer.h:93-95, and an unused kernel hints at an embedding
 * LayerNorm, bytetransformer/include/layernorm.h:219-240).
 * bt_embedding_layernorm: out[b,s,:] = LayerNorm(word_emb[token_ids[b,s]] + pos_emb[p] +
 *   type_emb[type_ids[b,s]]) * gamma + beta, p = position_ids[b,s] or s when position_ids is NULL,
 *   type 0 when type_ids is NULL.  Tables fp16 row-major [vocab_size|max_positions|type_vocab_size,
 *   hidden], ids int32 [batch_size, seq_len] (ids outside a table are clamped into it), gamma/beta
 *   fp16 or fp32, out fp16 [batch_size, seq_len, hidden] = the encoder's input.  hidden % 8 == 0,
 *   hidden <= 1024; all pointers but the ids 16-byte aligned.
 * bt_pooler: pooled[b,:] = tanh(encoder_out[b,0,:] * W + bias), W fp16 [hidden, hidden] as [in,out],
 *   pooled fp16 [batch_size, hidden]; hidden even, W 4-byte aligned. */
int bt_embedding_layernorm(const void* word_emb, const void* pos_emb, const void* type_emb,
                           const void* gamma, const void* beta, int gamma_beta_fp32,
                           const int* token_ids, const int* type_ids, const int* position_ids, void* out,
                           int batch_size, int seq_len, int hidden, int vocab_size, int max_positions,
                           int type_vocab_size, float eps, void* stream);
int bt_pooler(const void* encoder_out, const void* W, const void* bias, void* pooled, int batch_size,
              int seq_len, int hidden, void* stream);

/* The embedding front end fused with packing (the fusion the reference's unused kernel hints at,
 * bytetransformer/include/layernorm.h:219-240): the tables and LayerNorm parameters of the front end,
 * fp16 tables row-major, gamma/beta fp16 or fp32 (gamma_beta_fp32), ids clamped into their tables. */
typedef struct bt_embedding_weights {
  const void* word_emb;     /* [vocab_size, hidden] */
  const void* pos_emb;      /* [max_positions, hidden] */
  const void* type_emb;     /* [type_vocab_size, hidden] */
  const void* gamma;        /* [hidden] */
  const void* beta;         /* [hidden] */
  int gamma_beta_fp32;
  int vocab_size;
  int max_positions;
  int type_vocab_size;
  float eps;
} bt_embedding_weights;
/* bt_embedding_layernorm_packed: like bt_embedding_layernorm, but writes only the valid tokens, packed:
 *   out_packed[r,:] for r < batch_idx[batch_size] is the row of the token at padded position word_idx[r]
 *   (batch_idx / word_idx as bt_build_offsets produces them; the token count stays on the device).
 *   out_packed must hold batch_size*seq_len rows at most; rows from the token count on are not written.
 * bt_stack_forward_ids: the whole model front to back in one call - offsets from attr_mask, embeddings of
 *   the valid tokens straight into the packed activation (the padded [B,S,H] input tensor never exists),
 *   n_layers encoder layers, LayerNorm + scatter into out[batch_size, seq_len, hidden] with zero padding
 *   rows.  token_ids int32 [batch_size, seq_len]; type_ids / position_ids may be NULL (type 0, position =
 *   index in the sequence).  Workspace as for bt_stack_forward_padded (bt_workspace_bytes). */
int bt_embedding_layernorm_packed(const bt_embedding_weights* emb, const int* token_ids, const int* type_ids,
                                  const int* position_ids, const int* batch_idx, const int* word_idx,
                                  void* out_packed, int batch_size, int seq_len, int hidden, void* stream);
int bt_stack_forward_ids(bt_handle h, int n_layers, const bt_embedding_weights* emb, const int* token_ids,
                         const int* type_ids, const int* position_ids, const void* attr_mask, void* out,
                         void* workspace, size_t workspace_bytes, int batch_size, int seq_len, void* stream);

/* on != 0: reset the counters and bracket every kernel the handle launches with
 * CUDA events on the launching stream; on == 0: stop timing (counting goes on).
 * Replaces the reference's unused timing events (src/bert_transformer.cu:89-93). */
int bt_profile_enable(bt_handle h, int on);
/* Waits for the recorded events and returns, per kind, the summed kernel time in
 * milliseconds and the number of launches since the last bt_profile_enable(h, 1)
 * (or since bt_create).  Both arrays have BT_PROF_KINDS entries. */
int bt_profile_read(bt_handle h, double* ms_by_kind, long long* launches_by_kind);

/* Library build information, e.g. "bt_b200 sm_100a". */
const char* bt_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BT_B200_H_ */
