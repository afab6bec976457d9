// Host side of the library: the encoder object behind the C ABI, tensor-map
// management, workspace carving and the per-layer launch sequence.
//
// Launch sequence of one layer on a packed batch x[T,H] (compare the reference's
// nine steps in bytetransformer/src/bert_transformer.cu:62-124):
//   1. qkv  = x * Wqkv + b_qkv                         GEMM, bias epilogue
//   2. ctx  = fused MHA(qkv)                           one kernel, any length
//   3. pre  = ctx * Wo + b_o + x   (fp32)              GEMM, bias+residual epilogue
//   4. y    = LN(pre)                                  row kernel
//   5. mid  = gelu(y * W1 + b_1)                       GEMM, bias+GELU epilogue
//   6. pre  = mid * W2 + b_2 + y   (fp32)              GEMM, bias+residual epilogue
//   7. out  = LN(pre)   (last layer of a padded call: LN + scatter + zero fill)
// Offsets and pack run once per call, not once per layer, and the token count T
// never travels to the host: every kernel reads it from batch_idx[B].
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "../../include/bt_b200.h"

namespace bt {

__device__ int g_status_word = 0;

static bool g_pdl_on = true;
bool pdl_enabled() { return g_pdl_on; }
void set_pdl_enabled(bool on) { g_pdl_on = on; }
static thread_local bool t_next_launch_plain = false;
void pdl_next_launch_plain() { t_next_launch_plain = true; }
bool pdl_take_attr() {
  const bool plain = t_next_launch_plain;
  t_next_launch_plain = false;
  return g_pdl_on && !plain;
}

int* device_status_word() {
  int* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word) != cudaSuccess) return nullptr;
  return p;
}

// ------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn lookup_encode_fn() {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    return reinterpret_cast<EncodeTiledFn>(p);
  return nullptr;
}
static EncodeTiledFn get_encode_fn() {
  static const EncodeTiledFn fn = lookup_encode_fn();  // initialised once, also when threads race here
  return fn;
}

bool make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                  uint32_t box_rows, int elem_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld * elem_bytes) % 16 != 0) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// --------------------------------------------------------------------- encoder
struct TmapKey {
  const void* base;
  uint64_t rows, cols;
  uint32_t box_cols, box_rows;
  int elem_bytes;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_cols == o.box_cols && box_rows == o.box_rows &&
           elem_bytes == o.elem_bytes;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.cols * 1315423911ull + (h << 6) + (h >> 2));
    h ^= ((static_cast<uint64_t>(k.box_cols) << 40) | (static_cast<uint64_t>(k.box_rows) << 8) |
          static_cast<uint64_t>(k.elem_bytes)) + (h << 6) + (h >> 2);
    return static_cast<size_t>(h);
  }
};

struct LayerState {
  bt_layer_weights w;
  bool set = false;
};

}  // namespace bt

struct bt_encoder_s {
  bt_config cfg;
  int hidden = 0;
  int ffn = 0;
  int device = 0;
  int num_sms = 148;
  int* status = nullptr;
  std::string err;
  std::vector<bt::LayerState> layers;
  // cache of encoded tensor maps (activations and weights), emptied when it has grown to kTmapCap entries
  std::unordered_map<bt::TmapKey, CUtensorMap, bt::TmapKeyHash> tmaps;
  static constexpr size_t kTmapCap = 8192;

  // launch accounting / optional per-kernel event timing (bt_profile_*)
  long long launches[BT_PROF_KINDS] = {};
  bool prof_on = false;
  // LayerNorm inside the attention-output / FFN2 GEMM kernel (bt_debug_set_fused_layernorm):
  // 0 never, 1 from `fused_ln_min_tiles` 128-row tiles (of allocated rows) upwards, 2 always.  Measured on
  // B200 (12 layers, hidden 768, batch 16 through the padded entry point, ms per forward without / with the
  // fused kernels): 32 row tiles 1.11 / 1.16, 40 tiles 1.45 / 1.28, 48 tiles 1.42 / 1.31, 64 tiles 1.54 / 1.46,
  // 80 tiles 2.08 / 1.99, 96 tiles 2.14 / 2.10; at 141-148 tiles per call the fused kernels are worth 3 % of the
  // forward.  Below ~40 tiles the exchange of row statistics between CTAs lengthens the only wave by more
  // than the saved LayerNorm launch and fp32 round trip.  (An earlier form of the kernels lost up to 65
  // tiles; the threshold stood at 100 then.)
  int fused_ln = 1;
  int fused_ln_min_tiles = 40;
  uint32_t ln_epoch = 0;  // fused LayerNorm launches since the statistics scratch of the current call was zeroed
  bool fused_ln_ffn2_only = false;  // keep the attention-output LayerNorm as its own kernel
  std::vector<cudaEvent_t> ev_pool;
  size_t ev_used = 0;
  struct Span { int kind; cudaEvent_t beg, end; };
  std::vector<Span> spans;

  cudaEvent_t take_event() {
    if (ev_used == ev_pool.size()) {
      cudaEvent_t e = nullptr;
      if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
      ev_pool.push_back(e);
    }
    return ev_pool[ev_used++];
  }

  // Copies the tensor map of a row-major [rows, cols] tensor with the given box into `*out` (a copy, so
  // that later look-ups, which may empty the cache, cannot invalidate it).
  bool tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows,
            int elem_bytes = 2) {
    bt::TmapKey k{base, rows, cols, box_cols, box_rows, elem_bytes};
    auto it = tmaps.find(k);
    if (it != tmaps.end()) {
      *out = it->second;
      return true;
    }
    if (!bt::make_tmap_2d(out, base, rows, cols, cols, box_cols, box_rows, elem_bytes)) return false;
    if (tmaps.size() >= kTmapCap) tmaps.clear();
    tmaps.emplace(k, *out);
    return true;
  }
};

namespace bt {

// Counts one launch of `kind`; with profiling on, brackets it with two events on
// the launching stream.
struct LaunchScope {
  bt_handle h;
  cudaStream_t stream;
  cudaEvent_t end = nullptr;
  int kind;
  LaunchScope(bt_handle h_, int kind_, cudaStream_t s) : h(h_), stream(s), kind(kind_) {
    if (!h) return;
    h->launches[kind]++;
    if (h->prof_on) {
      cudaEvent_t beg = h->take_event();
      end = h->take_event();
      if (beg && end) {
        cudaEventRecord(beg, stream);
        h->spans.push_back({kind, beg, end});
      } else {
        end = nullptr;
      }
    }
  }
  ~LaunchScope() {
    if (end) cudaEventRecord(end, stream);
  }
};

static int fail(bt_handle h, int code, const char* msg) {
  if (h) h->err = msg;
  return code;
}
static int fail_cuda(bt_handle h, cudaError_t e, const char* where) {
  if (h) h->err = std::string(where) + ": " + cudaGetErrorString(e);
  return BT_ERR_CUDA;
}

// A handle belongs to one device: its status word, its cached tensor maps and (for the static-scratch
// entry) the scratch array are addresses on that device, while kernels go to whichever device is current.
static int check_device(bt_handle h) {
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess) return fail(h, BT_ERR_CUDA, "cudaGetDevice failed");
  if (cur != h->device) {
    h->err = "handle belongs to device " + std::to_string(h->device) + ", current device is " + std::to_string(cur);
    return BT_ERR_INVALID_ARG;
  }
  return BT_OK;
}
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Split-K of the fp32-sum GEMMs is considered up to kSplitKMaxRows allocated rows; the partial sums of
// all ranges together take at most kSplitKRowBudget rows of `pre` (8 ranges up to 256 rows, 4 up to
// 512, 2 up to 1024).
constexpr size_t kSplitKMaxRows = 1024;
constexpr size_t kSplitKRowBudget = 2048;

struct Workspace {
  int* batch_idx;
  int* word_idx;
  __half *xa, *xb, *qkv, *ctx, *y, *mid;
  float* pre;  // pre-LayerNorm sum, kept in fp32 (LayerNorm as its own kernel), or the row-statistics partials
  size_t ln_stats_bytes;  // leading bytes of `pre` that hold the tagged row-statistics partials (fused LayerNorm)
  // general-mask path of the padded entry points: the mask as one bit per (query, key), 128 bytes per row at
  // most (S <= 1024), behind a word that says whether the bits may be used; null on the packed entry
  int* mask_bits_flag;
  uint32_t* mask_bits;
  size_t bytes;
};

// rows = allocated packed rows; n_idx = ints reserved for batch_idx/word_idx (0 for the packed entry)
static Workspace carve(void* base, size_t rows, int hidden, int ffn, size_t n_batch_idx, size_t n_word_idx) {
  Workspace w;
  uint8_t* p = reinterpret_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    uint8_t* r = p ? p + off : nullptr;
    off += align_up(bytes, 1024);
    return r;
  };
  w.batch_idx = reinterpret_cast<int*>(take(n_batch_idx * 4));
  w.word_idx = reinterpret_cast<int*>(take(n_word_idx * 4));
  w.mask_bits_flag = reinterpret_cast<int*>(take(n_word_idx ? 16 : 0));
  w.mask_bits = reinterpret_cast<uint32_t*>(take(n_word_idx * 128));
  const size_t rh = rows * static_cast<size_t>(hidden) * 2;
  w.xa = reinterpret_cast<__half*>(take(rh));
  w.xb = reinterpret_cast<__half*>(take(rh));
  w.qkv = reinterpret_cast<__half*>(take(3 * rh));
  w.ctx = reinterpret_cast<__half*>(take(rh));
  // fp32 sums; with few rows the GEMMs that produce them cut K into ranges, one sum each
  const size_t pre_rows = rows <= kSplitKMaxRows ? kSplitKRowBudget : rows;
  w.pre = reinterpret_cast<float*>(take(pre_rows * static_cast<size_t>(hidden) * 4));
  w.y = reinterpret_cast<__half*>(take(rh));
  w.mid = reinterpret_cast<__half*>(take(rows * static_cast<size_t>(ffn) * 2));
  w.ln_stats_bytes = rows * static_cast<size_t>(hidden / 128 > 0 ? hidden / 128 : 1) * 16;
  w.bytes = off + 1024;  // slack so that an unaligned base can be rounded up
  return w;
}

struct LnArgs {
  uint32_t epoch = 0;  // tag of this launch in the statistics scratch
  __half* out_ln = nullptr;
  const void* gamma = nullptr;
  const void* beta = nullptr;
  bool gb_fp32 = false;
  float eps = 1e-6f;
};

static int run_gemm(bt_handle h, int kind, const __half* A, const void* W, __half* out, const void* bias,
                    const __half* residual, const int* m_dev, int m_rows, int N, int K, int epi, int gelu_kind,
                    cudaStream_t stream, const LnArgs* ln = nullptr, int split_k = 1) {
  GemmLaunch g;
  bool ok = h->tmap(&g.tm_a, A, m_rows, K, 64, 128) && h->tmap(&g.tm_b, W, K, N, 64, 64);
  if (epi == BT_EPI_BIAS_RESIDUAL_LAYERNORM)  // `out` is only the statistics scratch; the store map is the fp16 result's
    ok = ok && ln != nullptr && h->tmap(&g.tm_out, ln->out_ln, m_rows, N, 64, 32, 2) &&
         h->tmap(&g.tm_res, residual, m_rows, N, 64, 32, 2);
  else if (epi == BT_EPI_BIAS_RESIDUAL_F32OUT)
    ok = ok && h->tmap(&g.tm_out, out, m_rows, N, 32, 32, 4);
  else
    ok = ok && h->tmap(&g.tm_out, out, m_rows, N, 64, 32, 2);
  if (!ok) return fail(h, BT_ERR_CUDA, "cuTensorMapEncodeTiled failed (pointer alignment / driver entry point)");
  g.out = out;
  g.bias = reinterpret_cast<const __half*>(bias);
  g.residual = residual;
  g.m_dev = m_dev;
  g.m_rows = m_rows;
  g.N = N;
  g.K = K;
  g.epilogue = epi;
  g.gelu_kind = gelu_kind;
  g.block_n = 0;
  g.split_k = split_k;
  g.status = h->status;
  g.num_sms = h->num_sms;
  if (ln != nullptr) {
    g.ln_epoch = ln->epoch;
    g.out_ln = ln->out_ln;
    g.gamma = ln->gamma;
    g.beta = ln->beta;
    g.gb_fp32 = ln->gb_fp32;
    g.eps = ln->eps;
  }
  cudaError_t e;
  {
    LaunchScope scope(h, kind, stream);
    e = launch_gemm(g, stream);
  }
  if (e != cudaSuccess) return fail_cuda(h, e, "gemm launch");
  return BT_OK;
}

// General-mask attention: [B,S,S] mask applied to every (query, key) pair and an optional
// [heads,S,S] additive bias (bytetransformer/include/softmax.h:41-45); null mask = lengths only.
struct GeneralMask {
  const __half* mask = nullptr;
  const __half* bias = nullptr;
  const int* kv_bound = nullptr;  // per (sequence, query tile): leading keys that matter (launch_mask_key_bound)
  const uint32_t* bits = nullptr; // the mask as bits (launch_mask_bits), or null
  const int* bits_flag = nullptr;
};

static int run_mha(bt_handle h, const __half* qkv, __half* ctx, const int* batch_idx, int B, int max_len, int rows,
                   cudaStream_t stream, const GeneralMask* gm = nullptr) {
  MhaLaunch a;
  if (!h->tmap(&a.tm_qkv, qkv, rows, 3 * static_cast<uint64_t>(h->hidden), 64, 128))
    return fail(h, BT_ERR_CUDA, "cuTensorMapEncodeTiled failed for qkv");
  a.has_tm_ctx = h->tmap(&a.tm_ctx, ctx, rows, static_cast<uint64_t>(h->hidden), 64, 32);
  a.ctx = ctx;
  a.batch_idx = batch_idx;
  a.batch = B;
  a.max_len = max_len;
  a.rows = rows;
  a.head_num = h->cfg.head_num;
  a.hidden = h->hidden;
  a.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(h->cfg.size_per_head)) / h->cfg.tao;
  a.status = h->status;
  if (gm != nullptr && gm->mask != nullptr) {
    a.gen_mask = gm->mask;
    a.gen_bias = gm->bias;
    a.gen_kv_bound = gm->kv_bound;
    a.gen_bits = gm->bits;
    a.gen_bits_flag = gm->bits_flag;
    a.gen_inv_scale = sqrtf(static_cast<float>(h->cfg.size_per_head)) * h->cfg.tao;
  }
  cudaError_t e;
  {
    LaunchScope scope(h, BT_PROF_MHA, stream);
    e = launch_mha(a, stream);
  }
  if (e != cudaSuccess) return fail_cuda(h, e, "attention launch");
  return BT_OK;
}

// LayerNorm rides in the attention-output / FFN2 GEMM kernel once there are enough 128-row tiles
// to occupy the machine with 256-column tiles; below that the narrow-tile GEMM followed by the
// row kernel spreads the few rows over more SMs.
static bool want_fused_ln(bt_handle h, long long rows) {
  const int H = h->hidden;
  const long long row_tiles = (rows + 127) / 128;
  return (H % 256 == 0) && H <= 1024 && (h->fused_ln == 2 || (h->fused_ln == 1 && row_tiles >= h->fused_ln_min_tiles));
}

// The statistics scratch of the fused LayerNorm (the head of `pre`) holds words tagged with the number
// of the launch that wrote them; it is zeroed once per call (the caller's workspace starts out with
// arbitrary contents) and the fused launches of the call are numbered from 1.
static int prepare_ln_sync(bt_handle h, const Workspace& ws, long long rows, cudaStream_t stream) {
  h->ln_epoch = 0;
  if (!want_fused_ln(h, rows)) return BT_OK;
  cudaError_t e = cudaMemsetAsync(ws.pre, 0, ws.ln_stats_bytes, stream);
  return e == cudaSuccess ? BT_OK : fail_cuda(h, e, "memset of the LayerNorm statistics scratch");
}

// One layer on packed rows.  `x_in` -> `x_out` (packed) unless restore_to != null,
// in which case the last LayerNorm scatters into the padded tensor.
static int run_layer(bt_handle h, int layer, const __half* x_in, __half* x_out, __half* restore_to,
                     const Workspace& ws, const int* batch_idx, int B, int S_or_maxlen, int rows,
                     cudaStream_t stream, const GeneralMask* gm = nullptr) {
  if (layer < 0 || layer >= static_cast<int>(h->layers.size()) || !h->layers[layer].set)
    return fail(h, BT_ERR_INVALID_ARG, "layer weights not set");
  const bt_layer_weights& w = h->layers[layer].w;
  const int H = h->hidden, F = h->ffn;
  const int* m_dev = batch_idx + B;
  const bool gb32 = h->cfg.gamma_beta_fp32 != 0;
  int rc;
  if ((rc = run_gemm(h, BT_PROF_GEMM_QKV, x_in, w.qkv_kernel, ws.qkv, w.qkv_bias, nullptr, m_dev, rows, 3 * H, H, BT_EPI_BIAS, 0,
                     stream)) != BT_OK)
    return rc;
  if ((rc = run_mha(h, ws.qkv, ws.ctx, batch_idx, B, S_or_maxlen, rows, stream, gm)) != BT_OK) return rc;
  // LayerNorm rides in the GEMM kernel (clusters of H/256 CTAs per 128-row tile) once there are
  // enough row tiles to occupy the machine that way; below that the narrow-tile GEMM followed by
  // the row kernel spreads the few rows over more SMs.
  const bool fuse_any = want_fused_ln(h, rows);
  const bool fuse_ln = fuse_any && !h->fused_ln_ffn2_only;
  // Few rows: the two GEMMs that feed a LayerNorm cut K into ranges (one fp32 sum each, `rows * H`
  // floats apart in `pre`) and the LayerNorm kernel adds them up.
  auto split_for = [&](int K) {
    if (static_cast<size_t>(rows) > kSplitKMaxRows) return 1;
    int s = gemm_pick_split_k(rows, H, K, h->num_sms);
    while (s > 1 && static_cast<size_t>(s) * static_cast<size_t>(rows) > kSplitKRowBudget) s >>= 1;
    return (s >= 1 && (K / 64) % s == 0) ? s : 1;
  };
  const int split_attn = split_for(H), split_ffn2 = split_for(F);
  const long long split_stride = static_cast<long long>(rows) * H;
  cudaError_t e = cudaSuccess;
  if (fuse_ln) {
    LnArgs ln{++h->ln_epoch, ws.y, w.attr_output_layernorm_gamma, w.attr_output_layernorm_beta, gb32, h->cfg.ln_eps};
    if ((rc = run_gemm(h, BT_PROF_GEMM_ATTN_OUT, ws.ctx, w.attr_output_kernel, reinterpret_cast<__half*>(ws.pre),
                       w.attr_output_bias, x_in, m_dev, rows, H, H, BT_EPI_BIAS_RESIDUAL_LAYERNORM, 0, stream, &ln)) !=
        BT_OK)
      return rc;
  } else {
    if ((rc = run_gemm(h, BT_PROF_GEMM_ATTN_OUT, ws.ctx, w.attr_output_kernel, reinterpret_cast<__half*>(ws.pre),
                       w.attr_output_bias, x_in, m_dev, rows, H, H, BT_EPI_BIAS_RESIDUAL_F32OUT, 0, stream, nullptr,
                       split_attn)) != BT_OK)
      return rc;
    {
      LaunchScope scope(h, BT_PROF_LAYERNORM, stream);
      e = launch_layernorm(ws.pre, true, nullptr, nullptr, w.attr_output_layernorm_gamma, w.attr_output_layernorm_beta,
                           gb32, ws.y, m_dev, rows, H, h->cfg.ln_eps, stream, LnSplit{split_attn, split_stride});
    }
    if (e != cudaSuccess) return fail_cuda(h, e, "layernorm launch");
  }
  if ((rc = run_gemm(h, BT_PROF_GEMM_FFN1, ws.y, w.inter_kernel, ws.mid, w.inter_bias, nullptr, m_dev, rows, F, H, BT_EPI_BIAS_GELU,
                     h->cfg.gelu_kind, stream)) != BT_OK)
    return rc;
  if (fuse_any && restore_to == nullptr) {
    LnArgs ln{++h->ln_epoch, x_out, w.output_layernorm_gamma, w.output_layernorm_beta, gb32, h->cfg.ln_eps};
    return run_gemm(h, BT_PROF_GEMM_FFN2, ws.mid, w.output_kernel, reinterpret_cast<__half*>(ws.pre), w.output_bias,
                    ws.y, m_dev, rows, H, F, BT_EPI_BIAS_RESIDUAL_LAYERNORM, 0, stream, &ln);
  }
  if ((rc = run_gemm(h, BT_PROF_GEMM_FFN2, ws.mid, w.output_kernel, reinterpret_cast<__half*>(ws.pre), w.output_bias,
                     ws.y, m_dev, rows, H, F, BT_EPI_BIAS_RESIDUAL_F32OUT, 0, stream, nullptr, split_ffn2)) != BT_OK)
    return rc;
  LaunchScope scope(h, BT_PROF_LAYERNORM, stream);
  if (restore_to != nullptr)
    e = launch_layernorm_restore(ws.pre, true, nullptr, nullptr, w.output_layernorm_gamma, w.output_layernorm_beta, gb32,
                                 restore_to, batch_idx, B, S_or_maxlen, H, h->cfg.ln_eps, stream,
                                 LnSplit{split_ffn2, split_stride});
  else
    e = launch_layernorm(ws.pre, true, nullptr, nullptr, w.output_layernorm_gamma, w.output_layernorm_beta, gb32, x_out,
                         m_dev, rows, H, h->cfg.ln_eps, stream, LnSplit{split_ffn2, split_stride});
  if (e != cudaSuccess) return fail_cuda(h, e, "layernorm launch");
  return BT_OK;
}

static int check_shape(bt_handle h, int B, int S) {
  if (!h) return BT_ERR_INVALID_ARG;
  if (B <= 0 || S <= 0) return fail(h, BT_ERR_INVALID_ARG, "batch_size and seq_len must be positive");
  if (S > 1024) return fail(h, BT_ERR_INVALID_ARG, "Input seq_len too long (max 1024)");
  if (B > 65535) return fail(h, BT_ERR_INVALID_ARG, "batch_size too large (max 65535)");
  return BT_OK;
}

// Where the packed activation of a padded call comes from: the padded input tensor (pack), or token ids
// through the embedding tables (the front end writes packed rows directly).
struct IdsInput {
  const bt_embedding_weights* emb;
  const int* token_ids;
  const int* type_ids;
  const int* position_ids;
};

static int check_embedding(bt_handle h, const bt_embedding_weights* e, int hidden) {
  if (!e || !e->word_emb || !e->pos_emb || !e->type_emb || !e->gamma || !e->beta)
    return fail(h, BT_ERR_INVALID_ARG, "null embedding table / LayerNorm parameter");
  if (e->vocab_size <= 0 || e->max_positions <= 0 || e->type_vocab_size <= 0 || !(e->eps >= 0.f))
    return fail(h, BT_ERR_INVALID_ARG, "bad embedding table sizes or eps");
  if (hidden <= 0 || hidden % 8 != 0 || hidden > 1024) return fail(h, BT_ERR_INVALID_ARG, "hidden must be a multiple of 8, at most 1024");
  if (!aligned16(e->word_emb) || !aligned16(e->pos_emb) || !aligned16(e->type_emb) || !aligned16(e->gamma) ||
      !aligned16(e->beta))
    return fail(h, BT_ERR_INVALID_ARG, "embedding tables and LayerNorm parameters must be 16-byte aligned");
  return BT_OK;
}

static int stack_padded(bt_handle h, int first_layer, int n_layers, const void* input, const void* mask, void* out,
                        void* workspace, size_t workspace_bytes, int B, int S, void* stream_v,
                        const IdsInput* ids = nullptr) {
  int rc = check_shape(h, B, S);
  if (rc != BT_OK) return rc;
  if ((!input && !ids) || !mask || !out || !workspace) return fail(h, BT_ERR_INVALID_ARG, "null pointer argument");
  if (input == out) return fail(h, BT_ERR_INVALID_ARG, "input and output must not alias");
  if (n_layers <= 0) return fail(h, BT_ERR_INVALID_ARG, "n_layers must be positive");
  if (!aligned16(input) || !aligned16(mask) || !aligned16(out))
    return fail(h, BT_ERR_INVALID_ARG, "input, attr_mask and output must be 16-byte aligned");
  if (ids != nullptr) {
    if (!ids->token_ids) return fail(h, BT_ERR_INVALID_ARG, "null token_ids");
    if ((rc = check_embedding(h, ids->emb, h->hidden)) != BT_OK) return rc;
  }
  if ((rc = check_device(h)) != BT_OK) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const size_t rows = static_cast<size_t>(B) * S;
  Workspace need = carve(nullptr, rows, h->hidden, h->ffn, B + 1, rows);
  if (workspace_bytes < need.bytes) return fail(h, BT_ERR_WORKSPACE, "workspace smaller than bt_workspace_bytes()");
  void* base = reinterpret_cast<void*>(align_up(reinterpret_cast<uintptr_t>(workspace), 1024));
  Workspace ws = carve(base, rows, h->hidden, h->ffn, B + 1, rows);

  if ((rc = prepare_ln_sync(h, ws, static_cast<long long>(rows), stream)) != BT_OK) return rc;
  pdl_next_launch_plain();  // first kernel of the call: see kernels.h
  cudaError_t e;
  {
    LaunchScope scope(h, BT_PROF_OFFSETS, stream);
    e = launch_build_offsets(reinterpret_cast<const __half*>(mask), B, S, ws.batch_idx, ws.word_idx, stream);
  }
  if (e != cudaSuccess) return fail_cuda(h, e, "offsets launch");
  if (ids != nullptr) {
    const bt_embedding_weights& w = *ids->emb;
    LaunchScope scope(h, BT_PROF_PACK, stream);
    e = launch_embedding_layernorm(reinterpret_cast<const __half*>(w.word_emb), reinterpret_cast<const __half*>(w.pos_emb),
                                   reinterpret_cast<const __half*>(w.type_emb), w.gamma, w.beta, w.gamma_beta_fp32 != 0,
                                   ids->token_ids, ids->type_ids, ids->position_ids, ws.xa, static_cast<int>(rows), S,
                                   h->hidden, w.vocab_size, w.max_positions, w.type_vocab_size, w.eps, stream, ws.word_idx,
                                   ws.batch_idx + B);
  } else {
    LaunchScope scope(h, BT_PROF_PACK, stream);
    e = launch_pack_rows(reinterpret_cast<const __half*>(input), ws.xa, ws.batch_idx, B, S, h->hidden, stream);
  }
  if (e != cudaSuccess) return fail_cuda(h, e, "pack launch");
  __half* cur = ws.xa;
  __half* nxt = ws.xb;
  for (int l = 0; l < n_layers; ++l) {
    const bool last = (l == n_layers - 1);
    rc = run_layer(h, first_layer + l, cur, nxt, last ? reinterpret_cast<__half*>(out) : nullptr, ws, ws.batch_idx, B,
                   S, static_cast<int>(rows), stream);
    if (rc != BT_OK) return rc;
    __half* t = cur;
    cur = nxt;
    nxt = t;
  }
  return BT_OK;
}

// The general-mask path: nothing is packed (every sequence keeps its S rows, so the padded tensor IS
// the packed tensor with offsets b*S) and the attention kernel applies the whole [B,S,S] mask and the
// optional bias.  Every output row is computed, as on the reference's padded path.
static int stack_general(bt_handle h, int first_layer, int n_layers, const void* input, const void* mask,
                         const void* attention_bias, void* out, void* workspace, size_t workspace_bytes, int B, int S,
                         void* stream_v) {
  int rc = check_shape(h, B, S);
  if (rc != BT_OK) return rc;
  if (!input || !mask || !out || !workspace) return fail(h, BT_ERR_INVALID_ARG, "null pointer argument");
  if (input == out) return fail(h, BT_ERR_INVALID_ARG, "input and output must not alias");
  if (n_layers <= 0) return fail(h, BT_ERR_INVALID_ARG, "n_layers must be positive");
  if ((reinterpret_cast<uintptr_t>(mask) & 15u) != 0 || (reinterpret_cast<uintptr_t>(attention_bias) & 15u) != 0)
    return fail(h, BT_ERR_INVALID_ARG, "mask and attention_bias must be 16-byte aligned");
  if (!aligned16(input) || !aligned16(out)) return fail(h, BT_ERR_INVALID_ARG, "input and output must be 16-byte aligned");
  if ((rc = check_device(h)) != BT_OK) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const size_t rows = static_cast<size_t>(B) * S;
  Workspace need = carve(nullptr, rows, h->hidden, h->ffn, B + 1, rows);
  if (workspace_bytes < need.bytes) return fail(h, BT_ERR_WORKSPACE, "workspace smaller than bt_workspace_bytes()");
  void* base = reinterpret_cast<void*>(align_up(reinterpret_cast<uintptr_t>(workspace), 1024));
  Workspace ws = carve(base, rows, h->hidden, h->ffn, B + 1, rows);
  if ((rc = prepare_ln_sync(h, ws, static_cast<long long>(rows), stream)) != BT_OK) return rc;
  pdl_next_launch_plain();  // first kernel of the call: see kernels.h
  cudaError_t e;
  {
    LaunchScope scope(h, BT_PROF_OFFSETS, stream);
    e = launch_uniform_offsets(ws.batch_idx, B, S, stream, ws.mask_bits_flag);
  }
  if (e != cudaSuccess) return fail_cuda(h, e, "offsets launch");
  GeneralMask gm;
  gm.mask = reinterpret_cast<const __half*>(mask);
  gm.bias = reinterpret_cast<const __half*>(attention_bias);
  // Key tiles that no row of a query tile may see are left out of the attention (once per call; the
  // packed-index region of the workspace is free on this path: B * ceil(S/128) <= B * S ints).
  {
    LaunchScope scope(h, BT_PROF_OFFSETS, stream);
    e = launch_mask_key_bound(gm.mask, B, S, ws.word_idx, stream);
  }
  if (e != cudaSuccess) return fail_cuda(h, e, "mask key-bound launch");
  gm.kv_bound = ws.word_idx;
  if (gm.bias == nullptr) {
    // no bias: a mask of zeros and ones is applied from bits (one pre-pass per call; the kernel falls back to
    // the fp16 mask if the pre-pass meets any other value)
    {
      LaunchScope scope(h, BT_PROF_OFFSETS, stream);
      e = launch_mask_bits(gm.mask, B, S, ws.mask_bits, ws.mask_bits_flag, stream);
    }
    if (e != cudaSuccess) return fail_cuda(h, e, "mask bits launch");
    gm.bits = ws.mask_bits;
    gm.bits_flag = ws.mask_bits_flag;
  }
  const __half* cur = reinterpret_cast<const __half*>(input);
  for (int l = 0; l < n_layers; ++l) {
    const bool last = (l == n_layers - 1);
    __half* dst = last ? reinterpret_cast<__half*>(out) : ((l & 1) ? ws.xb : ws.xa);
    rc = run_layer(h, first_layer + l, cur, dst, nullptr, ws, ws.batch_idx, B, S, static_cast<int>(rows), stream, &gm);
    if (rc != BT_OK) return rc;
    cur = dst;
  }
  return BT_OK;
}

}  // namespace bt

using namespace bt;

extern "C" {

// BT_SOURCE_HASH: digest of the library's sources, passed by the build (bytetransformer_b200/build.py), so
// that a binary built from other sources than the ones beside it can be told apart.
#ifndef BT_SOURCE_HASH
#define BT_SOURCE_HASH "unknown"
#endif
const char* bt_version(void) { return "bt_b200 0.2 (sm_100a, tcgen05/TMEM/TMA) src:" BT_SOURCE_HASH; }

int bt_create(const bt_config* cfg, bt_handle* out) {
  if (!cfg || !out) return BT_ERR_INVALID_ARG;
  *out = nullptr;
  if (cfg->size_per_head != 64 || cfg->head_num <= 0 || cfg->head_num > 64) return BT_ERR_UNSUPPORTED;
  if (cfg->max_seq_len <= 0 || cfg->max_seq_len > 1024 || cfg->max_batch_size <= 0) return BT_ERR_INVALID_ARG;
  if (cfg->intermediate_mult <= 0 || !(cfg->tao > 0.f) || !(cfg->ln_eps >= 0.f)) return BT_ERR_INVALID_ARG;
  if (cfg->gelu_kind != BT_GELU_ERF && cfg->gelu_kind != BT_GELU_TANH) return BT_ERR_INVALID_ARG;
  int dev = cfg->device;
  if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) return BT_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return BT_ERR_CUDA;
  if (prop.major != 10) return BT_ERR_UNSUPPORTED;  // tcgen05 / tensor memory need sm_100
  int cur = 0;
  cudaGetDevice(&cur);
  if (cur != dev && cudaSetDevice(dev) != cudaSuccess) return BT_ERR_CUDA;
  int* status = device_status_word();
  if (cur != dev) cudaSetDevice(cur);
  if (status == nullptr) return BT_ERR_CUDA;
  bt_encoder_s* h = new (std::nothrow) bt_encoder_s();
  if (!h) return BT_ERR_INVALID_ARG;
  h->cfg = *cfg;
  h->hidden = cfg->head_num * cfg->size_per_head;
  h->ffn = h->hidden * cfg->intermediate_mult;
  h->device = dev;
  h->num_sms = prop.multiProcessorCount;
  h->status = status;
  *out = h;
  return BT_OK;
}

int bt_destroy(bt_handle h) {
  if (h)
    for (cudaEvent_t e : h->ev_pool) cudaEventDestroy(e);
  delete h;
  return BT_OK;
}

int bt_set_layer_weights(bt_handle h, int layer, const bt_layer_weights* w) {
  if (!h || !w) return BT_ERR_INVALID_ARG;
  if (layer < 0 || layer >= 4096) return fail(h, BT_ERR_INVALID_ARG, "layer index out of range");
  const void* const* p = reinterpret_cast<const void* const*>(w);
  for (int i = 0; i < 12; ++i) {
    if (p[i] == nullptr) return fail(h, BT_ERR_INVALID_ARG, "null weight pointer");
    if ((reinterpret_cast<uintptr_t>(p[i]) & 15u) != 0) return fail(h, BT_ERR_INVALID_ARG, "weight pointers must be 16-byte aligned");
  }
  if (static_cast<int>(h->layers.size()) <= layer) h->layers.resize(layer + 1);
  h->layers[layer].w = *w;
  h->layers[layer].set = true;
  return BT_OK;
}

int bt_workspace_bytes(bt_handle h, int batch_size, int seq_len, size_t* bytes) {
  if (!bytes) return BT_ERR_INVALID_ARG;
  int rc = check_shape(h, batch_size, seq_len);
  if (rc != BT_OK) return rc;
  const size_t rows = static_cast<size_t>(batch_size) * seq_len;
  *bytes = carve(nullptr, rows, h->hidden, h->ffn, batch_size + 1, rows).bytes;
  return BT_OK;
}

int bt_workspace_bytes_packed(bt_handle h, int batch_size, int total_tokens, size_t* bytes) {
  if (!h || !bytes) return BT_ERR_INVALID_ARG;
  if (batch_size <= 0 || total_tokens <= 0) return fail(h, BT_ERR_INVALID_ARG, "batch_size and total_tokens must be positive");
  *bytes = carve(nullptr, static_cast<size_t>(total_tokens), h->hidden, h->ffn, 0, 0).bytes;
  return BT_OK;
}

int bt_profile_enable(bt_handle h, int on) {
  if (!h) return BT_ERR_INVALID_ARG;
  h->prof_on = on != 0;
  if (on) {
    h->spans.clear();
    h->ev_used = 0;
    for (int i = 0; i < BT_PROF_KINDS; ++i) h->launches[i] = 0;
  }
  return BT_OK;
}

int bt_profile_read(bt_handle h, double* ms_by_kind, long long* launches_by_kind) {
  if (!h || !ms_by_kind || !launches_by_kind) return BT_ERR_INVALID_ARG;
  for (int i = 0; i < BT_PROF_KINDS; ++i) {
    ms_by_kind[i] = 0.0;
    launches_by_kind[i] = h->launches[i];
  }
  for (const auto& sp : h->spans) {
    cudaError_t e = cudaEventSynchronize(sp.end);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, sp.beg, sp.end);
    if (e != cudaSuccess) return fail_cuda(h, e, "bt_profile_read");
    ms_by_kind[sp.kind] += ms;
  }
  return BT_OK;
}

const char* bt_last_error(bt_handle h) { return h ? h->err.c_str() : "null handle"; }

int bt_device_status(bt_handle h, void* stream, int* status) {
  if (!h || !status) return BT_ERR_INVALID_ARG;
  {
    const int rc = check_device(h);
    if (rc != BT_OK) return rc;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, h->status, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail_cuda(h, e, "bt_device_status");
  if (v != 0) {
    e = cudaMemsetAsync(h->status, 0, sizeof(int), s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail_cuda(h, e, "bt_device_status reset");
  }
  *status = v;
  return BT_OK;
}

int bt_embedding_layernorm(const void* word_emb, const void* pos_emb, const void* type_emb, const void* gamma,
                           const void* beta, int gamma_beta_fp32, const int* token_ids, const int* type_ids,
                           const int* position_ids, void* out, int batch_size, int seq_len, int hidden, int vocab_size,
                           int max_positions, int type_vocab_size, float eps, void* stream) {
  if (!word_emb || !pos_emb || !type_emb || !gamma || !beta || !token_ids || !out) return BT_ERR_INVALID_ARG;
  if (batch_size <= 0 || seq_len <= 0 || hidden <= 0 || hidden % 8 != 0 || hidden > 1024 || vocab_size <= 0 ||
      max_positions <= 0 || type_vocab_size <= 0 || !(eps >= 0.f))
    return BT_ERR_INVALID_ARG;
  if (static_cast<long long>(batch_size) * seq_len > 0x7fffffffLL) return BT_ERR_INVALID_ARG;
  const void* ptrs[6] = {word_emb, pos_emb, type_emb, gamma, beta, out};
  for (const void* p : ptrs)
    if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_embedding_layernorm(
      reinterpret_cast<const __half*>(word_emb), reinterpret_cast<const __half*>(pos_emb),
      reinterpret_cast<const __half*>(type_emb), gamma, beta, gamma_beta_fp32 != 0, token_ids, type_ids, position_ids,
      reinterpret_cast<__half*>(out), batch_size * seq_len, seq_len, hidden, vocab_size, max_positions, type_vocab_size,
      eps, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_embedding_layernorm_packed(const bt_embedding_weights* emb, const int* token_ids, const int* type_ids,
                                  const int* position_ids, const int* batch_idx, const int* word_idx,
                                  void* out_packed, int batch_size, int seq_len, int hidden, void* stream) {
  if (!token_ids || !batch_idx || !word_idx || !out_packed || !aligned16(out_packed)) return BT_ERR_INVALID_ARG;
  if (batch_size <= 0 || seq_len <= 0 || static_cast<long long>(batch_size) * seq_len > 0x7fffffffLL) return BT_ERR_INVALID_ARG;
  const int rc = check_embedding(nullptr, emb, hidden);
  if (rc != BT_OK) return rc;
  cudaError_t e = launch_embedding_layernorm(
      reinterpret_cast<const __half*>(emb->word_emb), reinterpret_cast<const __half*>(emb->pos_emb),
      reinterpret_cast<const __half*>(emb->type_emb), emb->gamma, emb->beta, emb->gamma_beta_fp32 != 0, token_ids, type_ids,
      position_ids, reinterpret_cast<__half*>(out_packed), batch_size * seq_len, seq_len, hidden, emb->vocab_size,
      emb->max_positions, emb->type_vocab_size, emb->eps, reinterpret_cast<cudaStream_t>(stream), word_idx,
      batch_idx + batch_size);
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_stack_forward_ids(bt_handle h, int n_layers, const bt_embedding_weights* emb, const int* token_ids,
                         const int* type_ids, const int* position_ids, const void* attr_mask, void* out,
                         void* workspace, size_t workspace_bytes, int batch_size, int seq_len, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  IdsInput ids{emb, token_ids, type_ids, position_ids};
  return stack_padded(h, 0, n_layers, nullptr, attr_mask, out, workspace, workspace_bytes, batch_size, seq_len, stream,
                      &ids);
}

int bt_pooler(const void* encoder_out, const void* W, const void* bias, void* pooled, int batch_size, int seq_len,
              int hidden, void* stream) {
  if (!encoder_out || !W || !bias || !pooled || batch_size <= 0 || seq_len <= 0 || hidden <= 0) return BT_ERR_INVALID_ARG;
  if (!aligned16(encoder_out) || !aligned16(W) || !aligned16(bias) || !aligned16(pooled)) return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_pooler(reinterpret_cast<const __half*>(encoder_out), reinterpret_cast<const __half*>(W),
                                reinterpret_cast<const __half*>(bias), reinterpret_cast<__half*>(pooled), batch_size,
                                seq_len, hidden, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaErrorInvalidValue) return BT_ERR_INVALID_ARG;
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_selftest_bounded_wait(bt_handle h, long long max_cycles, int* gave_up_dev, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  {
    const int rc = check_device(h);
    if (rc != BT_OK) return rc;
  }
  cudaError_t e = launch_bounded_wait_selftest(h->status, max_cycles, gave_up_dev, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(h, e, "self-test launch");
  return BT_OK;
}

int bt_layer_forward_padded(bt_handle h, int layer, const void* input, const void* attr_mask, void* out,
                            void* workspace, size_t workspace_bytes, int batch_size, int seq_len, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  return stack_padded(h, layer, 1, input, attr_mask, out, workspace, workspace_bytes, batch_size, seq_len, stream);
}

// Scratch of bt_layer_forward_padded_static(): a fixed array in the library's
// device image instead of a caller-supplied workspace.  Every device that loads
// the library carries these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[BT_STATIC_SCRATCH_BYTES];

// `g_static_scratch` names a host-side shadow in host code, not device memory, so
// the address a kernel may use is asked from the runtime once per device, with that
// device current.
static int static_scratch_address(int device, void** out) {
  static std::mutex mu;
  static void* addr[64] = {};
  if (device < 0 || device >= 64) return BT_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[device] == nullptr) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) return BT_ERR_CUDA;
    if (cur != device && cudaSetDevice(device) != cudaSuccess) return BT_ERR_CUDA;
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (cur != device) cudaSetDevice(cur);
    if (e != cudaSuccess || p == nullptr) return BT_ERR_CUDA;
    addr[device] = p;
  }
  *out = addr[device];
  return BT_OK;
}

int bt_layer_forward_padded_static(bt_handle h, int layer, const void* input, const void* attr_mask, void* out,
                                   int batch_size, int seq_len, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  size_t need = 0;
  int rc = bt_workspace_bytes(h, batch_size, seq_len, &need);
  if (rc != BT_OK) return rc;
  if ((rc = check_device(h)) != BT_OK) return rc;  // the scratch address below is only valid on the handle's device
  if (need > static_cast<size_t>(BT_STATIC_SCRATCH_BYTES))
    return fail(h, BT_ERR_WORKSPACE,
                "batch_size*seq_len needs more scratch than the built-in BT_STATIC_SCRATCH_BYTES; "
                "use bt_layer_forward_padded() with a caller workspace");
  void* scratch = nullptr;
  rc = static_scratch_address(h->device, &scratch);
  if (rc != BT_OK) return fail(h, rc, "cudaGetSymbolAddress failed for the built-in scratch array");
  return stack_padded(h, layer, 1, input, attr_mask, out, scratch, static_cast<size_t>(BT_STATIC_SCRATCH_BYTES),
                      batch_size, seq_len, stream);
}

int bt_layer_forward_padded_general(bt_handle h, int layer, const void* input, const void* attr_mask,
                                    const void* attention_bias, void* out, void* workspace, size_t workspace_bytes,
                                    int batch_size, int seq_len, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  return stack_general(h, layer, 1, input, attr_mask, attention_bias, out, workspace, workspace_bytes, batch_size,
                       seq_len, stream);
}

int bt_stack_forward_padded_general(bt_handle h, int n_layers, const void* input, const void* attr_mask,
                                    const void* attention_bias, void* out, void* workspace, size_t workspace_bytes,
                                    int batch_size, int seq_len, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  return stack_general(h, 0, n_layers, input, attr_mask, attention_bias, out, workspace, workspace_bytes, batch_size,
                       seq_len, stream);
}

int bt_mask_is_right_padded(const void* attr_mask, int batch_size, int seq_len, int* scratch_dev, int* result,
                            void* stream) {
  if (!attr_mask || !scratch_dev || !result || batch_size <= 0 || seq_len <= 0) return BT_ERR_INVALID_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = launch_mask_is_right_padded(reinterpret_cast<const __half*>(attr_mask), batch_size, seq_len,
                                              scratch_dev, s);
  if (e == cudaSuccess) e = cudaMemcpyAsync(result, scratch_dev, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_stack_forward_padded(bt_handle h, int n_layers, const void* input, const void* attr_mask, void* out,
                            void* workspace, size_t workspace_bytes, int batch_size, int seq_len, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  return stack_padded(h, 0, n_layers, input, attr_mask, out, workspace, workspace_bytes, batch_size, seq_len, stream);
}

int bt_stack_forward_packed(bt_handle h, int n_layers, const void* x_packed, const int* cu_seqlens, int batch_size,
                            int max_len, int total_tokens, void* out_packed, void* workspace, size_t workspace_bytes,
                            void* stream_v) {
  if (!h) return BT_ERR_INVALID_ARG;
  if (!x_packed || !cu_seqlens || !out_packed || !workspace) return fail(h, BT_ERR_INVALID_ARG, "null pointer argument");
  if (batch_size <= 0 || batch_size > 65535 || total_tokens <= 0 || max_len <= 0 || n_layers <= 0)
    return fail(h, BT_ERR_INVALID_ARG, "bad batch_size / total_tokens / max_len / n_layers");
  if (x_packed == out_packed) return fail(h, BT_ERR_INVALID_ARG, "input and output must not alias");
  if (!aligned16(x_packed) || !aligned16(out_packed))
    return fail(h, BT_ERR_INVALID_ARG, "x_packed and out_packed must be 16-byte aligned");
  {
    const int rc = check_device(h);
    if (rc != BT_OK) return rc;
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  Workspace need = carve(nullptr, static_cast<size_t>(total_tokens), h->hidden, h->ffn, 0, 0);
  if (workspace_bytes < need.bytes) return fail(h, BT_ERR_WORKSPACE, "workspace smaller than bt_workspace_bytes_packed()");
  void* base = reinterpret_cast<void*>(align_up(reinterpret_cast<uintptr_t>(workspace), 1024));
  Workspace ws = carve(base, static_cast<size_t>(total_tokens), h->hidden, h->ffn, 0, 0);
  {
    const int rc = prepare_ln_sync(h, ws, total_tokens, stream);
    if (rc != BT_OK) return rc;
  }
  pdl_next_launch_plain();  // first kernel of the call: see kernels.h
  const __half* cur = reinterpret_cast<const __half*>(x_packed);
  for (int l = 0; l < n_layers; ++l) {
    const bool last = (l == n_layers - 1);
    __half* dst = last ? reinterpret_cast<__half*>(out_packed) : ((l & 1) ? ws.xb : ws.xa);
    int rc = run_layer(h, l, cur, dst, nullptr, ws, cu_seqlens, batch_size, max_len, total_tokens, stream);
    if (rc != BT_OK) return rc;
    cur = dst;
  }
  return BT_OK;
}

int bt_build_offsets(const void* attr_mask, int batch_size, int seq_len, int* batch_idx, int* word_idx, void* stream) {
  if (!attr_mask || !batch_idx || !word_idx || batch_size <= 0 || seq_len <= 0 || !aligned16(attr_mask))
    return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_build_offsets(reinterpret_cast<const __half*>(attr_mask), batch_size, seq_len, batch_idx,
                                       word_idx, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_pack_rows(const void* padded, void* packed, const int* batch_idx, const int* word_idx, int batch_size,
                 int seq_len, int hidden, void* stream) {
  (void)word_idx;  // right padding makes each sequence one contiguous run; batch_idx is enough
  if (!padded || !packed || !batch_idx || batch_size <= 0 || batch_size > 65535 || seq_len <= 0 || hidden <= 0 ||
      hidden % 8 != 0 || !aligned16(padded) || !aligned16(packed))
    return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_pack_rows(reinterpret_cast<const __half*>(padded), reinterpret_cast<__half*>(packed),
                                   batch_idx, batch_size, seq_len, hidden, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_restore_rows(const void* packed, void* padded, const int* batch_idx, int batch_size, int seq_len, int hidden,
                    void* stream) {
  if (!packed || !padded || !batch_idx || batch_size <= 0 || batch_size > 65535 || seq_len <= 0 || hidden <= 0 ||
      hidden % 8 != 0 || !aligned16(packed) || !aligned16(padded))
    return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_restore_rows(reinterpret_cast<const __half*>(packed), reinterpret_cast<__half*>(padded),
                                      batch_idx, batch_size, seq_len, hidden, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_gemm(bt_handle h, const void* A, const void* W, void* out, const void* bias, const void* residual,
            const int* m_dev, int m_rows, int N, int K, int epilogue, int gelu_kind, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  if (!A || !W || !out) return fail(h, BT_ERR_INVALID_ARG, "null pointer argument");
  if (m_rows <= 0 || N <= 0 || K <= 0 || N % 64 != 0 || K % 64 != 0)
    return fail(h, BT_ERR_INVALID_ARG, "bt_gemm needs m_rows > 0, N % 64 == 0, K % 64 == 0");
  if (epilogue < BT_EPI_NONE || epilogue > BT_EPI_BIAS_RESIDUAL_F32OUT) return fail(h, BT_ERR_INVALID_ARG, "bad epilogue");
  if (epilogue != BT_EPI_NONE && !bias) return fail(h, BT_ERR_INVALID_ARG, "epilogue needs bias");
  if ((epilogue == BT_EPI_BIAS_RESIDUAL || epilogue == BT_EPI_BIAS_RESIDUAL_F32OUT) && !residual) return fail(h, BT_ERR_INVALID_ARG, "epilogue needs residual");
  {
    const int rc = check_device(h);
    if (rc != BT_OK) return rc;
  }
  pdl_next_launch_plain();  // W may come straight from the caller's kernel before: see kernels.h
  return run_gemm(h, BT_PROF_GEMM_OTHER, reinterpret_cast<const __half*>(A), W, reinterpret_cast<__half*>(out), bias,
                  reinterpret_cast<const __half*>(residual), m_dev, m_rows, N, K, epilogue, gelu_kind,
                  reinterpret_cast<cudaStream_t>(stream));
}

int bt_gemm_layernorm(bt_handle h, const void* A, const void* W, const void* bias, const void* residual,
                      const void* gamma, const void* beta, int gamma_beta_fp32, float eps, void* scratch_f32, void* out,
                      const int* m_dev, int m_rows, int N, int K, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  if (!A || !W || !bias || !residual || !gamma || !beta || !scratch_f32 || !out)
    return fail(h, BT_ERR_INVALID_ARG, "null pointer argument");
  if (m_rows <= 0 || N <= 0 || K <= 0 || N % 256 != 0 || N > 1024 || K % 64 != 0)
    return fail(h, BT_ERR_INVALID_ARG, "bt_gemm_layernorm needs m_rows > 0, N % 256 == 0, N <= 1024, K % 64 == 0");
  {
    const int rc = check_device(h);
    if (rc != BT_OK) return rc;
  }
  // scratch: [m_rows][N/128] tagged partials of 16 bytes, zeroed here; this launch is number 1 on it
  cudaError_t me = cudaMemsetAsync(scratch_f32, 0, static_cast<size_t>(m_rows) * (N / 128) * 16,
                                   reinterpret_cast<cudaStream_t>(stream));
  if (me != cudaSuccess) return fail_cuda(h, me, "memset of the LayerNorm statistics scratch");
  LnArgs ln{1u, reinterpret_cast<__half*>(out), gamma, beta, gamma_beta_fp32 != 0, eps};
  return run_gemm(h, BT_PROF_GEMM_OTHER, reinterpret_cast<const __half*>(A), W, reinterpret_cast<__half*>(scratch_f32),
                  bias, reinterpret_cast<const __half*>(residual), m_dev, m_rows, N, K, BT_EPI_BIAS_RESIDUAL_LAYERNORM, 0,
                  reinterpret_cast<cudaStream_t>(stream), &ln);
}

// Diagnostics hook: LayerNorm inside the attention-output / FFN2 GEMM kernels: 0 = never (row
// kernel), 1 = when the call has enough 128-row tiles (default), 2 = always; values above 2
// keep mode 1 and set the tile threshold to that value.
int bt_debug_set_fused_layernorm(bt_handle h, int on) {
  if (!h) return BT_ERR_INVALID_ARG;
  h->fused_ln_ffn2_only = false;
  if (on == 3) {  // mode 1 for the FFN2 GEMM only
    h->fused_ln = 1;
    h->fused_ln_ffn2_only = true;
  } else if (on > 3) {
    h->fused_ln = 1;
    h->fused_ln_min_tiles = on;
  } else {
    h->fused_ln = on < 0 ? 0 : on;
  }
  return BT_OK;
}

int bt_attention(bt_handle h, const void* qkv, void* ctx, const int* batch_idx, int batch_size, int max_len,
                 int rows_allocated, void* stream) {
  if (!h) return BT_ERR_INVALID_ARG;
  if (!qkv || !ctx || !batch_idx || batch_size <= 0 || batch_size > 65535 || max_len <= 0 || rows_allocated <= 0)
    return fail(h, BT_ERR_INVALID_ARG, "bad argument to bt_attention");
  if (!aligned16(qkv) || !aligned16(ctx)) return fail(h, BT_ERR_INVALID_ARG, "qkv and ctx must be 16-byte aligned");
  {
    const int rc = check_device(h);
    if (rc != BT_OK) return rc;
  }
  return run_mha(h, reinterpret_cast<const __half*>(qkv), reinterpret_cast<__half*>(ctx), batch_idx, batch_size,
                 max_len, rows_allocated, reinterpret_cast<cudaStream_t>(stream));
}

int bt_add_bias_residual_layernorm(const void* x, int x_fp32, const void* bias, const void* residual, const void* gamma,
                                   const void* beta, int gamma_beta_fp32, void* out, const int* m_dev, int m_rows,
                                   int hidden, float eps, void* stream) {
  if (!x || !gamma || !beta || !out || m_rows <= 0 || hidden <= 0 || hidden % 8 != 0 || hidden > 1024)
    return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_layernorm(x, x_fp32 != 0, reinterpret_cast<const __half*>(bias),
                                   reinterpret_cast<const __half*>(residual), gamma, beta, gamma_beta_fp32 != 0,
                                   reinterpret_cast<__half*>(out), m_dev, m_rows, hidden, eps,
                                   reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_add_bias_residual_layernorm_restore(const void* x, int x_fp32, const void* bias, const void* residual, const void* gamma,
                                           const void* beta, int gamma_beta_fp32, void* out_padded,
                                           const int* batch_idx, int batch_size, int seq_len, int hidden, float eps,
                                           void* stream) {
  if (!x || !gamma || !beta || !out_padded || !batch_idx || batch_size <= 0 || seq_len <= 0 || hidden <= 0 ||
      hidden % 8 != 0 || hidden > 1024)
    return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_layernorm_restore(
      x, x_fp32 != 0, reinterpret_cast<const __half*>(bias),
      reinterpret_cast<const __half*>(residual), gamma, beta, gamma_beta_fp32 != 0,
      reinterpret_cast<__half*>(out_padded), batch_idx, batch_size, seq_len, hidden, eps,
      reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_add_bias_gelu(void* x, const void* bias, const int* m_dev, int m_rows, int n, int gelu_kind, void* stream) {
  if (!x || !bias || m_rows <= 0 || n <= 0 || n % 8 != 0) return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_add_bias_gelu(reinterpret_cast<__half*>(x), reinterpret_cast<const __half*>(bias), m_dev,
                                       m_rows, n, gelu_kind, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

int bt_masked_softmax(void* logits, const void* attr_mask, int batch_size, int head_num, int seq_len, float scale,
                      void* stream) {
  if (!logits || !attr_mask || batch_size <= 0 || head_num <= 0 || seq_len <= 0 || seq_len > 1024)
    return BT_ERR_INVALID_ARG;
  cudaError_t e = launch_masked_softmax(reinterpret_cast<__half*>(logits), reinterpret_cast<const __half*>(attr_mask),
                                        batch_size, head_num, seq_len, scale, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? BT_OK : BT_ERR_CUDA;
}

}  // extern "C"
