// Header-only C++ shim: the reference's `BertTransformer<OpType>` class API over the
// C ABI of libbt_b200.so, so that code written against
// bytetransformer/include/bert_transformer.h (class at :99-223, parameter structs at
// :31-96, `AttentionParam` at bytetransformer/include/attention.h:25-39) compiles and
// runs unchanged against this library.
//
// Same names, constructor arguments, method set and ownership rules: the caller owns
// every pointer (weights, input, mask, output, the `cal_bufsize()`-byte buffer, the
// stream); the object stores raw weight pointers only.  Differences:
//   * only OperationType::HALF runs (the FP32 template is not built for sm_100a);
//     constructing the FP32 variant throws std::runtime_error;
//   * `is_remove_padding = false` or a non-NULL `attention_bias` selects the general-mask path: nothing
//     is packed, the whole [B,S,S] mask is applied element by element as (1 - mask) * -10000, every
//     output row is computed - the reference's padded path, which is also where it applies the bias
//     (its unfused softmax).  `is_remove_padding = true` packs by the valid keys of mask row 0 whatever
//     the batch size (the reference turns packing off for batches of one or two,
//     bytetransformer/include/bert_transformer.h:135-136; on right-padded masks the valid rows agree).
//     `use_fused_attention` is accepted and ignored (attention is fused on both paths, equal results);
//     `cublas_handle`, `cublas_Algo`, `position_ids`, `token_type_ids` are accepted and unused, as in
//     the reference for the latter two;
//   * errors surface as std::runtime_error with the library's message, never exit().
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "bt_b200.h"

struct cublasContext;
typedef struct cublasContext* cublasHandle_t;

namespace bytetransformer {

enum class OperationType { FP32, HALF };
enum ModelType { Bert };

template <OperationType OpType>
class Traits;
template <>
class Traits<OperationType::FP32> {
 public:
  typedef float DataType;
};
template <>
class Traits<OperationType::HALF> {
 public:
  typedef __half DataType;
};

template <OperationType OpType>
class AttentionParam {
 public:
  typedef typename Traits<OpType>::DataType DataType_;
  const DataType_* attr_bias_QKV = nullptr;  // [3H]
  float tao = 1.0f;
  int cublas_Algo[2] = {99, 99};
};

template <OperationType OpType>
class BertTransformerParam {
 public:
  typedef typename Traits<OpType>::DataType DataType_;
  AttentionParam<OpType> attention_param;
  const DataType_* attr_kernel_QKV = nullptr;
  const DataType_* attr_output_kernel = nullptr;
  const DataType_* attr_output_bias = nullptr;
  const void* attr_output_layernorm_gamma = nullptr;
  const void* attr_output_layernorm_beta = nullptr;
  const DataType_* inter_kernel = nullptr;
  const DataType_* inter_bias = nullptr;
  const DataType_* output_kernel = nullptr;
  const DataType_* output_bias = nullptr;
  const void* output_layernorm_gamma = nullptr;
  const void* output_layernorm_beta = nullptr;
  int intermediate_size = 4;
  int cublas_Algo[3] = {99, 99, 99};
};

template <typename T>
struct BertTransformerInferParam {
  const T* input_tensor;  // [batch_size, seq_len, hidden_dim]
  const T* atten_mask;    // [batch_size, seq_len, seq_len], 1 = attend, 0 = masked
  T* transformer_output;  // [batch_size, seq_len, hidden_dim]
  void* buf;              // cal_bufsize() bytes of device memory
  int batch_size;
  int seq_len;
  cublasHandle_t cublas_handle;  // unused
  cudaStream_t stream;
  const T* attention_bias = NULL;          // [head_num, seq_len, seq_len]: selects the general-mask path
  const uint32_t* position_ids = NULL;     // unused
  const uint32_t* token_type_ids = NULL;   // unused
};

template <OperationType OpType>
class BertTransformer {
 public:
  typedef typename Traits<OpType>::DataType DataType_;

  BertTransformer(const int max_batch_size, const int head_num, const int size_per_head, const int max_seq_len,
                  const bool use_fused_attention = true, const bool is_remove_padding = true,
                  const bool use_fp32 = false, const ModelType model_type = ModelType::Bert)
      : max_batch_size_(max_batch_size), max_seq_len_(max_seq_len), use_fp32_(use_fp32),
        is_remove_padding_(is_remove_padding) {
    (void)use_fused_attention;  // attention is fused on both paths, with equal results
    (void)model_type;
    if (OpType != OperationType::HALF)
      throw std::runtime_error("bt_b200: only OperationType::HALF is built for sm_100a");
    cfg_.head_num = head_num;
    cfg_.size_per_head = size_per_head;
    cfg_.max_batch_size = max_batch_size;
    cfg_.max_seq_len = max_seq_len;
    cfg_.intermediate_mult = 4;
    cfg_.ln_eps = 1e-6f;
    cfg_.gelu_kind = BT_GELU_ERF;
    cfg_.tao = 1.0f;
    cfg_.gamma_beta_fp32 = use_fp32 ? 1 : 0;
    cfg_.device = -1;
  }
  BertTransformer(const BertTransformer&) = delete;
  BertTransformer& operator=(const BertTransformer&) = delete;
  ~BertTransformer() {
    if (handle_) bt_destroy(handle_);
  }

  // Optional knobs that the reference hard-codes in its kernels; call before initialize().
  void set_layernorm_eps(float eps) { cfg_.ln_eps = eps; }
  void set_gelu_tanh(bool tanh_form) { cfg_.gelu_kind = tanh_form ? BT_GELU_TANH : BT_GELU_ERF; }

  void initialize(BertTransformerParam<OpType> param) {
    param_ = param;
    cfg_.intermediate_mult = param.intermediate_size;
    cfg_.tao = param.attention_param.tao;
    if (handle_) {
      bt_destroy(handle_);
      handle_ = nullptr;
    }
    check(bt_create(&cfg_, &handle_), "bt_create");
    bt_layer_weights w;
    w.qkv_kernel = param.attr_kernel_QKV;
    w.qkv_bias = param.attention_param.attr_bias_QKV;
    w.attr_output_kernel = param.attr_output_kernel;
    w.attr_output_bias = param.attr_output_bias;
    w.attr_output_layernorm_gamma = param.attr_output_layernorm_gamma;
    w.attr_output_layernorm_beta = param.attr_output_layernorm_beta;
    w.inter_kernel = param.inter_kernel;
    w.inter_bias = param.inter_bias;
    w.output_kernel = param.output_kernel;
    w.output_bias = param.output_bias;
    w.output_layernorm_gamma = param.output_layernorm_gamma;
    w.output_layernorm_beta = param.output_layernorm_beta;
    check(bt_set_layer_weights(handle_, 0, &w), "bt_set_layer_weights");
  }

  unsigned long long cal_bufsize() {
    if (!handle_) throw std::runtime_error("bt_b200: initialize() must be called before cal_bufsize()");
    size_t bytes = 0;
    check(bt_workspace_bytes(handle_, max_batch_size_, max_seq_len_, &bytes), "bt_workspace_bytes");
    buf_bytes_ = bytes;
    return static_cast<unsigned long long>(bytes);
  }

  void infer(BertTransformerInferParam<DataType_> infer_param) {
    if (!handle_) throw std::runtime_error("bt_b200: initialize() must be called before infer()");
    if (buf_bytes_ == 0) cal_bufsize();
    if (!is_remove_padding_ || infer_param.attention_bias != NULL) {
      // the reference's padded path: nothing is packed, the whole [B,S,S] mask is applied element by element
      // as (1 - mask) * -10000, the optional bias is added, every output row is computed
      check(bt_layer_forward_padded_general(handle_, 0, infer_param.input_tensor, infer_param.atten_mask,
                                            infer_param.attention_bias, infer_param.transformer_output, infer_param.buf,
                                            buf_bytes_, infer_param.batch_size, infer_param.seq_len, infer_param.stream),
            "bt_layer_forward_padded_general");
      return;
    }
    check(bt_layer_forward_padded(handle_, 0, infer_param.input_tensor, infer_param.atten_mask,
                                  infer_param.transformer_output, infer_param.buf, buf_bytes_, infer_param.batch_size,
                                  infer_param.seq_len, infer_param.stream),
          "bt_layer_forward_padded");
  }

 private:
  void check(int rc, const char* where) {
    if (rc != BT_OK)
      throw std::runtime_error(std::string("bt_b200 ") + where + " failed (code " + std::to_string(rc) + "): " +
                               (handle_ ? bt_last_error(handle_) : "no handle"));
  }
  bt_config cfg_{};
  bt_handle handle_ = nullptr;
  BertTransformerParam<OpType> param_;
  int max_batch_size_, max_seq_len_;
  bool use_fp32_;
  bool is_remove_padding_;
  size_t buf_bytes_ = 0;
};

}  // namespace bytetransformer
