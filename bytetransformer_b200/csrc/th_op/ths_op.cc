// PyTorch plugin: the functional operator `ByteTransformer::BertTransformer` and the
// TorchScript class `ByteTransformer.BertTransformer`, with the schemas, argument
// checks and pickle state of the reference plugin
// (bytetransformer/th_op/ths_op_f.cc:28-95, th_op/ths_op.h:29-110, th_op/ths_op.cc:27-43).
//
// All computation goes through the C ABI of libbt_b200.so; torch only supplies
// tensors, the caching allocator for the workspace, the current stream and the
// device guard.  fp32 tensors select the reference's FP32 template; that template
// is not built for sm_100a, so anything but fp16 is rejected with a clear error.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <vector>

#include "bt_b200.h"

namespace bt_th {

using torch::Tensor;

#define BT_CHECK_CUDA(x) TORCH_CHECK(x.is_cuda(), #x " must be a CUDA tensor")
#define BT_CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define BT_CHECK_TYPE(x, st) TORCH_CHECK(x.scalar_type() == st, "Inconsistency of Tensor type: " #x)
#define BT_CHECK_INPUT(x, st) \
  BT_CHECK_CUDA(x);           \
  BT_CHECK_CONTIGUOUS(x);     \
  BT_CHECK_TYPE(x, st)
#define BT_CHECK_INPUT_LOOSE(x) \
  BT_CHECK_CUDA(x);             \
  BT_CHECK_CONTIGUOUS(x)

// Owns one C-ABI encoder holding a single layer.
class LayerEncoder {
 public:
  LayerEncoder(int64_t head_num, int64_t head_size, const std::vector<Tensor>& w) : weights_(w) {
    TORCH_CHECK(w.size() == 12, "expected 12 weight tensors");
    const at::ScalarType st = w[0].scalar_type();
    TORCH_CHECK(st == at::ScalarType::Half,
                "Wrong Tensor type: this build runs fp16 only (the FP32 path is not built for sm_100a)");
    const bool gb_fp32 = w[10].scalar_type() == at::ScalarType::Float;
    for (int i : {4, 5, 10, 11})
      TORCH_CHECK(w[i].scalar_type() == (gb_fp32 ? at::ScalarType::Float : at::ScalarType::Half),
                  "LayerNorm gamma/beta must all be fp16 or all be fp32");
    const int64_t H = head_num * head_size;
    TORCH_CHECK(w[0].dim() == 2 && w[0].size(0) == H && w[0].size(1) == 3 * H, "qkv_kernel must be [H,3H]");
    TORCH_CHECK(w[6].dim() == 2 && w[6].size(0) == H && w[6].size(1) == 4 * H, "inter_kernel must be [H,4H]");
    bt_config cfg;
    cfg.head_num = static_cast<int>(head_num);
    cfg.size_per_head = static_cast<int>(head_size);
    cfg.max_batch_size = 65535;
    cfg.max_seq_len = 1024;
    cfg.intermediate_mult = 4;
    cfg.ln_eps = 1e-6f;
    cfg.gelu_kind = BT_GELU_ERF;
    cfg.tao = 1.0f;
    cfg.gamma_beta_fp32 = gb_fp32 ? 1 : 0;
    cfg.device = w[0].device().index();
    const int rc = bt_create(&cfg, &handle_);
    TORCH_CHECK(rc == BT_OK, "bt_create failed (code ", rc, "): head_size must be 64 and the device sm_100");
    bt_layer_weights lw;
    const void** p = reinterpret_cast<const void**>(&lw);
    for (int i = 0; i < 12; ++i) p[i] = w[i].data_ptr();
    const int rc2 = bt_set_layer_weights(handle_, 0, &lw);
    TORCH_CHECK(rc2 == BT_OK, "bt_set_layer_weights failed: ", bt_last_error(handle_));
  }
  ~LayerEncoder() { bt_destroy(handle_); }
  LayerEncoder(const LayerEncoder&) = delete;
  LayerEncoder& operator=(const LayerEncoder&) = delete;

  // is_remove_padding = true: the packed path (lengths = valid keys of mask row 0, right padding, padding
  // rows of the output zero).  false, or an attention_bias: the reference's padded semantics - nothing is
  // packed, the whole [B,S,S] mask is applied element by element as (1 - mask) * -10000, the optional
  // [head_num,S,S] bias is added to the scaled scores, every output row is computed
  // (bytetransformer/th_op/bert_transformer_ext.h:80-111, bytetransformer/include/softmax.h:41-45).
  Tensor forward(const Tensor& input, const Tensor& attr_mask, bool is_remove_padding = true,
                 const Tensor& attention_bias = Tensor()) {
    TORCH_CHECK(input.dim() == 3, "input must be [batch, seq_len, hidden]");
    const int batch = static_cast<int>(input.size(0));
    const int seq = static_cast<int>(input.size(1));
    TORCH_CHECK(seq <= 1024, "Input seq_len too long");
    TORCH_CHECK(attr_mask.dim() == 3 && attr_mask.size(0) == batch && attr_mask.size(1) == seq &&
                    attr_mask.size(2) == seq,
                "attr_mask must be [batch, seq_len, seq_len]");
    c10::cuda::CUDAGuard guard(input.device());
    Tensor out = torch::empty_like(input);
    size_t bytes = 0;
    int rc = bt_workspace_bytes(handle_, batch, seq, &bytes);
    TORCH_CHECK(rc == BT_OK, "bt_workspace_bytes failed: ", bt_last_error(handle_));
    Tensor buf = torch::empty({static_cast<int64_t>(bytes)}, torch::dtype(torch::kInt8).device(input.device()));
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    if (!is_remove_padding || attention_bias.defined()) {
      const void* bias = nullptr;
      if (attention_bias.defined()) {
        TORCH_CHECK(attention_bias.is_cuda() && attention_bias.is_contiguous() &&
                        attention_bias.scalar_type() == input.scalar_type() && attention_bias.dim() == 3 &&
                        attention_bias.size(1) == seq && attention_bias.size(2) == seq,
                    "attention_bias must be a contiguous CUDA tensor [head_num, seq_len, seq_len] of the input's type");
        bias = attention_bias.data_ptr();
      }
      rc = bt_layer_forward_padded_general(handle_, 0, input.data_ptr(), attr_mask.data_ptr(), bias, out.data_ptr(),
                                           buf.data_ptr(), bytes, batch, seq, stream);
      TORCH_CHECK(rc == BT_OK, "bt_layer_forward_padded_general failed: ", bt_last_error(handle_));
      return out;
    }
    rc = bt_layer_forward_padded(handle_, 0, input.data_ptr(), attr_mask.data_ptr(), out.data_ptr(), buf.data_ptr(),
                                 bytes, batch, seq, stream);
    TORCH_CHECK(rc == BT_OK, "bt_layer_forward_padded failed: ", bt_last_error(handle_));
    return out;
  }

  const std::vector<Tensor>& weights() const { return weights_; }

 private:
  bt_handle handle_ = nullptr;
  std::vector<Tensor> weights_;  // keeps the device memory alive; the library stores raw pointers
};

static void check_weights(const std::vector<Tensor>& w) {
  const at::ScalarType st = w[0].scalar_type();
  const Tensor &qkv_kernel = w[0], &qkv_bias = w[1], &attr_output_kernel = w[2], &attr_output_bias = w[3],
               &attr_output_layernorm_gamma = w[4], &attr_output_layernorm_beta = w[5], &inter_kernel = w[6],
               &inter_bias = w[7], &output_kernel = w[8], &output_bias = w[9], &output_layernorm_gamma = w[10],
               &output_layernorm_beta = w[11];
  BT_CHECK_INPUT(qkv_kernel, st);
  BT_CHECK_INPUT(qkv_bias, st);
  BT_CHECK_INPUT(attr_output_kernel, st);
  BT_CHECK_INPUT(attr_output_bias, st);
  BT_CHECK_INPUT_LOOSE(attr_output_layernorm_gamma);
  BT_CHECK_INPUT_LOOSE(attr_output_layernorm_beta);
  BT_CHECK_INPUT(inter_kernel, st);
  BT_CHECK_INPUT(inter_bias, st);
  BT_CHECK_INPUT(output_kernel, st);
  BT_CHECK_INPUT(output_bias, st);
  BT_CHECK_INPUT_LOOSE(output_layernorm_gamma);
  BT_CHECK_INPUT_LOOSE(output_layernorm_beta);
}

// Functional form: builds the encoder object per call, like the reference.
Tensor TransformerEncoder(int64_t head_num, int64_t head_size, Tensor qkv_kernel, Tensor qkv_bias,
                          Tensor attr_output_kernel, Tensor attr_output_bias, Tensor attr_output_layernorm_gamma,
                          Tensor attr_output_layernorm_beta, Tensor inter_kernel, Tensor inter_bias,
                          Tensor output_kernel, Tensor output_bias, Tensor output_layernorm_gamma,
                          Tensor output_layernorm_beta, Tensor input, Tensor attr_mask, bool is_remove_padding,
                          bool use_fused_attention) {
  (void)use_fused_attention;  // accepted for compatibility: attention is fused on both paths, with equal results
  std::vector<Tensor> weights{qkv_kernel,   qkv_bias,      attr_output_kernel,          attr_output_bias,
                              attr_output_layernorm_gamma, attr_output_layernorm_beta,  inter_kernel,
                              inter_bias,   output_kernel, output_bias,                 output_layernorm_gamma,
                              output_layernorm_beta};
  check_weights(weights);
  const at::ScalarType st = qkv_kernel.scalar_type();
  BT_CHECK_INPUT(input, st);
  BT_CHECK_INPUT(attr_mask, st);
  LayerEncoder enc(head_num, head_size, weights);
  return enc.forward(input, attr_mask, is_remove_padding);
}

class BertTransformer : public torch::jit::CustomClassHolder {
 public:
  BertTransformer(int64_t head_num, int64_t head_size, Tensor qkv_kernel, Tensor qkv_bias, Tensor attr_output_kernel,
                  Tensor attr_output_bias, Tensor attr_output_layernorm_gamma, Tensor attr_output_layernorm_beta,
                  Tensor inter_kernel, Tensor inter_bias, Tensor output_kernel, Tensor output_bias,
                  Tensor output_layernorm_gamma, Tensor output_layernorm_beta)
      : st_(qkv_kernel.scalar_type()) {
    std::vector<Tensor> weights{qkv_kernel,   qkv_bias,      attr_output_kernel,         attr_output_bias,
                                attr_output_layernorm_gamma, attr_output_layernorm_beta, inter_kernel,
                                inter_bias,   output_kernel, output_bias,                output_layernorm_gamma,
                                output_layernorm_beta};
    check_weights(weights);
    enc_ = std::make_unique<LayerEncoder>(head_num, head_size, weights);
    head_info_ = torch::empty({2}, torch::dtype(torch::kInt64));
    head_info_[0] = head_num;
    head_info_[1] = head_size;
  }

  Tensor forward(Tensor input, Tensor attr_mask) { return forwardv2(input, attr_mask, true, true); }

  Tensor forwardv2(Tensor input, Tensor attr_mask, bool is_remove_padding, bool use_fused_attention) {
    (void)use_fused_attention;
    BT_CHECK_INPUT(input, st_);
    BT_CHECK_INPUT(attr_mask, st_);
    return enc_->forward(input, attr_mask, is_remove_padding);
  }

  // The reference's encoder object takes an optional attention_bias [head_num,S,S] that its operator
  // schema does not expose (bytetransformer/th_op/bert_transformer_ext.h:83,106); this method does.
  Tensor forward_with_bias(Tensor input, Tensor attr_mask, Tensor attention_bias) {
    BT_CHECK_INPUT(input, st_);
    BT_CHECK_INPUT(attr_mask, st_);
    BT_CHECK_INPUT(attention_bias, st_);
    return enc_->forward(input, attr_mask, false, attention_bias);
  }

  // 12 weight tensors + int64 [head_num, head_size], the reference's pickle state
  std::vector<Tensor> get_pickle_info() const {
    std::vector<Tensor> tmp(enc_->weights());
    tmp.push_back(head_info_);
    return tmp;
  }

 private:
  const at::ScalarType st_;
  std::unique_ptr<LayerEncoder> enc_;
  Tensor head_info_;
};

// The whole stack as one object: `ByteTransformer.BertEncoder(head_num, head_size, weights)` with the
// 12 tensors of every layer in turn (12 * n_layers tensors, each layer in the order of the one-layer class).
// The reference has no such class: its Python test loops over one-layer objects and so re-packs the tokens for
// every layer (unit_test/python_scripts/bert_transformer_test.py:191-200); here offsets and packing run once
// per forward (bt_stack_forward_padded) and the activations stay packed between the layers.
class BertEncoder : public torch::jit::CustomClassHolder {
 public:
  BertEncoder(int64_t head_num, int64_t head_size, std::vector<Tensor> weights)
      : weights_(std::move(weights)), head_num_(head_num), head_size_(head_size) {
    TORCH_CHECK(!weights_.empty() && weights_.size() % 12 == 0, "expected 12 weight tensors per layer");
    n_layers_ = static_cast<int>(weights_.size() / 12);
    st_ = weights_[0].scalar_type();
    TORCH_CHECK(st_ == at::ScalarType::Half,
                "Wrong Tensor type: this build runs fp16 only (the FP32 path is not built for sm_100a)");
    const bool gb_fp32 = weights_[10].scalar_type() == at::ScalarType::Float;
    bt_config cfg;
    cfg.head_num = static_cast<int>(head_num);
    cfg.size_per_head = static_cast<int>(head_size);
    cfg.max_batch_size = 65535;
    cfg.max_seq_len = 1024;
    cfg.intermediate_mult = 4;
    cfg.ln_eps = 1e-6f;
    cfg.gelu_kind = BT_GELU_ERF;
    cfg.tao = 1.0f;
    cfg.gamma_beta_fp32 = gb_fp32 ? 1 : 0;
    cfg.device = weights_[0].device().index();
    const int rc = bt_create(&cfg, &handle_);
    TORCH_CHECK(rc == BT_OK, "bt_create failed (code ", rc, "): head_size must be 64 and the device sm_100");
    for (int l = 0; l < n_layers_; ++l) {
      std::vector<Tensor> w(weights_.begin() + 12 * l, weights_.begin() + 12 * (l + 1));
      check_weights(w);
      for (int i : {4, 5, 10, 11})
        TORCH_CHECK(w[i].scalar_type() == (gb_fp32 ? at::ScalarType::Float : at::ScalarType::Half),
                    "LayerNorm gamma/beta must all be fp16 or all be fp32, in every layer");
      bt_layer_weights lw;
      const void** p = reinterpret_cast<const void**>(&lw);
      for (int i = 0; i < 12; ++i) p[i] = w[i].data_ptr();
      const int rc2 = bt_set_layer_weights(handle_, l, &lw);
      TORCH_CHECK(rc2 == BT_OK, "bt_set_layer_weights failed: ", bt_last_error(handle_));
    }
  }
  ~BertEncoder() { bt_destroy(handle_); }

  Tensor forward(Tensor input, Tensor attr_mask) { return forwardv2(input, attr_mask, true); }

  // is_remove_padding as in the one-layer class: true = packed path, false = every row computed and the whole
  // [B,S,S] mask applied element by element.
  Tensor forwardv2(Tensor input, Tensor attr_mask, bool is_remove_padding) {
    BT_CHECK_INPUT(input, st_);
    BT_CHECK_INPUT(attr_mask, st_);
    TORCH_CHECK(input.dim() == 3, "input must be [batch, seq_len, hidden]");
    const int batch = static_cast<int>(input.size(0));
    const int seq = static_cast<int>(input.size(1));
    TORCH_CHECK(seq <= 1024, "Input seq_len too long");
    TORCH_CHECK(attr_mask.dim() == 3 && attr_mask.size(0) == batch && attr_mask.size(1) == seq &&
                    attr_mask.size(2) == seq,
                "attr_mask must be [batch, seq_len, seq_len]");
    c10::cuda::CUDAGuard guard(input.device());
    Tensor out = torch::empty_like(input);
    size_t bytes = 0;
    int rc = bt_workspace_bytes(handle_, batch, seq, &bytes);
    TORCH_CHECK(rc == BT_OK, "bt_workspace_bytes failed: ", bt_last_error(handle_));
    Tensor buf = torch::empty({static_cast<int64_t>(bytes)}, torch::dtype(torch::kInt8).device(input.device()));
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    if (is_remove_padding)
      rc = bt_stack_forward_padded(handle_, n_layers_, input.data_ptr(), attr_mask.data_ptr(), out.data_ptr(),
                                   buf.data_ptr(), bytes, batch, seq, stream);
    else
      rc = bt_stack_forward_padded_general(handle_, n_layers_, input.data_ptr(), attr_mask.data_ptr(), nullptr,
                                           out.data_ptr(), buf.data_ptr(), bytes, batch, seq, stream);
    TORCH_CHECK(rc == BT_OK, "stack forward failed: ", bt_last_error(handle_));
    return out;
  }

  int64_t num_layers() const { return n_layers_; }

  // 12 * n_layers weight tensors + int64 [head_num, head_size]
  std::vector<Tensor> get_pickle_info() const {
    std::vector<Tensor> tmp(weights_);
    Tensor info = torch::empty({2}, torch::dtype(torch::kInt64));
    info[0] = head_num_;
    info[1] = head_size_;
    tmp.push_back(info);
    return tmp;
  }

 private:
  std::vector<Tensor> weights_;  // keeps the device memory alive; the library stores raw pointers
  int64_t head_num_, head_size_;
  int n_layers_ = 0;
  at::ScalarType st_ = at::ScalarType::Half;
  bt_handle handle_ = nullptr;
};

static auto registry = torch::RegisterOperators(
    "ByteTransformer::BertTransformer("
    "int head_num, int head_size,"
    "Tensor qkv_kernel, Tensor qkv_bias,"
    "Tensor attr_output_kernel, Tensor attr_output_bias,"
    "Tensor attr_output_layernorm_gamma, Tensor attr_output_layernorm_beta,"
    "Tensor inter_kernel, Tensor inter_bias, Tensor output_kernel, Tensor output_bias,"
    "Tensor output_layernorm_gamma, Tensor output_layernorm_beta, Tensor input, Tensor attr_mask,"
    "bool is_remove_padding = True, bool use_fused_attention = True) -> "
    "Tensor",
    &TransformerEncoder);

static auto bert_transformer_class =
    torch::jit::class_<BertTransformer>("ByteTransformer", "BertTransformer")
        .def(torch::jit::init<int64_t, int64_t, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor,
                              Tensor, Tensor, Tensor, Tensor>())
        .def("forward", &BertTransformer::forward)
        .def("forwardv2", &BertTransformer::forwardv2)
        .def("forward_with_bias", &BertTransformer::forward_with_bias)
        .def_pickle(
            [](const c10::intrusive_ptr<BertTransformer>& self) -> std::vector<Tensor> {
              return self->get_pickle_info();
            },
            [](std::vector<Tensor> state) -> c10::intrusive_ptr<BertTransformer> {
              const int64_t head_num = state[12][0].item().to<int64_t>();
              const int64_t head_size = state[12][1].item().to<int64_t>();
              return c10::make_intrusive<BertTransformer>(head_num, head_size, state[0], state[1], state[2], state[3],
                                                          state[4], state[5], state[6], state[7], state[8], state[9],
                                                          state[10], state[11]);
            });

static auto bert_encoder_class =
    torch::jit::class_<BertEncoder>("ByteTransformer", "BertEncoder")
        .def(torch::jit::init<int64_t, int64_t, std::vector<Tensor>>())
        .def("forward", &BertEncoder::forward)
        .def("forwardv2", &BertEncoder::forwardv2)
        .def("num_layers", &BertEncoder::num_layers)
        .def_pickle(
            [](const c10::intrusive_ptr<BertEncoder>& self) -> std::vector<Tensor> { return self->get_pickle_info(); },
            [](std::vector<Tensor> state) -> c10::intrusive_ptr<BertEncoder> {
              const Tensor info = state.back();
              state.pop_back();
              return c10::make_intrusive<BertEncoder>(info[0].item().to<int64_t>(), info[1].item().to<int64_t>(),
                                                      std::move(state));
            });

}  // namespace bt_th
