// Replays a test case stored in the reference's text format through the C++ class API of
// include/bert_transformer.h.
//
// The reference's flow (unit_test/bert_transformer_test.cc:33-203, unit_test/helper.h:39-85):
//   bert_transformer_test batch_size seq_len head_num size_per_head [data_type] ...
// run in a directory that holds qkv_kernel.in ... from_tensor.in, atten_mask.in and
// transformer_out.out, each with one float per line.  This driver takes the same four leading
// arguments, reads the same files, runs one BertTransformer<HALF>::infer and prints the largest
// and the mean absolute difference to transformer_out.out.
//
//   text_case_driver B S head_num size_per_head [directory=. [fp32_gamma_beta=0 [max_abs_tolerance=-1]]]
//
// It also writes its own result to <directory>/transformer_out.cuda.out in the same format.
// Exit code: 0 ok, 1 usage / missing file, 2 CUDA error, 3 library error, 4 difference above
// max_abs_tolerance (only when a non-negative tolerance is given).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "bert_transformer.h"

using namespace bytetransformer;

namespace {

bool read_floats(const std::string& path, size_t n, std::vector<float>* out) {
  std::FILE* f = std::fopen(path.c_str(), "r");
  if (!f) {
    std::fprintf(stderr, "cannot open %s\n", path.c_str());
    return false;
  }
  out->resize(n);
  size_t got = 0;
  for (; got < n; ++got)
    if (std::fscanf(f, "%f", &(*out)[got]) != 1) break;
  std::fclose(f);
  if (got != n) std::fprintf(stderr, "%s: %zu values, expected %zu\n", path.c_str(), got, n);
  return got == n;
}

// Host floats -> device buffer of fp16 (or fp32 when as_fp32).
void* to_device(const std::vector<float>& v, bool as_fp32) {
  void* d = nullptr;
  if (as_fp32) {
    if (cudaMalloc(&d, v.size() * 4) != cudaSuccess) return nullptr;
    if (cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
    return d;
  }
  std::vector<__half> h(v.size());
  for (size_t i = 0; i < v.size(); ++i) h[i] = __float2half(v[i]);
  if (cudaMalloc(&d, h.size() * 2) != cudaSuccess) return nullptr;
  if (cudaMemcpy(d, h.data(), h.size() * 2, cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
  return d;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 5) {
    std::fprintf(stderr, "usage: %s batch_size seq_len head_num size_per_head [directory [fp32_gamma_beta [max_abs_tol]]]\n",
                 argv[0]);
    return 1;
  }
  const int B = std::atoi(argv[1]), S = std::atoi(argv[2]), nh = std::atoi(argv[3]), hs = std::atoi(argv[4]);
  const std::string dir = argc > 5 ? std::string(argv[5]) + "/" : std::string("./");
  const bool gb32 = argc > 6 && std::atoi(argv[6]) != 0;
  const double tol = argc > 7 ? std::atof(argv[7]) : -1.0;
  if (B <= 0 || S <= 0 || nh <= 0 || hs <= 0) return 1;
  const size_t H = size_t(nh) * hs, F = 4 * H;

  struct Item { const char* file; size_t n; bool fp32; };
  const Item items[12] = {
      {"qkv_kernel.in", H * 3 * H, false}, {"qkv_bias.in", 3 * H, false},
      {"attr_output_kernel.in", H * H, false}, {"attr_output_bias.in", H, false},
      {"attr_output_layernorm_gamma.in", H, gb32}, {"attr_output_layernorm_beta.in", H, gb32},
      {"inter_kernel.in", H * F, false}, {"inter_bias.in", F, false},
      {"output_kernel.in", F * H, false}, {"output_bias.in", H, false},
      {"output_layernorm_gamma.in", H, gb32}, {"output_layernorm_beta.in", H, gb32}};
  void* w[12];
  std::vector<float> tmp;
  for (int i = 0; i < 12; ++i) {
    if (!read_floats(dir + items[i].file, items[i].n, &tmp)) return 1;
    if (!(w[i] = to_device(tmp, items[i].fp32))) return 2;
  }
  if (!read_floats(dir + "from_tensor.in", size_t(B) * S * H, &tmp)) return 1;
  void* x = to_device(tmp, false);
  if (!read_floats(dir + "atten_mask.in", size_t(B) * S * S, &tmp)) return 1;
  void* mask = to_device(tmp, false);
  void* out = nullptr;
  if (!x || !mask || cudaMalloc(&out, size_t(B) * S * H * 2) != cudaSuccess) return 2;

  try {
    BertTransformer<OperationType::HALF> layer(B, nh, hs, S, true, true, gb32);
    BertTransformerParam<OperationType::HALF> p;
    p.attr_kernel_QKV = static_cast<const __half*>(w[0]);
    p.attention_param.attr_bias_QKV = static_cast<const __half*>(w[1]);
    p.attr_output_kernel = static_cast<const __half*>(w[2]);
    p.attr_output_bias = static_cast<const __half*>(w[3]);
    p.attr_output_layernorm_gamma = w[4];
    p.attr_output_layernorm_beta = w[5];
    p.inter_kernel = static_cast<const __half*>(w[6]);
    p.inter_bias = static_cast<const __half*>(w[7]);
    p.output_kernel = static_cast<const __half*>(w[8]);
    p.output_bias = static_cast<const __half*>(w[9]);
    p.output_layernorm_gamma = w[10];
    p.output_layernorm_beta = w[11];
    layer.initialize(p);
    const unsigned long long buf_size = layer.cal_bufsize();
    std::printf("buf_size %llu bytes, %f in MB\n", buf_size, buf_size / 1024.0 / 1024.0);
    void* buf = nullptr;
    if (cudaMalloc(&buf, buf_size) != cudaSuccess) return 2;
    BertTransformerInferParam<__half> ip{static_cast<const __half*>(x), static_cast<const __half*>(mask),
                                         static_cast<__half*>(out), buf, B, S, nullptr, nullptr};
    layer.infer(ip);
    if (cudaDeviceSynchronize() != cudaSuccess) return 2;
  } catch (const std::runtime_error& ex) {
    std::fprintf(stderr, "%s\n", ex.what());
    return 3;
  }

  std::vector<__half> h(size_t(B) * S * H);
  if (cudaMemcpy(h.data(), out, h.size() * 2, cudaMemcpyDeviceToHost) != cudaSuccess) return 2;
  {
    std::FILE* o = std::fopen((dir + "transformer_out.cuda.out").c_str(), "w");
    if (!o) return 1;
    for (size_t i = 0; i < h.size(); ++i) std::fprintf(o, "%f\n", __half2float(h[i]));
    std::fclose(o);
  }
  std::vector<float> want;
  if (!read_floats(dir + "transformer_out.out", h.size(), &want)) {
    std::printf("no transformer_out.out to compare with\n");
    return 0;
  }
  double max_diff = 0.0, sum_diff = 0.0;
  size_t at = 0;
  for (size_t i = 0; i < h.size(); ++i) {
    const double d = std::fabs(double(__half2float(h[i])) - double(want[i]));
    sum_diff += d;
    if (d > max_diff) {
      max_diff = d;
      at = i;
    }
  }
  std::printf("Check with transformer_out.out max_diff %f (at %zu: got %f, expect %f) mean_diff %f\n", max_diff, at,
              __half2float(h[at]), want[at], sum_diff / double(h.size()));
  if (tol >= 0.0 && max_diff > tol) return 4;
  return 0;
}
