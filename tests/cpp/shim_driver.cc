// Test driver for include/bert_transformer.h, in the spirit of the reference's
// unit_test/bert_transformer_test.cc: loads tensors from a file, runs one
// BertTransformer<HALF>::infer through the class API, writes the output back.
//
// File format (little endian): int32 B, S, head_num, use_fp32; then the 12 weights
// in the reference's order, input [B,S,H], mask [B,S,S] — fp16 raw, except
// LayerNorm gamma/beta which are fp32 when use_fp32 != 0.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "bert_transformer.h"

using namespace bytetransformer;

#define CK(x)                                                                   \
  do {                                                                          \
    cudaError_t e_ = (x);                                                       \
    if (e_ != cudaSuccess) {                                                    \
      std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));           \
      return 2;                                                                 \
    }                                                                           \
  } while (0)

static void* upload(std::FILE* f, size_t bytes) {
  std::vector<char> h(bytes);
  if (std::fread(h.data(), 1, bytes, f) != bytes) return nullptr;
  void* d = nullptr;
  if (cudaMalloc(&d, bytes) != cudaSuccess) return nullptr;
  cudaMemcpy(d, h.data(), bytes, cudaMemcpyHostToDevice);
  return d;
}

int main(int argc, char** argv) {
  if (argc == 2 && std::string(argv[1]) == "--link-check") {
    // No device needed: the class must compile, link and report errors as exceptions.
    try {
      BertTransformer<OperationType::HALF> t(4, 12, 64, 64);
      BertTransformerParam<OperationType::HALF> p;
      t.initialize(p);
      std::printf("initialized (a device is present)\n");
    } catch (const std::runtime_error& e) {
      std::printf("runtime_error: %s\n", e.what());
    }
    try {
      BertTransformer<OperationType::FP32> t32(4, 12, 64, 64);
      std::printf("unexpected: FP32 accepted\n");
      return 1;
    } catch (const std::runtime_error& e) {
      std::printf("FP32 rejected: %s\n", e.what());
    }
    return 0;
  }
  if (argc != 3) {
    std::fprintf(stderr, "usage: %s in.bin out.bin | --link-check\n", argv[0]);
    return 1;
  }
  std::FILE* f = std::fopen(argv[1], "rb");
  if (!f) return 1;
  int hdr[4];
  if (std::fread(hdr, 4, 4, f) != 4) return 1;
  const int B = hdr[0], S = hdr[1], nh = hdr[2], fp32gb = hdr[3];
  const size_t H = size_t(nh) * 64, F = 4 * H;
  const size_t e = 2, g = fp32gb ? 4 : 2;
  const size_t sizes[12] = {H * 3 * H * e, 3 * H * e, H * H * e, H * e, H * g, H * g,
                            H * F * e,     F * e,     F * H * e, H * e, H * g, H * g};
  void* w[12];
  for (int i = 0; i < 12; ++i)
    if (!(w[i] = upload(f, sizes[i]))) return 2;
  void* x = upload(f, size_t(B) * S * H * e);
  void* mask = upload(f, size_t(B) * S * S * e);
  std::fclose(f);
  if (!x || !mask) return 2;
  void* out = nullptr;
  CK(cudaMalloc(&out, size_t(B) * S * H * e));

  try {
    BertTransformer<OperationType::HALF> layer(B, nh, 64, S, true, true, fp32gb != 0);
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
    void* buf = nullptr;
    CK(cudaMalloc(&buf, buf_size));
    cudaStream_t stream;
    CK(cudaStreamCreate(&stream));
    BertTransformerInferParam<__half> ip{static_cast<const __half*>(x), static_cast<const __half*>(mask),
                                         static_cast<__half*>(out), buf, B, S, nullptr, stream};
    layer.infer(ip);
    layer.infer(ip);  // the object is reusable across calls
    CK(cudaStreamSynchronize(stream));
  } catch (const std::runtime_error& ex) {
    std::fprintf(stderr, "%s\n", ex.what());
    return 3;
  }
  std::vector<char> h(size_t(B) * S * H * e);
  CK(cudaMemcpy(h.data(), out, h.size(), cudaMemcpyDeviceToHost));
  std::FILE* o = std::fopen(argv[2], "wb");
  if (!o) return 1;
  std::fwrite(h.data(), 1, h.size(), o);
  std::fclose(o);
  return 0;
}
