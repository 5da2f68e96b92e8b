// Drives the operator through the C++ host mirror (ttt_rs_b200/host/fused_tile_multi.hpp) the way a compiled-code
// caller would: inputs from raw files, device buffers from a cudaMalloc-backed allocator, forward_launch +
// backward_launch, outputs back to raw files.  tests/test_cpp_host_gpu.py compares them with the ctypes path.
//   usage: host_mirror_roundtrip <dir> B H T K      (bf16 tensors as raw little-endian files in <dir>)
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <string>
#include <vector>

#include "ttt_rs_b200/host/fused_tile_multi.hpp"

using namespace ttt_b200;

struct CudaAllocator : Allocator {
  std::vector<void*> live;
  void* alloc(size_t bytes) override {
    void* p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) return nullptr;
    live.push_back(p);
    return p;
  }
  void free(void*) override {}  // released together at exit: nothing here reuses memory while work is queued
  ~CudaAllocator() override {
    for (void* p : live) cudaFree(p);
  }
};

static std::vector<char> read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) {
    std::fprintf(stderr, "cannot open %s\n", path.c_str());
    std::exit(2);
  }
  return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}
static DeviceTensor upload(CudaAllocator& a, const std::string& path, std::vector<int64_t> shape, int dtype) {
  DeviceTensor t = empty(a, std::move(shape), dtype);
  const std::vector<char> h = read_file(path);
  if (h.size() != t.bytes()) {
    std::fprintf(stderr, "%s: %zu bytes, expected %zu\n", path.c_str(), h.size(), t.bytes());
    std::exit(2);
  }
  cudaMemcpy(t.ptr, h.data(), h.size(), cudaMemcpyHostToDevice);
  return t;
}
static void download(const DeviceTensor& t, const std::string& path) {
  std::vector<char> h(t.bytes());
  cudaMemcpy(h.data(), t.ptr, h.size(), cudaMemcpyDeviceToHost);
  std::ofstream(path, std::ios::binary).write(h.data(), (std::streamsize)h.size());
}

int main(int argc, char** argv) {
  if (argc != 6) return 2;
  const std::string dir = argv[1];
  const int64_t B = std::atoll(argv[2]), H = std::atoll(argv[3]), T = std::atoll(argv[4]);
  const int K = std::atoi(argv[5]);
  const int64_t F = 64;
  CudaAllocator a;
  TttInputs in;
  in.xq = upload(a, dir + "/xq.bin", {B, H, T, F}, TTT_BF16);
  in.xk = upload(a, dir + "/xk.bin", {B, H, T, F}, TTT_BF16);
  in.xv = upload(a, dir + "/xv.bin", {B, H, T, F}, TTT_BF16);
  in.weight = upload(a, dir + "/weight.bin", {B, H, F, F}, TTT_BF16);
  in.bias = upload(a, dir + "/bias.bin", {B, H, F}, TTT_BF16);
  in.token_eta = upload(a, dir + "/token_eta.bin", {T}, TTT_BF16);
  in.ttt_lr_eta = upload(a, dir + "/ttt_lr_eta.bin", {B, H, T}, TTT_BF16);
  in.ln_weight = upload(a, dir + "/ln_weight.bin", {H, F}, TTT_BF16);
  in.ln_bias = upload(a, dir + "/ln_bias.bin", {H, F}, TTT_BF16);
  TttOutputs gout;
  gout.output = upload(a, dir + "/grad_output.bin", {B, H, T, F}, TTT_BF16);

  FusedTttConfig cfg = FusedTttConfig::make(16, 64, 1e-6f, 128);
  cfg.checkpoint_interval = K;
  try {
    auto fw = TttTileMultiKernel::forward_launch(in, cfg, a, nullptr);
    TttInputs g = TttTileMultiKernel::backward_launch(fw.second, gout, cfg, a, nullptr);
    if (cudaDeviceSynchronize() != cudaSuccess) {
      std::fprintf(stderr, "CUDA error: %s\n", cudaGetErrorString(cudaGetLastError()));
      return 1;
    }
    download(fw.first.output, dir + "/out_output.bin");
    download(fw.first.weight, dir + "/out_weight.bin");
    download(g.xq, dir + "/out_grad_xq.bin");
    download(g.xk, dir + "/out_grad_xk.bin");
    download(g.xv, dir + "/out_grad_xv.bin");
    download(g.weight, dir + "/out_grad_weight.bin");
    download(g.token_eta, dir + "/out_grad_token_eta.bin");
    // an unsupported tile configuration must throw, like the reference's panic
    FusedTttConfig bad = cfg;
    bad.mini_batch_len = 32;  // (16 and 8 are built)
    bool threw = false;
    try {
      TttTileMultiKernel::forward_launch(in, bad, a, nullptr);
    } catch (const std::runtime_error&) {
      threw = true;
    }
    if (!threw) return 3;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "%s\n", e.what());
    return 1;
  }
  std::puts("ok");
  return 0;
}
