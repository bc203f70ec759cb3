// Times the MLP training step of the benchmark configurations (batch 512,
// 784 -> 1024 -> 1024 -> 10, ReLU after the first two layers, forward + backward) as a caller
// of the layer stack drives it: matrix::Sequential of LinearLayer / ReLULayer from gonngpu.hpp,
// result tensors made and released per operation, blocking calls.  Prints one JSON line.
//
//   g++ -std=c++17 -O2 -o mlp_step mlp_step.cpp -L.. -lgonngpu_cuda -Wl,-rpath,..
//   ./mlp_step [steps] [fuse: 1|0]
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>

#include "gonngpu.hpp"

int main(int argc, char** argv) {
  const int steps = argc > 1 ? std::atoi(argv[1]) : 200;
  const bool fuse = argc > 2 ? std::atoi(argv[2]) != 0 : true;
  const int batch = 512, d0 = 784, d1 = 1024, d2 = 1024, d3 = 10;
  try {
    std::mt19937 rng(2);
    std::uniform_real_distribution<float> u01(0.f, 1.f);
    std::normal_distribution<float> n01(0.f, 1.f);
    auto l1 = matrix::NewLinearLayer(d0, d1, true, 11), l2 = matrix::NewLinearLayer(d1, d2, true, 12),
         l3 = matrix::NewLinearLayer(d2, d3, true, 13);
    for (auto* l : {l1.get(), l2.get(), l3.get()}) {
      const float sd = float(std::sqrt(2.0 / l->InputSize));
      for (auto& w : l->Weight->Data) w = n01(rng) * sd;
    }
    matrix::Sequential net({l1, matrix::NewReLULayer(), l2, matrix::NewReLULayer(), l3}, fuse);
    std::vector<float> X(size_t(batch) * d0), dY(size_t(batch) * d3);
    for (auto& x : X) x = u01(rng);
    for (auto& g : dY) g = 1e-2f * n01(rng);
    auto tX = tensor::NewTensor({batch, d0}, X);
    auto tdY = tensor::NewTensor({batch, d3}, dY);
    gonngpu_set_blocking(0);  // calls are enqueued; one wait per step, as a training loop that reads its loss
    for (int i = 0; i < 10; ++i) {
      net.Forward(tX);
      net.Backward(tdY);
    }
    CError err{nullptr};
    gonngpu_synchronize(&err);
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < steps; ++i) {
      net.Forward(tX);
      net.Backward(tdY);
      gonngpu_synchronize(&err);
    }
    const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / steps;
    gonngpu_set_blocking(1);
    const double flops = 3 * 2.0 * batch * (double(d0) * d1 + double(d1) * d2 + double(d2) * d3);
    std::printf("{\"op\": \"c3 MLP step through Sequential (C++ mirror of the layer stack), %s\", \"us\": %.2f, "
                "\"tflops\": %.2f, \"steps\": %d}\n",
                fuse ? "Linear+ReLU pairs fused" : "unfused", us, flops / us / 1e6, steps);
  } catch (const std::exception& e) {
    std::printf("{\"error\": \"%s\"}\n", e.what());
    return 1;
  }
  return 0;
}
