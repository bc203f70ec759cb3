// Exercises the C++ host mirror (go-nngpu_b200/host/gonngpu.hpp) the way the
// reference's Go callers use their API.  With no argument it runs the checks
// that need no GPU (shape validation, error text); with "gpu" it also runs the
// device path and compares against plain float64 loops computed here.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>

#include "../../go-nngpu_b200/host/gonngpu.hpp"

static int failures = 0;
#define CHECK(cond)                                                   \
  do {                                                                \
    if (!(cond)) {                                                    \
      std::printf("CHECK failed at line %d: %s\n", __LINE__, #cond);  \
      ++failures;                                                     \
    }                                                                 \
  } while (0)

#define CHECK_LE(value, bound)                                                         \
  do {                                                                                 \
    const double v_ = (value);                                                         \
    if (!(v_ <= (bound))) {                                                            \
      std::printf("CHECK failed at line %d: %s = %g > %g\n", __LINE__, #value, v_, double(bound)); \
      ++failures;                                                                      \
    }                                                                                  \
  } while (0)

static std::vector<double> ref_gemm(const std::vector<float>& A, const std::vector<float>& B, int M,
                                    int K, int N) {
  std::vector<double> C(size_t(M) * N, 0.0);
  for (int i = 0; i < M; ++i)
    for (int k = 0; k < K; ++k)
      for (int j = 0; j < N; ++j) C[size_t(i) * N + j] += double(A[size_t(i) * K + k]) * double(B[size_t(k) * N + j]);
  return C;
}

static double rel_frob(const std::vector<float>& got, const std::vector<double>& ref) {
  double num = 0, den = 0;
  for (size_t i = 0; i < ref.size(); ++i) {
    num += (got[i] - ref[i]) * (got[i] - ref[i]);
    den += ref[i] * ref[i];
  }
  return std::sqrt(num / (den > 0 ? den : 1));
}

static void host_only() {
  // tensor.NewTensor length check and message (tensor/tensor.go:95-97)
  try {
    tensor::NewTensor({2, 3}, std::vector<float>(5));
    CHECK(false);
  } catch (const gonngpu::Error& e) {
    CHECK(std::string(e.what()) == "data length (5) does not match shape dimensions (6)");
  }
  // MatMul shape errors come before any device work (matrix.go:54-59)
  auto a = tensor::NewTensor({2, 3}, std::vector<float>(6));
  auto b = tensor::NewTensor({2, 3}, std::vector<float>(6));
  try {
    matrix::MatMul(a, b);
    CHECK(false);
  } catch (const gonngpu::Error& e) {
    CHECK(std::string(e.what()) ==
          "incompatible matrix dimensions for multiplication: A columns (3) != B rows (2)");
  }
  auto v = tensor::NewTensor({6}, std::vector<float>(6));
  try {
    matrix::Transpose(v);
    CHECK(false);
  } catch (const gonngpu::Error& e) {
    CHECK(std::string(e.what()) == "Transpose requires 2D tensor (matrix)");
  }
  // element-wise family: shape errors and their text (matrix.go:407-427, 551-558, 704-707)
  {
    auto c = tensor::NewTensor({3, 2}, std::vector<float>(6));
    try {
      matrix::Sub(a, c);
      CHECK(false);
    } catch (const gonngpu::Error& e) {
      CHECK(std::string(e.what()) == "incompatible matrix dimensions for subtraction: A (2x3) != B (3x2)");
    }
    try {
      matrix::Add(a, c);
      CHECK(false);
    } catch (const gonngpu::Error& e) {
      CHECK(std::string(e.what()) == "incompatible matrix dimensions for addition: A (2x3) vs B (3x2)");
    }
    try {
      matrix::ScalarMul(v, 2.0f);
      CHECK(false);
    } catch (const gonngpu::Error& e) {
      CHECK(std::string(e.what()) == "ScalarMul requires 2D tensor (matrix)");
    }
    auto t3 = tensor::NewTensor({1, 2, 3}, std::vector<float>(6));
    try {
      matrix::ActivationForward(t3, matrix::Softmax, 0.f);
      CHECK(false);
    } catch (const gonngpu::Error& e) {
      CHECK(std::string(e.what()) == "softmax currently supports only 1D and 2D tensors");
    }
    try {
      matrix::ActivationBackward(a, c, matrix::ReLU, 0.f);
      CHECK(false);
    } catch (const gonngpu::Error& e) {
      CHECK(std::string(e.what()) == "gradient and activation output shape mismatch at dimension 0");
    }
  }
  // gonum-style facade: bounds checks panic (gonum-compat.go:54-56)
  auto g = matrix::NewGPUDense(2, 2, {1, 2, 3, 4});
  CHECK(g->Dims().first == 2 && g->At(1, 0) == 3.0);
  try {
    g->At(2, 0);
    CHECK(false);
  } catch (const gonngpu::Panic&) {
  }
  g->Set(0, 1, 7.5);
  CHECK(g->At(0, 1) == 7.5);
  CHECK(matrix::native_activation_code(matrix::Sigmoid) == 2 &&
        matrix::native_activation_code(matrix::LeakyReLU) == 1);
}

// Host logic of the layer stack, the memory statistics and the precision selectors.
static void host_only_layers() {
  // tensor.go:66-77: nothing allocated yet
  auto st = tensor::GetGlobalMemoryStats();
  CHECK(st.currentUsage == 0 && st.numAllocations == 0);
  tensor::GlobalMemoryPool pool;
  int x = 0, y = 0;
  pool.trackAllocation(&x, 100);
  pool.trackAllocation(&y, 50);
  pool.trackDeallocation(&x);
  pool.trackDeallocation(&x);  // unknown pointers are ignored (tensor.go:59)
  auto ps = pool.GetStats();
  CHECK(ps.currentUsage == 50 && ps.peakUsage == 150 && ps.numAllocations == 1);
  // layers.go:78-80
  auto lin = matrix::NewLinearLayer(4, 3, true);
  CHECK(lin->Weight->Shape[0] == 4 && lin->Weight->Shape[1] == 3 && lin->Bias->Shape[0] == 3);
  const float bound = float(std::sqrt(2.0 / 7.0));
  for (float w : lin->Weight->Data) CHECK(w >= -bound && w <= bound);
  for (float b : lin->Bias->Data) CHECK(b == 0.f);
  CHECK(lin->GetParameters().size() == 2 && matrix::NewLinearLayer(4, 3, false)->GetParameters().size() == 1);
  try {
    lin->Backward(tensor::NewTensor({2, 3}, std::vector<float>(6)));
    CHECK(false);
  } catch (const gonngpu::Panic& e) {
    CHECK(std::string(e.what()) == "Backward called before Forward");
  }
  try {
    matrix::NewReLULayer()->Backward(tensor::NewTensor({2, 3}, std::vector<float>(6)));
    CHECK(false);
  } catch (const gonngpu::Panic& e) {
    CHECK(std::string(e.what()) == "Backward called before Forward");
  }
  // mixed-precision-efficient.go:104-118, mixed-precision-fixed.go:103-124
  CHECK(matrix::EfficientMixedPrecisionTrainer::simulateFloat16Precision(2.f) == 2.f * 0.9999f);
  CHECK(matrix::EfficientMixedPrecisionTrainer::simulateFloat16Precision(1e-5f) == 1e-5f * 0.95f);
  CHECK(matrix::EfficientMixedPrecisionTrainer::simulateFloat16Precision(-70000.f) == -70000.f * 0.999f);
  CHECK(matrix::FixedMixedPrecisionTrainer::fastPrecisionReduction(2.f) == 2.f * 0.99995f);
  CHECK(matrix::FixedMixedPrecisionTrainer::fastPrecisionReduction(-1e-6f) == -1e-6f * 0.995f);
  try {
    matrix::FixedMixedPrecisionTrainer().OptimalMatMul(tensor::NewTensor({2, 3}, std::vector<float>(6)),
                                                       tensor::NewTensor({2, 3}, std::vector<float>(6)));
    CHECK(false);
  } catch (const gonngpu::Error& e) {
    CHECK(std::string(e.what()) == "incompatible matrix dimensions: A[2,3] * B[2,3]");
  }
}

static void with_gpu() {
  std::mt19937 rng(7);
  std::uniform_real_distribution<float> u(-1.f, 1.f);
  const int M = 150, K = 70, N = 90;
  std::vector<float> A(size_t(M) * K), B(size_t(K) * N), bias(N);
  for (auto& x : A) x = u(rng);
  for (auto& x : B) x = u(rng);
  for (auto& x : bias) x = u(rng);
  auto ref = ref_gemm(A, B, M, K, N);

  auto tA = tensor::NewTensor({M, K}, A), tB = tensor::NewTensor({K, N}, B);
  auto tC = matrix::MatMul(tA, tB);
  CHECK(tC->IsOnGPU());
  tC->RetrieveCPU();
  CHECK(rel_frob(tC->Data, ref) <= 1e-5);

  // Transpose twice is the identity, bit for bit
  auto tT = matrix::Transpose(tA);
  auto tTT = matrix::Transpose(tT);
  tTT->RetrieveCPU();
  CHECK(std::memcmp(tTT->Data.data(), A.data(), A.size() * 4) == 0);
  tT->RetrieveCPU();
  CHECK(tT->Shape[0] == K && tT->Data[size_t(3) * M + 5] == A[size_t(5) * K + 3]);

  // backward GEMMs without materialised transposes: (A^T)^T . B == A . B
  auto tC2 = matrix::MatMulTransposed(tT, true, tB, false);
  tC2->RetrieveCPU();
  CHECK(rel_frob(tC2->Data, ref) <= 1e-5);

  // fused linear + bias + ReLU / Sigmoid through the Go-level enum
  auto tBias = tensor::NewTensor({N}, bias);
  matrix::FusedLinearConfig cfg;
  cfg.Bias = true;
  auto y = matrix::FusedLinearActivationForward({tA, tB, tBias}, cfg);  // nil activation = ReLU
  y->RetrieveCPU();
  std::vector<double> want(ref);
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) want[size_t(i) * N + j] = std::max(0.0, want[size_t(i) * N + j] + bias[j]);
  CHECK(rel_frob(y->Data, want) <= 1e-5);
  matrix::FusedActivationConfig sig{matrix::Sigmoid, 0.f};
  cfg.Activation = &sig;
  y = matrix::FusedLinearActivationForward({tA, tB, tBias}, cfg);
  y->RetrieveCPU();
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j)
      want[size_t(i) * N + j] = 1.0 / (1.0 + std::exp(-(ref[size_t(i) * N + j] + bias[j])));
  CHECK(rel_frob(y->Data, want) <= 1e-5);

  // alpha/beta GEMM: the Go wrapper hands in a zeroed C, so beta multiplies zeros
  auto g2 = matrix::OptimizedGEMM(tA, tB, 2.0f, 0.5f);
  g2->RetrieveCPU();
  for (size_t i = 0; i < want.size(); ++i) want[i] = 2.0 * ref[i];
  CHECK(rel_frob(g2->Data, want) <= 1e-5);

  // mixed precision forward
  auto h = matrix::ForwardFloat16(tA, tB);
  h->RetrieveCPU();
  CHECK(rel_frob(h->Data, ref) <= 1e-2);

  // element-wise family and activations through the Go-shaped API
  {
    auto s1 = matrix::Add(tA, tA);                       // equal shapes: element-wise entry
    auto s2 = matrix::Sub(s1, tA);
    s2->RetrieveCPU();
    for (size_t i = 0; i < A.size(); ++i) CHECK(s2->Data[i] == (A[i] + A[i]) - A[i]);
    auto row = tensor::NewTensor({1, K}, std::vector<float>(size_t(K), 0.5f));
    auto s3 = matrix::Add(tA, row);                      // [M,K] + [1,K]: broadcasting entry
    s3->RetrieveCPU();
    CHECK(s3->Data[7] == A[7] + 0.5f);
    auto p = matrix::Mul(tA, tA);
    auto q = matrix::ScalarAdd(matrix::ScalarMul(p, 2.0f), 1.0f);
    q->RetrieveCPU();
    for (size_t i = 0; i < A.size(); i += 97) CHECK(q->Data[i] == (A[i] * A[i]) * 2.0f + 1.0f);
    auto ones = tensor::NewTensor({M, K}, std::vector<float>(A.size(), 1.0f));
    auto d = matrix::Div(tA, ones);
    d->RetrieveCPU();
    CHECK(d->Data[11] == A[11]);
    auto zeros = tensor::NewTensor({M, K}, std::vector<float>(A.size(), 0.0f));
    try {
      matrix::Div(tA, zeros);
      CHECK(false);
    } catch (const gonngpu::Error& e) {
      CHECK(std::string(e.what()) ==
            "GPU matrix element-wise division failed (code -4): Division by zero encountered at element 0.");
    }
    auto sm = matrix::ActivationForward(tA, matrix::Softmax, 0.f);
    sm->RetrieveCPU();
    for (int i = 0; i < M; i += 13) {
      double rs = 0;
      for (int j = 0; j < K; ++j) rs += sm->Data[size_t(i) * K + j];
      CHECK(std::fabs(rs - 1.0) <= 1e-5);
    }
    auto sg = matrix::ActivationForward(tA, matrix::Sigmoid, 0.f);
    auto gsg = matrix::ActivationBackward(ones, sg, matrix::Sigmoid, 0.f);
    sg->RetrieveCPU();
    gsg->RetrieveCPU();
    for (size_t i = 0; i < A.size(); i += 101) {
      const double want = 1.0 / (1.0 + std::exp(-double(A[i])));
      CHECK(std::fabs(sg->Data[i] - want) <= 1e-6);
      CHECK(std::fabs(gsg->Data[i] - want * (1.0 - want)) <= 1e-6);
    }
    auto lk = matrix::ActivationForward(tA, matrix::LeakyReLU, 0.1f);
    lk->RetrieveCPU();
    for (size_t i = 0; i < A.size(); i += 89) CHECK(lk->Data[i] == (A[i] > 0 ? A[i] : 0.1f * A[i]));
  }

  // gonum-style drop-in
  std::vector<double> Ad(A.begin(), A.end()), Bd(B.begin(), B.end());
  auto dA = mat::NewDense(M, K, Ad), dB = mat::NewDense(K, N, Bd);
  auto prod = matrix::GPUMatMul(*dA, *dB);
  std::vector<float> pf(prod->RawData().begin(), prod->RawData().end());
  CHECK(rel_frob(pf, ref) <= 1e-5);
  auto recv = matrix::NewGPUDense(1, 1, {0.0});
  auto gA = matrix::FromGonum(*dA);
  recv->Mul(*gA, *dB);  // one GPUDense operand, one plain matrix
  CHECK(recv->Dims().first == M && recv->Dims().second == N);
  CHECK(std::fabs(recv->At(3, 4) - ref[size_t(3) * N + 4]) <= 1e-4);
  auto back = recv->T()->ToGonum();
  CHECK(back->Dims().first == N && std::fabs(back->At(4, 3) - ref[size_t(3) * N + 4]) <= 1e-4);

  // batched product over 3-D tensors
  {
    const int nb = 3, bm = 40, bk = 50, bn = 24;
    std::vector<float> bA(size_t(nb) * bm * bk), bB(size_t(nb) * bk * bn);
    for (auto& x : bA) x = u(rng);
    for (auto& x : bB) x = u(rng);
    auto tbA = tensor::NewTensor({nb, bm, bk}, bA), tbB = tensor::NewTensor({nb, bk, bn}, bB);
    auto tbC = matrix::OptimizedBatchMatMul(tbA, tbB);
    tbC->RetrieveCPU();
    for (int b = 0; b < nb; ++b) {
      std::vector<float> a1(bA.begin() + size_t(b) * bm * bk, bA.begin() + size_t(b + 1) * bm * bk);
      std::vector<float> b1(bB.begin() + size_t(b) * bk * bn, bB.begin() + size_t(b + 1) * bk * bn);
      std::vector<float> c1(tbC->Data.begin() + size_t(b) * bm * bn, tbC->Data.begin() + size_t(b + 1) * bm * bn);
      CHECK(rel_frob(c1, ref_gemm(a1, b1, bm, bk, bn)) <= 1e-5);
    }
    try {
      matrix::OptimizedBatchMatMul(tA, tB);
      CHECK(false);
    } catch (const gonngpu::Error& e) {
      CHECK(std::string(e.what()) == "batch matrix multiplication requires 3D tensors");
    }
  }

  // linear layer backward in one call, with the ReLU mask of the layer's output
  {
    std::vector<float> dY(size_t(M) * N), act(size_t(M) * N);
    for (auto& x : dY) x = u(rng);
    for (auto& x : act) x = std::max(0.f, u(rng));
    auto tdY = tensor::NewTensor({M, N}, dY), tact = tensor::NewTensor({M, N}, act);
    auto g = matrix::LinearBackward(tA, tB, tdY, tact);
    g.Input->RetrieveCPU();
    g.Weight->RetrieveCPU();
    g.Bias->RetrieveCPU();
    std::vector<double> dAct(size_t(M) * N), dW(size_t(K) * N, 0.0), dX(size_t(M) * K, 0.0), dbias(N, 0.0);
    for (size_t i = 0; i < dAct.size(); ++i) dAct[i] = act[i] > 0.f ? dY[i] : 0.0;
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) {
        const double gv = dAct[size_t(i) * N + j];
        dbias[j] += gv;
        for (int k = 0; k < K; ++k) {
          dW[size_t(k) * N + j] += double(A[size_t(i) * K + k]) * gv;
          dX[size_t(i) * K + k] += gv * double(B[size_t(k) * N + j]);
        }
      }
    CHECK(rel_frob(g.Weight->Data, dW) <= 1e-5);
    CHECK(rel_frob(g.Input->Data, dX) <= 1e-5);
    CHECK(rel_frob(g.Bias->Data, dbias) <= 1e-5);
  }

  // modifying Data after RetrieveCPU is seen by the next device op (aliasing
  // semantics the eager layers rely on, layers.go:271-279)
  tC->Data[0] = 1234.0f;
  auto again = matrix::Transpose(tC);
  again->RetrieveCPU();
  CHECK(again->Data[0] == 1234.0f);
}

// float64 reference of Y = X.W + b (optionally ReLU) on the host.
static std::vector<double> ref_linear(const std::vector<float>& X, const std::vector<float>& W,
                                      const std::vector<float>& b, int M, int K, int N, bool relu) {
  auto Y = ref_gemm(X, W, M, K, N);
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      double v = Y[size_t(i) * N + j] + (b.empty() ? 0.0 : double(b[j]));
      Y[size_t(i) * N + j] = relu ? std::max(v, 0.0) : v;
    }
  return Y;
}
static std::vector<float> narrow(const std::vector<double>& v) { return std::vector<float>(v.begin(), v.end()); }

// The MLP training step of the benchmark configurations (batch 512, 784 -> 1024 -> 1024 -> 10,
// ReLU after the first two layers) driven through the layer stack a caller of the
// reference uses (layers.go: Sequential of LinearLayer / ReLULayer), fused and unfused,
// against float64 loops.
static void mlp_step_through_layers(bool fuse) {
  const int batch = 512, d0 = 784, d1 = 1024, d2 = 1024, d3 = 10;
  std::mt19937 rng(2);
  std::uniform_real_distribution<float> u01(0.f, 1.f);
  std::normal_distribution<float> n01(0.f, 1.f);
  auto l1 = matrix::NewLinearLayer(d0, d1, true, 11), l2 = matrix::NewLinearLayer(d1, d2, true, 12),
       l3 = matrix::NewLinearLayer(d2, d3, true, 13);
  // He-normal weights, small non-zero biases (so that a lost bias would show)
  for (auto* l : {l1.get(), l2.get(), l3.get()}) {
    const float sd = float(std::sqrt(2.0 / l->InputSize));
    for (auto& w : l->Weight->Data) w = n01(rng) * sd;
    for (auto& b : l->Bias->Data) b = 0.1f * n01(rng);
  }
  matrix::Sequential net({l1, matrix::NewReLULayer(), l2, matrix::NewReLULayer(), l3}, fuse);
  std::vector<float> X(size_t(batch) * d0), dY(size_t(batch) * d3);
  for (auto& x : X) x = u01(rng);
  for (auto& g : dY) g = 1e-2f * n01(rng);
  auto tX = tensor::NewTensor({batch, d0}, X);
  auto out = net.Forward(tX);
  auto gin = net.Backward(tensor::NewTensor({batch, d3}, dY));
  out->RetrieveCPU();
  gin->RetrieveCPU();

  auto h1 = ref_linear(X, l1->Weight->Data, l1->Bias->Data, batch, d0, d1, true);
  auto h1f = narrow(h1);
  auto h2 = ref_linear(h1f, l2->Weight->Data, l2->Bias->Data, batch, d1, d2, true);
  auto h2f = narrow(h2);
  auto y = ref_linear(h2f, l3->Weight->Data, l3->Bias->Data, batch, d2, d3, false);
  CHECK(out->Shape[0] == batch && out->Shape[1] == d3);
  CHECK_LE(rel_frob(out->Data, y), 1e-5);
  // The ReLU derivative is a step: a pre-activation within rounding of zero may be masked on
  // the device and not in float64 (one such element moves a gradient by ~1e-3 of its norm).
  // The reference backward therefore takes its masks from the device's own activations,
  // obtained by running the same layers one by one, after checking them against float64.
  matrix::ReLULayer r1, r2;
  auto h1dev = r1.Forward(l1->Forward(tX));
  auto h2dev = r2.Forward(l2->Forward(h1dev));
  h1dev->RetrieveCPU();
  h2dev->RetrieveCPU();
  CHECK_LE(rel_frob(h1dev->Data, h1), 1e-5);
  CHECK_LE(rel_frob(h2dev->Data, h2), 1e-5);
  size_t flips = 0;
  for (size_t i = 0; i < h1.size(); ++i) flips += (h1dev->Data[i] > 0) != (h1[i] > 0);
  for (size_t i = 0; i < h2.size(); ++i) flips += (h2dev->Data[i] > 0) != (h2[i] > 0);
  CHECK(flips <= 8);  // only elements at rounding distance from zero may differ
  std::vector<char> on1(h1.size()), on2(h2.size());  // the derivative the device applies
  for (size_t i = 0; i < h1.size(); ++i) on1[i] = h1dev->Data[i] > 0;
  for (size_t i = 0; i < h2.size(); ++i) on2[i] = h2dev->Data[i] > 0;
  (void)net.Forward(tX);  // the layers' caches belong to the net's own forward pass again
  gin = net.Backward(tensor::NewTensor({batch, d3}, dY));
  gin->RetrieveCPU();

  // backward in float64: g3 = dY; dW3 = h2^T g3; g2 = (g3 W3^T) masked by h2 > 0; ...
  auto backward = [&](const std::vector<double>& g, const std::vector<double>& in, const std::vector<float>& W,
                      int M, int K, int N, std::vector<double>& dW, std::vector<double>& db,
                      std::vector<double>& dX) {
    dW.assign(size_t(K) * N, 0.0);
    db.assign(N, 0.0);
    dX.assign(size_t(M) * K, 0.0);
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) {
        const double gv = g[size_t(i) * N + j];
        if (gv == 0.0) continue;
        db[j] += gv;
        for (int k = 0; k < K; ++k) {
          dW[size_t(k) * N + j] += in[size_t(i) * K + k] * gv;
          dX[size_t(i) * K + k] += gv * double(W[size_t(k) * N + j]);
        }
      }
  };
  std::vector<double> g3(dY.begin(), dY.end()), dW3, db3, dX3, dW2, db2, dX2, dW1, db1, dX1;
  std::vector<double> Xd(X.begin(), X.end());
  backward(g3, h2, l3->Weight->Data, batch, d2, d3, dW3, db3, dX3);
  for (size_t i = 0; i < dX3.size(); ++i)
    if (!on2[i]) dX3[i] = 0.0;
  backward(dX3, h1, l2->Weight->Data, batch, d1, d2, dW2, db2, dX2);
  for (size_t i = 0; i < dX2.size(); ++i)
    if (!on1[i]) dX2[i] = 0.0;
  backward(dX2, Xd, l1->Weight->Data, batch, d0, d1, dW1, db1, dX1);
  auto grads = net.GetGradients();
  CHECK(grads.size() == 6);
  const std::vector<double>* refs[6] = {&dW1, &db1, &dW2, &db2, &dW3, &db3};
  for (int i = 0; i < 6; ++i) {
    grads[i]->RetrieveCPU();
    CHECK(grads[i]->Data.size() == refs[i]->size());
    CHECK_LE(rel_frob(grads[i]->Data, *refs[i]), 1e-5);
  }
  CHECK_LE(rel_frob(gin->Data, dX1), 1e-5);
  CHECK(net.GetParameters().size() == 6);
}

static void layers_stats_unified_selectors() {
  std::mt19937 rng(9);
  std::uniform_real_distribution<float> u(-1.f, 1.f);
  // The bias a LinearLayer adds must be what a following device operation reads: the
  // reference adds it into the host slice after the product (layers.go:271-279), which
  // a discrete GPU's buffer would never see.
  {
    const int M = 33, K = 20, N = 17;
    auto lin = matrix::NewLinearLayer(K, N, true, 5);
    for (auto& b : lin->Bias->Data) b = 3.0f + u(rng);
    std::vector<float> X(size_t(M) * K);
    for (auto& x : X) x = u(rng);
    auto y = lin->Forward(tensor::NewTensor({M, K}, X));
    CHECK(y->IsOnGPU());
    auto yT = matrix::Transpose(y);  // reads the device copy
    yT->RetrieveCPU();
    y->RetrieveCPU();
    auto ref = ref_linear(X, lin->Weight->Data, lin->Bias->Data, M, K, N, false);
    CHECK(rel_frob(y->Data, ref) <= 1e-5);
    bool same = true;
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) same = same && yT->Data[size_t(j) * M + i] == y->Data[size_t(i) * N + j];
    CHECK(same);
  }
  // tensor.go:22-77: EnsureGPU / ReleaseGPU move the global statistics
  {
    const auto before = tensor::GetGlobalMemoryStats();
    auto t = tensor::NewTensor({8, 16}, std::vector<float>(128, 1.f));
    t->EnsureGPU();
    auto mid = tensor::GetGlobalMemoryStats();
    CHECK(mid.currentUsage == before.currentUsage + 512 && mid.numAllocations == before.numAllocations + 1);
    CHECK(mid.peakUsage >= mid.currentUsage);
    t->ReleaseGPU();
    auto after = tensor::GetGlobalMemoryStats();
    CHECK(after.currentUsage == before.currentUsage && after.numAllocations == before.numAllocations);
    CHECK(after.peakUsage == mid.peakUsage);
  }
  // matrix.go:19-50 + tensor-unified-memory.go: with a global device MatMul runs on unified buffers
  {
    const int M = 40, K = 24, N = 56;
    std::vector<float> A(size_t(M) * K), B(size_t(K) * N);
    for (auto& x : A) x = u(rng);
    for (auto& x : B) x = u(rng);
    auto tA = tensor::NewTensor({M, K}, A), tB = tensor::NewTensor({K, N}, B);
    tA->EnsureGPU();
    DevicePtr dev = tA->DevicePointer();
    CHECK(dev != nullptr);
    matrix::SetGlobalMatrixDevice(dev);
    auto& ad = matrix::GetGlobalTensorAdapter(dev);
    auto tC = matrix::MatMul(tA, tB);
    CHECK(ad.NumBuffers() == 3 && ad.GetUnifiedGPUBuffer(tC) != nullptr);
    CHECK(!tC->IsOnGPU());  // the tensor's own buffer was never made (as in the reference)
    const float* c = ad.GetUnifiedCPUData(tC);
    CHECK(c != nullptr);
    std::vector<float> got(c, c + size_t(M) * N);
    CHECK(rel_frob(got, ref_gemm(A, B, M, K, N)) <= 1e-5);
    const long hits = ad.ZeroCopyHits();
    ad.EnsureUnifiedGPU(tA);  // already there: counted as a hit, no second buffer
    CHECK(ad.ZeroCopyHits() == hits + 1 && ad.NumBuffers() == 3);
    for (auto& t : {tA, tB, tC}) ad.ReleaseUnifiedBuffer(t);
    CHECK(ad.NumBuffers() == 0 && ad.GetUnifiedGPUBuffer(tA) == nullptr);
    matrix::SetGlobalMatrixDevice(nullptr);
    auto tC2 = matrix::MatMul(tA, tB);  // back on the tensors' own buffers
    tC2->RetrieveCPU();
    CHECK(rel_frob(tC2->Data, ref_gemm(A, B, M, K, N)) <= 1e-5);
  }
  // precision selectors: which path a size takes, and what it returns
  {
    auto mk = [&](int r, int c) {
      std::vector<float> v(size_t(r) * c);
      for (auto& x : v) x = u(rng);
      return tensor::NewTensor({r, c}, v);
    };
    auto a = mk(64, 48), b = mk(48, 32);
    auto ref = ref_gemm(a->Data, b->Data, 64, 48, 32);
    auto scaled = [&](double f) {
      auto r = ref;
      for (auto& x : r) x *= f;
      return r;
    };
    auto e = matrix::EfficientMixedPrecisionTrainer().EfficientMatMul(a, b);  // small: scaled on the host
    CHECK(!e->IsOnGPU() && rel_frob(e->Data, scaled(0.9999)) <= 2e-5);
    auto f = matrix::FixedMixedPrecisionTrainer().OptimalMatMul(a, b);
    CHECK(!f->IsOnGPU() && rel_frob(f->Data, scaled(0.99995)) <= 2e-5);
    auto z = matrix::ZeroCopyMixedPrecisionOps().OptimalMatMul(a, b);
    CHECK(rel_frob(z->Data, scaled(0.9999)) <= 2e-5);
    auto o = matrix::OptimizedMixedPrecisionOps().MatMulOptimized(a, b);  // fp16 inputs, fp32 sums
    o->RetrieveCPU();
    CHECK(rel_frob(o->Data, ref) <= 1e-2 && rel_frob(o->Data, ref) > 1e-6);
    matrix::MixedPrecisionConfig off;
    off.Enabled = false;
    auto p = matrix::OptimizedMixedPrecisionOps(off).MatMulOptimized(a, b);  // disabled: plain MatMul
    p->RetrieveCPU();
    CHECK(rel_frob(p->Data, ref) <= 1e-5);
    auto big_a = mk(300, 600), big_b = mk(600, 300);  // above every threshold: float32 path
    auto big = matrix::FixedMixedPrecisionTrainer().OptimalMatMul(big_a, big_b);
    CHECK(big->IsOnGPU());
    big->RetrieveCPU();
    CHECK(rel_frob(big->Data, ref_gemm(big_a->Data, big_b->Data, 300, 600, 300)) <= 1e-5);
  }
  // the sharded form of ForwardFloat16 against the one-device form and the float64 loops
  {
    const int M = 9000, K = 96, N = 136;
    std::vector<float> A(size_t(M) * K), B(size_t(K) * N);
    for (auto& x : A) x = u(rng);
    for (auto& x : B) x = u(rng);
    auto tA = tensor::NewTensor({M, K}, A), tB = tensor::NewTensor({K, N}, B);
    auto one = matrix::ForwardFloat16(tA, tB);
    one->RetrieveCPU();
    auto all = matrix::ForwardFloat16Sharded(tA, tB, 0);
    auto first = matrix::ForwardFloat16Sharded(tA, tB, 1);
    CHECK(!all->IsOnGPU() && all->Data.size() == one->Data.size());
    CHECK_LE(rel_frob(all->Data, std::vector<double>(one->Data.begin(), one->Data.end())), 1e-6);
    CHECK_LE(rel_frob(first->Data, std::vector<double>(all->Data.begin(), all->Data.end())), 1e-6);
    CHECK_LE(rel_frob(all->Data, ref_gemm(A, B, M, K, N)), 1e-2);
  }
  // GradFusedLinearActivation: forward through the fused kernel, backward with the right mask
  {
    const int M = 30, K = 12, N = 20;
    auto mkg = [&](std::vector<int> shape, bool grad) {
      size_t n = 1;
      for (int d : shape) n *= size_t(d);
      std::vector<float> v(n);
      for (auto& x : v) x = u(rng);
      auto g = std::make_shared<matrix::GradientTensor>();
      g->Tensor = tensor::NewTensor(shape, v);
      g->RequiresGrad = grad;
      return g;
    };
    auto x = mkg({M, K}, false), w = mkg({K, N}, true), b = mkg({N}, true);
    matrix::FusedLinearConfig cfg;
    cfg.Bias = true;  // nil Activation means ReLU (fused-operations.go:433)
    auto out = matrix::GradFusedLinearActivation(x, w, b, cfg);
    CHECK(out->RequiresGrad && !out->IsLeaf && bool(out->BackwardFn));
    std::vector<float> dY(size_t(M) * N);
    for (auto& v : dY) v = u(rng);
    auto grads = out->BackwardFn(tensor::NewTensor({M, N}, dY));
    CHECK(grads.size() == 3);
    out->Tensor->RetrieveCPU();
    auto y = ref_linear(x->Tensor->Data, w->Tensor->Data, b->Tensor->Data, M, K, N, true);
    CHECK(rel_frob(out->Tensor->Data, y) <= 1e-5);
    std::vector<double> dW(size_t(K) * N, 0.0), db(N, 0.0);
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) {
        if (!(y[size_t(i) * N + j] > 0)) continue;
        db[j] += dY[size_t(i) * N + j];
        for (int k = 0; k < K; ++k) dW[size_t(k) * N + j] += double(x->Tensor->Data[size_t(i) * K + k]) * dY[size_t(i) * N + j];
      }
    grads[1]->RetrieveCPU();
    grads[2]->RetrieveCPU();
    CHECK(rel_frob(grads[1]->Data, dW) <= 1e-5 && rel_frob(grads[2]->Data, db) <= 1e-5);
  }
}

int main(int argc, char** argv) {
  host_only();
  host_only_layers();
  if (argc > 1 && std::strcmp(argv[1], "gpu") == 0) {
    try {
      with_gpu();
      layers_stats_unified_selectors();
      mlp_step_through_layers(true);
      mlp_step_through_layers(false);
    } catch (const std::exception& e) {
      std::printf("exception: %s\n", e.what());
      ++failures;
    }
  }
  std::printf(failures ? "FAILED (%d)\n" : "host mirror ok\n", failures);
  return failures ? 1 : 0;
}
