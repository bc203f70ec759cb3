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

int main(int argc, char** argv) {
  host_only();
  if (argc > 1 && std::strcmp(argv[1], "gpu") == 0) {
    try {
      with_gpu();
    } catch (const std::exception& e) {
      std::printf("exception: %s\n", e.what());
      ++failures;
    }
  }
  std::printf(failures ? "FAILED (%d)\n" : "host mirror ok\n", failures);
  return failures ? 1 : 0;
}
