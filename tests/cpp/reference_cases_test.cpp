// GPU tests through the C++ operator API: the reference's own known-answer cases
// for the quantized-matmul path, replayed as its tests call them
// (tests/harness/OpRegistry.h:1929-1957, 1995-2192; tests/runtime/RuntimeTests.cpp:2861-2938;
// tests/runtime/OpCoverageTests.cpp:255-277), plus the raw-GGUF-block entry point
// against the CPU checker (oracle/cut_oracle.c, linked here as the checker only).
#include <cstdint>
#include <random>

#include "check.h"
#include "cut_api.h"
#include "gguf_upload.h"
#include "gguf_writer.h"

using namespace cut;

extern "C" {
// CPU checker (test infrastructure)
void orc_qmatmul_blocks(int fmt, const float *A, const uint8_t *W, float *C, const float *D, size_t M, size_t K, size_t N,
                        size_t lda, size_t ldc, size_t ldd, int fusion_type, int fusion_op, int acc64);
void orc_dequant_rows(int fmt, const uint8_t *data, float *out, size_t rows, size_t cols, size_t ldo);
uint16_t orc_f32_to_f16_trunc(float v);
uint16_t orc_f32_to_f16_runner(float v);
void orc_rmsnorm(const float *x, const float *weight, float *y, size_t rows, size_t dim, size_t ldx, float eps);
float orc_argreduce(const float *v, size_t n, int is_max);
void orc_rope_kv_write(int kv_half, const float *q, const float *k, const float *v, uint32_t pos, const float *cos_t, const float *sin_t,
                       void *k_cache, void *v_cache, float *q_out, size_t q_dim, size_t kv_dim, size_t head_dim, size_t ld);
void orc_attention(int kv_half, const float *q, const void *k_cache, const void *v_cache, size_t seq_len, float *out, size_t n_heads,
                   size_t n_kv_heads, size_t head_dim, size_t ld, float scale);
}

namespace {

uint16_t f32_to_f16(float v) { return orc_f32_to_f16_trunc(v); }  // tests/harness/OpRefs.h:164-177
uint8_t packNibbles(uint8_t lo, uint8_t hi) { return (lo & 0xFu) | ((hi & 0xFu) << 4); }

std::vector<float> generateTestData(size_t count, uint32_t seed = 42) {  // tests/harness/OpRefs.h:241-266
  std::mt19937 gen(seed);
  std::uniform_real_distribution<float> dist(0.1f, 10.0f);
  std::vector<float> v(count);
  for (auto &x : v) x = dist(gen);
  return v;
}

Runtime *rt = nullptr;

void q8Simple() {
  const uint32_t M = 1, K = 32, N = 2, blocksK = K / 32;
  std::vector<float> dataA(M * K, 1.0f);
  std::vector<int8_t> dataB(K * N);
  for (uint32_t k = 0; k < K; ++k) { dataB[k * N + 0] = 1; dataB[k * N + 1] = 2; }
  std::vector<uint16_t> scales(blocksK * N, f32_to_f16(1.0f));
  auto bufA = rt->createTensor({M, K}, DataType::Float32, dataA.data());
  auto bufB = rt->createTensor({K, N}, DataType::Int8, dataB.data());
  auto bufS = rt->createTensor({blocksK, N}, DataType::Float16, scales.data());
  auto bufC = rt->ops().matmul(bufA, bufB, bufS);
  std::vector<float> out(M * N);
  rt->copyFromTensor(bufC, out.data(), M * N * sizeof(float));
  CHECK_NEAR(out[0], 32.0f, 1e-3f);
  CHECK_NEAR(out[1], 64.0f, 1e-3f);
}

void q8WithScales() {
  const uint32_t M = 1, K = 64, N = 2, blocksK = K / 32;
  std::vector<float> dataA(M * K, 1.0f);
  std::vector<int8_t> dataB(K * N, 4);
  std::vector<uint16_t> scales = {f32_to_f16(0.5f), f32_to_f16(2.0f), f32_to_f16(1.0f), f32_to_f16(0.25f)};
  auto bufC = rt->ops().matmul(rt->createTensor({M, K}, DataType::Float32, dataA.data()),
                               rt->createTensor({K, N}, DataType::Int8, dataB.data()),
                               rt->createTensor({blocksK, N}, DataType::Float16, scales.data()));
  std::vector<float> out(M * N);
  rt->copyFromTensor(bufC, out.data(), M * N * sizeof(float));
  CHECK_NEAR(out[0], 192.0f, 1.0f);
  CHECK_NEAR(out[1], 288.0f, 1.0f);
}

void q4SimpleAndWithScales() {
  {
    const uint32_t M = 1, K = 32, N = 2;
    std::vector<float> dataA(M * K, 1.0f);
    std::vector<uint8_t> packedB(K * (N / 2));
    for (uint32_t k = 0; k < K; ++k) packedB[k * (N / 2)] = packNibbles(9, 10);
    std::vector<uint16_t> scales(N, f32_to_f16(1.0f));
    auto bufC = rt->ops().matmul(rt->createTensor({M, K}, DataType::Float32, dataA.data()),
                                 rt->createTensor({K, N / 2}, DataType::Int8, packedB.data()),
                                 rt->createTensor({1, N}, DataType::Float16, scales.data()));
    std::vector<float> out(M * N);
    rt->copyFromTensor(bufC, out.data(), M * N * sizeof(float));
    CHECK_NEAR(out[0], 32.0f, 1e-3f);
    CHECK_NEAR(out[1], 64.0f, 1e-3f);
  }
  {
    const uint32_t M = 1, K = 64, N = 2;
    std::vector<float> dataA(M * K, 1.0f);
    std::vector<uint8_t> packedB(K * (N / 2));
    for (uint32_t k = 0; k < K; ++k) packedB[k * (N / 2)] = packNibbles(12, 12);
    std::vector<uint16_t> scales = {f32_to_f16(0.5f), f32_to_f16(2.0f), f32_to_f16(1.0f), f32_to_f16(0.25f)};
    auto bufC = rt->ops().matmul(rt->createTensor({M, K}, DataType::Float32, dataA.data()),
                                 rt->createTensor({K, N / 2}, DataType::Int8, packedB.data()),
                                 rt->createTensor({2, N}, DataType::Float16, scales.data()));
    std::vector<float> out(M * N);
    rt->copyFromTensor(bufC, out.data(), M * N * sizeof(float));
    CHECK_NEAR(out[0], 192.0f, 1.0f);
    CHECK_NEAR(out[1], 288.0f, 1.0f);
  }
}

// q8_vsregular (M=2,K=64,N=4) and q8_allvariants (M=1,K=512,N=16): every compiled variant whose
// name lacks "Dot", tolerance |ref| * 2% + 0.1 (OpRegistry.h:2028-2052, 2118-2152)
void q8VsRegularAllVariants(uint32_t M, uint32_t K, uint32_t N) {
  const uint32_t blocksPerRow = K / 32;
  auto dataA = generateTestData(M * K, 42);
  std::vector<int8_t> dataB(K * N);
  for (size_t i = 0; i < dataB.size(); ++i) dataB[i] = static_cast<int8_t>((i * 7 + 3) % 21 - 10);
  std::vector<float> scaleFloats(blocksPerRow * N);
  for (size_t i = 0; i < scaleFloats.size(); ++i) scaleFloats[i] = 0.1f + 0.05f * static_cast<float>(i);
  std::vector<uint16_t> scaleF16(scaleFloats.size());
  for (size_t i = 0; i < scaleFloats.size(); ++i) scaleF16[i] = f32_to_f16(scaleFloats[i]);
  auto bufA = rt->createTensor({M, K}, DataType::Float32, dataA.data());
  auto bufB = rt->createTensor({K, N}, DataType::Int8, dataB.data());
  auto bufS = rt->createTensor({blocksPerRow, N}, DataType::Float16, scaleF16.data());
  std::vector<float> ref(M * N, 0.0f);
  for (uint32_t m = 0; m < M; ++m)
    for (uint32_t n = 0; n < N; ++n)
      for (uint32_t k = 0; k < K; ++k)
        ref[m * N + n] += dataA[m * K + k] * static_cast<float>(dataB[k * N + n]) * scaleFloats[(k / 32) * N + n];
  int tested = 0;
  for (int vi = -1; vi < kMatMulQ8VariantCount; ++vi) {
    if (vi >= 0 && !getCompiledMatMulQ8(vi, DataType::Float32, DataType::Float16, DataType::Float32).has_value()) continue;
    if (vi >= 0 && std::string(getMatMulQ8VariantName(vi)).find("Dot") != std::string::npos) continue;
    auto bufC = vi < 0 ? rt->ops().matmul(bufA, bufB, bufS) : rt->ops().matmul(bufA, bufB, bufS, vi);
    std::vector<float> got(M * N);
    rt->copyFromTensor(bufC, got.data(), M * N * sizeof(float));
    for (uint32_t i = 0; i < M * N; ++i) CHECK_NEAR(got[i], ref[i], std::abs(ref[i]) * 0.01f + 0.1f);
    ++tested;
  }
  CHECK(tested > 2);
}

void q4VsReferenceAllVariants(uint32_t M, uint32_t K, uint32_t N) {  // OpRegistry.h:2088-2116, 2154-2192
  const uint32_t blocksPerRow = K / 32;
  auto dataA = generateTestData(M * K, 42);
  std::vector<uint8_t> nibbles(K * N);
  for (size_t i = 0; i < nibbles.size(); ++i) nibbles[i] = static_cast<uint8_t>((i * 7 + 3) % 16);
  std::vector<uint8_t> packedB(K * (N / 2));
  for (uint32_t k = 0; k < K; ++k)
    for (uint32_t n = 0; n < N; n += 2) packedB[k * (N / 2) + n / 2] = packNibbles(nibbles[k * N + n], nibbles[k * N + n + 1]);
  std::vector<float> scaleFloats(blocksPerRow * N);
  for (size_t i = 0; i < scaleFloats.size(); ++i) scaleFloats[i] = 0.1f + 0.05f * static_cast<float>(i);
  std::vector<uint16_t> scaleF16(scaleFloats.size());
  for (size_t i = 0; i < scaleFloats.size(); ++i) scaleF16[i] = f32_to_f16(scaleFloats[i]);
  auto bufA = rt->createTensor({M, K}, DataType::Float32, dataA.data());
  auto bufB = rt->createTensor({K, N / 2}, DataType::Int8, packedB.data());
  auto bufS = rt->createTensor({blocksPerRow, N}, DataType::Float16, scaleF16.data());
  std::vector<float> ref(M * N, 0.0f);
  for (uint32_t m = 0; m < M; ++m)
    for (uint32_t n = 0; n < N; ++n)
      for (uint32_t k = 0; k < K; ++k)
        ref[m * N + n] += dataA[m * K + k] * static_cast<float>(static_cast<int>(nibbles[k * N + n]) - 8) *
                          scaleFloats[(k / 32) * N + n];
  for (int vi = -1; vi < kMatMulQ4VariantCount; ++vi) {
    auto bufC = vi < 0 ? rt->ops().matmul(bufA, bufB, bufS) : rt->ops().matmul(bufA, bufB, bufS, vi);
    std::vector<float> got(M * N);
    rt->copyFromTensor(bufC, got.data(), M * N * sizeof(float));
    for (uint32_t i = 0; i < M * N; ++i) CHECK_NEAR(got[i], ref[i], std::abs(ref[i]) * 0.01f + 0.1f);
  }
}

void q8VsRegular() { q8VsRegularAllVariants(2, 64, 4); }
void q8AllVariants() { q8VsRegularAllVariants(1, 512, 16); }
void q4VsReference() { q4VsReferenceAllVariants(2, 64, 4); }
void q4AllVariants() { q4VsReferenceAllVariants(1, 64, 4); }

// tests/runtime/RuntimeTests.cpp:2861-2938, N trimmed to 1024 to keep the scalar CPU reference quick
void q8ModelGeometryBatchedVsPerRow() {
  const uint32_t M = 4, K = 5120, N = 1024, blocksPerRow = K / 32;
  std::vector<float> dataA(M * K);
  std::mt19937 gen(42);
  std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
  for (auto &x : dataA) x = dist(gen);
  std::vector<int8_t> dataB(K * N);
  for (size_t i = 0; i < dataB.size(); ++i) dataB[i] = static_cast<int8_t>((i * 7 + 3) % 21 - 10);
  std::vector<float> scaleFloats(blocksPerRow * N);
  for (size_t i = 0; i < scaleFloats.size(); ++i) scaleFloats[i] = (1.0f + (float)(i % 7)) * 0.03125f;
  std::vector<uint16_t> scaleF16(scaleFloats.size());
  for (size_t i = 0; i < scaleFloats.size(); ++i) scaleF16[i] = f32_to_f16(scaleFloats[i]);
  auto bufB = rt->createTensor({K, N}, DataType::Int8, dataB.data());
  auto bufS = rt->createTensor({blocksPerRow, N}, DataType::Float16, scaleF16.data());
  std::vector<float> batchedOut(M * N), perRowOut(M * N), silu(M * N);
  {
    auto bufA = rt->createTensor({M, K}, DataType::Float32, dataA.data());
    rt->copyFromTensor(rt->ops().matmul(bufA, bufB, bufS), batchedOut.data(), M * N * sizeof(float));
    rt->copyFromTensor(rt->ops().matmulUnary(UnarySilu, bufA, bufB, bufS), silu.data(), M * N * sizeof(float));
  }
  for (uint32_t m = 0; m < M; ++m) {
    auto bufRow = rt->createTensor({K}, DataType::Float32, dataA.data() + m * K);
    rt->copyFromTensor(rt->ops().matmul(bufRow, bufB, bufS), perRowOut.data() + m * N, N * sizeof(float));
  }
  int bad = 0;
  for (uint32_t m = 0; m < M; ++m)
    for (uint32_t n = 0; n < N; ++n) {
      double sum = 0.0;
      for (uint32_t k = 0; k < K; ++k)
        sum += (double)dataA[m * K + k] * (double)dataB[k * N + n] * (double)scaleFloats[(k / 32) * N + n];
      const float r = (float)sum, b = batchedOut[m * N + n], p = perRowOut[m * N + n];
      if (!(std::abs(b - r) <= std::abs(r) * 2e-3f + 0.05f)) ++bad;
      if (!(std::abs(b - p) <= std::abs(p) * 2e-3f + 0.05f)) ++bad;
      const float sr = r / (1.0f + std::exp(-r));
      if (!(std::abs(silu[m * N + n] - sr) <= std::abs(sr) * 2e-3f + 0.05f)) ++bad;
    }
  CHECK(bad == 0);
}

void dequantQ4K() {  // OpRegistry.h:1929-1957
  const uint32_t rows = 1, cols = 256;
  std::vector<uint8_t> rawBlock(144, 0);
  uint16_t d_f16 = f32_to_f16(1.0f), dmin_f16 = f32_to_f16(0.0f);
  std::memcpy(rawBlock.data(), &d_f16, 2);
  std::memcpy(rawBlock.data() + 2, &dmin_f16, 2);
  for (int j = 0; j < 4; ++j) { rawBlock[4 + j] = 1; rawBlock[4 + j + 4] = 0; }
  for (int j = 4; j < 8; ++j) rawBlock[4 + j + 4] = 1;
  uint8_t *qs = rawBlock.data() + 16;
  for (int i = 0; i < 128; ++i) qs[i] = static_cast<uint8_t>(((i % 8) & 0xF) | (((i % 8 + 1) & 0xF) << 4));
  auto raw = rt->createTensor({static_cast<uint32_t>(rawBlock.size())}, DataType::Int8, rawBlock.data());
  auto result = rt->ops().dequantize(raw, static_cast<uint32_t>(DequantFormat::Q4_K), rows, cols);
  std::vector<float> out(rows * cols), want(rows * cols);
  rt->copyFromTensor(result, out.data(), rows * cols * sizeof(float));
  for (uint32_t i = 0; i < cols; ++i) CHECK(std::isfinite(out[i]));
  for (uint32_t i = 0; i < 32; ++i) CHECK_NEAR(out[i], (float)(qs[i] & 0xF), 0.01f);
  orc_dequant_rows(2, rawBlock.data(), want.data(), rows, cols, cols);
  CHECK(std::memcmp(out.data(), want.data(), out.size() * sizeof(float)) == 0);
}

void transposeQ4NibbleBitExact() {  // OpCoverageTests.cpp:255-277
  const uint32_t N = 32, K = 32;
  auto Mv = [](uint32_t n, uint32_t k) -> uint8_t { return static_cast<uint8_t>((n * K + k) & 0xF); };
  std::vector<uint8_t> in(N * (K / 2));
  for (uint32_t n = 0; n < N; ++n)
    for (uint32_t j = 0; j < K / 2; ++j) in[n * (K / 2) + j] = static_cast<uint8_t>(Mv(n, j) | (Mv(n, j + 16) << 4));
  auto tIn = rt->createTensor({N, K / 2}, DataType::Int8, in.data());
  auto out = rt->ops().transposeQ4(tIn, N, K);
  CHECK(rt->getTensor(out).getShape() == (std::vector<uint32_t>{K, N / 2}));
  std::vector<uint8_t> got(K * (N / 2));
  rt->copyFromTensor(out, got.data(), got.size());
  int bad = 0;
  for (uint32_t k = 0; k < K; ++k)
    for (uint32_t n = 0; n < N; n += 2)
      if (got[k * (N / 2) + n / 2] != static_cast<uint8_t>(Mv(n, k) | (Mv(n + 1, k) << 4))) ++bad;
  CHECK(bad == 0);
}

// raw GGUF blocks through Operations::matmulBlocks against the CPU checker
void blocksAgainstChecker(int fmt, DequantFormat df, uint32_t M, uint32_t K, uint32_t N, bool half, int fusion) {
  const uint32_t bb = fmt == 0 ? 34 : fmt == 1 ? 18 : 144, be = fmt == 2 ? 256 : 32;
  std::mt19937 gen(1234 + fmt + M);
  std::vector<uint8_t> raw((size_t)N * (K / be) * bb);
  for (auto &b : raw) b = (uint8_t)gen();
  std::normal_distribution<float> nd(0.f, 0.02f);
  for (size_t blk = 0; blk < raw.size() / bb; ++blk) {  // sane fp16 scales at the head of every block
    uint16_t d = orc_f32_to_f16_runner(std::abs(nd(gen)) / 8.f);
    std::memcpy(&raw[blk * bb], &d, 2);
    if (fmt == 2) std::memcpy(&raw[blk * bb + 2], &d, 2);
  }
  std::normal_distribution<float> na(0.f, 1.f);
  std::vector<float> A(M * K), D(M * N);
  for (auto &x : A) x = na(gen);
  for (auto &x : D) x = na(gen);
  std::vector<uint16_t> A16(M * K);
  if (half)
    for (size_t i = 0; i < A.size(); ++i) {
      A16[i] = orc_f32_to_f16_runner(A[i]);
      // the checker sees the rounded activations: decode them back (exact)
      uint32_t h = A16[i], sign = (h & 0x8000u) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF;
      float f;
      if (e == 0) f = (float)m * 5.960464477539063e-08f;
      else { uint32_t bits = ((e + 112) << 23) | (m << 13); std::memcpy(&f, &bits, 4); }
      A[i] = sign ? -f : f;
    }
  auto tA = half ? rt->createTensor({M, K}, DataType::Float16, A16.data()) : rt->createTensor({M, K}, DataType::Float32, A.data());
  auto tW = rt->createTensor({(uint32_t)raw.size()}, DataType::Int8, raw.data());
  auto tD = rt->createTensor({M, N}, DataType::Float32, D.data());
  Tensor tC = fusion == 0   ? rt->ops().matmulBlocks(tA, tW, df, N)
              : fusion == 1 ? rt->ops().matmulBlocksUnary(UnarySilu, tA, tW, df, N)
                            : rt->ops().matmulBlocksBinary(BinaryAdd, tA, tW, df, N, tD);
  std::vector<float> got(M * N), ref(M * N);
  rt->copyFromTensor(tC, got.data(), got.size() * sizeof(float));
  orc_qmatmul_blocks(fmt, A.data(), raw.data(), ref.data(), D.data(), M, K, N, K, N, N, fusion, fusion == 1 ? 133 : 0, 1);
  double num = 0, den = 0;
  for (size_t i = 0; i < got.size(); ++i) {
    num += (double)(got[i] - ref[i]) * (got[i] - ref[i]);
    den += (double)ref[i] * ref[i];
  }
  CHECK(std::sqrt(num / den) <= 1e-3);  // rel-L2 tolerance of the path
}

void blocksEntryPoint() {
  blocksAgainstChecker(0, DequantFormat::Q8_0, 1, 1024, 300, false, 0);
  blocksAgainstChecker(1, DequantFormat::Q4_0, 1, 1024, 300, true, 0);
  blocksAgainstChecker(2, DequantFormat::Q4_K, 8, 512, 128, true, 0);
  blocksAgainstChecker(1, DequantFormat::Q4_0, 3, 512, 64, false, 1);
  blocksAgainstChecker(2, DequantFormat::Q4_K, 2, 512, 64, true, 2);
  blocksAgainstChecker(0, DequantFormat::Q8_0, 2, 96, 10, false, 0);   // K % 256 != 0: SIMT variant
  blocksAgainstChecker(1, DequantFormat::Q4_0, 40, 512, 64, true, 0);  // M too large for the mat-vec
}

// cached command buffer: record once, replay as one CUDA graph launch
// (interface/runner/llama/llama.cpp:2109-2126; core/backends/cuda/CudaCommandBuffer.cpp:261-285)
void reusableCommandBuffer() {
  const uint32_t K = 512, N = 64;
  std::vector<uint8_t> raw((size_t)N * (K / 32) * 34);
  std::mt19937 gen(7);
  for (auto &b : raw) b = (uint8_t)gen();
  for (size_t blk = 0; blk < raw.size() / 34; ++blk) { uint16_t d = 0x2000; std::memcpy(&raw[blk * 34], &d, 2); }
  std::vector<float> A(K, 1.0f), out1(N), out2(N);
  auto tA = rt->createTensor({K}, DataType::Float32, A.data());
  auto tW = rt->createTensor({(uint32_t)raw.size()}, DataType::Int8, raw.data());
  auto tC = rt->ops().matmulBlocks(tA, tW, DequantFormat::Q8_0, N);
  ComputeHandle cb = rt->iface().submitReusable();
  rt->iface().wait(cb);
  rt->copyFromTensor(tC, out1.data(), N * sizeof(float));
  for (auto &x : A) x = 2.0f;
  rt->copyToTensor(tA, A.data(), K * sizeof(float));
  rt->iface().resubmit(cb);
  rt->iface().wait(cb);
  rt->copyFromTensor(tC, out2.data(), N * sizeof(float));
  int bad = 0;
  for (uint32_t n = 0; n < N; ++n)
    if (!(std::abs(out2[n] - 2.0f * out1[n]) <= 1e-4f * std::abs(out1[n]) + 1e-6f)) ++bad;
  CHECK(bad == 0);
  CHECK_THROWS(rt->iface().resubmit(ComputeHandle()), "not a reusable");
}

// A recorded command buffer keeps the scratch it was built on: record a split-K mat-vec (its partial
// sums live in the backend's workspace), then run work that needs a much larger workspace (an fp32
// prefill: the GEMM's fp16 copy of A), then replay the first command buffer and compare.
void reusableSurvivesWorkspaceGrowth() {
  const uint32_t K = 8192, N = 256;  // long K, few rows: the mat-vec splits K
  std::vector<uint8_t> raw((size_t)N * (K / 32) * 18);
  std::mt19937 gen(11);
  for (auto &b : raw) b = (uint8_t)gen();
  for (size_t blk = 0; blk < raw.size() / 18; ++blk) { uint16_t d = 0x2000; std::memcpy(&raw[blk * 18], &d, 2); }
  std::vector<float> A(K);
  for (uint32_t k = 0; k < K; ++k) A[k] = (float)((int)(gen() % 17) - 8) / 8.0f;
  auto tA = rt->createTensor({K}, DataType::Float32, A.data());
  auto tW = rt->createTensor({(uint32_t)raw.size()}, DataType::Int8, raw.data());
  auto tC = rt->ops().matmulBlocks(tA, tW, DequantFormat::Q4_0, N);
  ComputeHandle cb = rt->iface().submitReusable();
  rt->iface().wait(cb);
  std::vector<float> out1(N), out2(N), want(N);
  rt->copyFromTensor(tC, out1.data(), N * sizeof(float));
  orc_qmatmul_blocks(1, A.data(), raw.data(), want.data(), nullptr, 1, K, N, K, N, 0, 0, 0, 0);
  double num = 0, den = 0;
  for (uint32_t n = 0; n < N; ++n) num += (out1[n] - want[n]) * (double)(out1[n] - want[n]), den += want[n] * (double)want[n];
  CHECK(std::sqrt(num / den) <= 1e-3);
  {  // 64 fp32 rows x K = 4096: the tensor-core GEMM asks for 2 * M * K bytes, far more than the mat-vec's partial sums
    const uint32_t M2 = 64, K2 = 4096, N2 = 128;
    std::vector<uint8_t> raw2((size_t)N2 * (K2 / 32) * 18);
    for (auto &b : raw2) b = (uint8_t)gen();
    for (size_t blk = 0; blk < raw2.size() / 18; ++blk) { uint16_t d = 0x2000; std::memcpy(&raw2[blk * 18], &d, 2); }
    std::vector<float> A2((size_t)M2 * K2, 0.25f);
    auto tA2 = rt->createTensor({M2, K2}, DataType::Float32, A2.data());
    auto tW2 = rt->createTensor({(uint32_t)raw2.size()}, DataType::Int8, raw2.data());
    auto tC2 = rt->ops().matmulBlocks(tA2, tW2, DequantFormat::Q4_0, N2);
    ComputeHandle h = rt->iface().submit();
    rt->iface().wait(h);
  }
  std::fill(out2.begin(), out2.end(), -1.0f);
  rt->iface().resubmit(cb);
  rt->iface().wait(cb);
  rt->copyFromTensor(tC, out2.data(), N * sizeof(float));
  int bad = 0;
  for (uint32_t n = 0; n < N; ++n) bad += (out1[n] != out2[n]);
  CHECK(bad == 0);
}

// Results of a reusable command buffer are copied to pinned host memory behind every replay; reading them must
// always give what the device buffer holds: the new result after every replay with new inputs, and the buffer's own
// contents again once something else has written it.
void resultCopiesFollowReplaysAndWrites() {
  const uint32_t K = 512, N = 96;
  std::vector<uint8_t> raw((size_t)N * (K / 32) * 34);
  std::mt19937 gen(23);
  for (auto &b : raw) b = (uint8_t)gen();
  for (size_t blk = 0; blk < raw.size() / 34; ++blk) { uint16_t d = 0x2400; std::memcpy(&raw[blk * 34], &d, 2); }
  std::vector<float> A1(K), A2(K), want(N), got(N);
  for (uint32_t k = 0; k < K; ++k) A1[k] = (float)((int)(gen() % 17) - 8) / 8.0f, A2[k] = (float)((int)(gen() % 13) - 6) / 4.0f;
  auto tA = rt->createTensor({K}, DataType::Float32, A1.data());
  auto tW = rt->createTensor({(uint32_t)raw.size()}, DataType::Int8, raw.data());
  auto tC = rt->ops().matmulBlocks(tA, tW, DequantFormat::Q8_0, N);
  // a second operator consumes tC: tC is then no result of the command buffer (read back the slow way), tR is
  std::vector<float> ones(N, 1.0f), gotR(N);
  auto tOnes = rt->createTensor({N}, DataType::Float32, ones.data());
  auto tR = rt->ops().rmsNorm(tC, tOnes, 1e-6f);
  ComputeHandle cb = rt->iface().submitReusable();
  rt->iface().wait(cb);
  auto relErr = [&](const std::vector<float> &a) {
    orc_qmatmul_blocks(0, a.data(), raw.data(), want.data(), nullptr, 1, K, N, K, N, 0, 0, 0, 0);
    double num = 0, den = 0;
    for (uint32_t n = 0; n < N; ++n) num += (got[n] - want[n]) * (double)(got[n] - want[n]), den += want[n] * (double)want[n];
    return std::sqrt(num / den);
  };
  for (int round = 0; round < 4; ++round) {
    const std::vector<float> &a = (round & 1) ? A2 : A1;
    rt->copyToTensor(tA, a.data(), K * sizeof(float));
    rt->iface().resubmit(cb);
    rt->iface().wait(cb);
    rt->copyFromTensor(tC, got.data(), N * sizeof(float));
    CHECK(relErr(a) <= 1e-3);
    rt->copyFromTensor(tR, gotR.data(), N * sizeof(float));
    double ss = 0;
    for (uint32_t n = 0; n < N; ++n) ss += got[n] * (double)got[n];
    const double inv = 1.0 / std::sqrt(ss / N + 1e-6);
    double worst = 0;
    for (uint32_t n = 0; n < N; ++n) worst = std::max(worst, std::fabs(gotR[n] - got[n] * inv));
    CHECK(worst <= 1e-4 * (1.0 + std::sqrt(ss / N) * inv));
  }
  // something else writes the result buffer: the next read returns the buffer, not the stale copy
  std::vector<float> sevens(N, 7.0f);
  rt->copyToTensor(tR, sevens.data(), N * sizeof(float));
  rt->copyFromTensor(tR, gotR.data(), N * sizeof(float));
  int bad = 0;
  for (uint32_t n = 0; n < N; ++n) bad += (gotR[n] != 7.0f);
  CHECK(bad == 0);
  // and a replay refreshes it again
  rt->copyToTensor(tA, A1.data(), K * sizeof(float));
  rt->iface().resubmit(cb);
  rt->iface().wait(cb);
  rt->copyFromTensor(tC, got.data(), N * sizeof(float));
  CHECK(relErr(A1) <= 1e-3);
}

// A tuning rule (runtime/VariantSelector.cpp:283-428) sends a 32-token matmul over a narrow weight to the decode
// mat-vec, which then runs two groups of 16 rows; without the rule the same call takes the tensor-core GEMM.  Both
// against the checker.
void tunedVariantRunsRowGroups() {
  const uint32_t M = 32, K = 1024, N = 264;
  std::vector<uint8_t> raw((size_t)N * (K / 32) * 18);
  std::mt19937 gen(31);
  for (auto &b : raw) b = (uint8_t)gen();
  for (size_t blk = 0; blk < raw.size() / 18; ++blk) { uint16_t d = 0x2000; std::memcpy(&raw[blk * 18], &d, 2); }
  std::vector<float> A((size_t)M * K), want((size_t)M * N), got((size_t)M * N);
  for (auto &a : A) a = (float)((int)(gen() % 17) - 8) / 8.0f;
  orc_qmatmul_blocks(1, A.data(), raw.data(), want.data(), nullptr, M, K, N, K, N, 0, 0, 0, 0);
  auto tA = rt->createTensor({M, K}, DataType::Float16, nullptr);
  {  // fp16 activations: 32 rows are two groups of 16
    std::vector<uint16_t> h(A.size());
    for (size_t i = 0; i < A.size(); ++i) {  // multiples of 1/8 up to 1: exact in fp16
      const float v = A[i];
      uint32_t bits;
      std::memcpy(&bits, &v, 4);
      const uint32_t sign = (bits >> 16) & 0x8000u, exp = (bits >> 23) & 0xFFu, man = bits & 0x7FFFFFu;
      h[i] = (uint16_t)(exp == 0 ? sign : sign | ((exp - 112u) << 10) | (man >> 13));
    }
    rt->copyToTensor(tA, h.data(), h.size() * 2);
  }
  auto tW = rt->createTensor({(uint32_t)raw.size()}, DataType::Int8, raw.data());
  auto relErr = [&]() {
    double num = 0, den = 0;
    for (size_t i = 0; i < got.size(); ++i) num += (got[i] - want[i]) * (double)(got[i] - want[i]), den += want[i] * (double)want[i];
    return std::sqrt(num / den);
  };
  auto &vs = VariantSelector::instance();
  vs.clear();
  {
    MatMulOpNode n0(rt->store(), tA, tW, DequantFormat::Q4_0, N);
    CHECK(*n0.spec() == 2);  // built-in: the GEMM
  }
  CHECK(vs.loadFromString(R"({"operators": {"MatMulQBlocks": {"backends": {"cuda": {"default_variant": 1,
        "rules": [{"variant": 1, "conditions": {"shape": [32, 1024, 264]}}]}}}}})"));
  {
    MatMulOpNode n1(rt->store(), tA, tW, DequantFormat::Q4_0, N);
    CHECK(*n1.spec() == 1);  // the rule: mat-vec in row groups
  }
  auto tC = rt->ops().matmulBlocks(tA, tW, DequantFormat::Q4_0, N);
  rt->copyFromTensor(tC, got.data(), got.size() * sizeof(float));
  CHECK(relErr() <= 1e-3);
  vs.clear();
  auto tC2 = rt->ops().matmulBlocks(tA, tW, DequantFormat::Q4_0, N);
  rt->copyFromTensor(tC2, got.data(), got.size() * sizeof(float));
  CHECK(relErr() <= 3e-3);
}

// GGUF file -> device weights without the CPU detour (interface/runner/llama/llama.cpp:831-866, 934-1027): raw blocks
// are uploaded as they lie in the file; fused QKV is a concatenation of rows, gate / up become alternating rows for the
// paired mat-vec, a Q6_K tensor is re-encoded to Q8_0 blocks on the device.  Every product is checked against the CPU
// checker run on the bytes of the file.
void ggufUploadAndMatmul() {
  const uint32_t K = 512;
  std::mt19937 gen(21);
  auto blocks = [&](uint32_t rows, uint32_t blockBytes, uint32_t blockElems, uint32_t dOff, uint16_t dBits) {
    std::vector<uint8_t> raw((size_t)rows * (K / blockElems) * blockBytes);
    for (auto &b : raw) b = (uint8_t)gen();
    for (size_t blk = 0; blk < raw.size() / blockBytes; ++blk) std::memcpy(&raw[blk * blockBytes + dOff], &dBits, 2);
    return raw;
  };
  auto q = blocks(32, 18, 32, 0, 0x2000), k = blocks(16, 18, 32, 0, 0x2000), v = blocks(16, 18, 32, 0, 0x2000);
  auto gate = blocks(48, 144, 256, 0, 0x1C00), up = blocks(48, 144, 256, 0, 0x1C00);
  for (auto *t : {&gate, &up})
    for (size_t blk = 0; blk < t->size() / 144; ++blk) { uint16_t m = 0x1800; std::memcpy(&(*t)[blk * 144 + 2], &m, 2); }
  auto down = blocks(24, 210, 256, 208, 0x1400);
  std::vector<float> norm(K);
  for (auto &x : norm) x = 0.5f + (float)(gen() % 100) / 100.0f;
  GGUFWriter w;
  w.header(7, 0);
  uint64_t off = 0;
  auto place = [&](size_t bytes) { const uint64_t o = off; off = (off + bytes + 31) / 32 * 32; return o; };
  const uint64_t oq = place(q.size()), ok_ = place(k.size()), ov = place(v.size()), og = place(gate.size()), ou = place(up.size()),
                 od = place(down.size()), on = place(norm.size() * 4);
  w.tensor2d("q", K, 32, 2, oq); w.tensor2d("k", K, 16, 2, ok_); w.tensor2d("v", K, 16, 2, ov);
  w.tensor2d("gate", K, 48, 12, og); w.tensor2d("up", K, 48, 12, ou); w.tensor2d("down", K, 24, 14, od);
  w.str("norm"); w.put<uint32_t>(1); w.put<uint64_t>(K); w.put<uint32_t>(0); w.put<uint64_t>(on);
  const size_t dataStart = (w.b.size() + 31) / 32 * 32;
  w.b.resize(dataStart + off);
  auto fill = [&](uint64_t o, const void *src, size_t n) { std::memcpy(w.b.data() + dataStart + o, src, n); };
  fill(oq, q.data(), q.size()); fill(ok_, k.data(), k.size()); fill(ov, v.data(), v.size()); fill(og, gate.data(), gate.size());
  fill(ou, up.data(), up.size()); fill(od, down.data(), down.size()); fill(on, norm.data(), norm.size() * 4);
  const std::string path = "/tmp/cutb_reference_cases.gguf";
  CHECK(w.save(path));

  GGUFFile file(path);
  GGUFUploader upl(*rt, file);
  std::vector<float> A(K);
  for (auto &x : A) x = (float)((int)(gen() % 33) - 16) / 16.0f;
  auto tA = rt->createTensor({K}, DataType::Float32, A.data());
  auto relL2 = [](const std::vector<float> &got, const std::vector<float> &want) {
    double num = 0, den = 0;
    for (size_t i = 0; i < want.size(); ++i) num += (got[i] - want[i]) * (double)(got[i] - want[i]), den += want[i] * (double)want[i];
    return std::sqrt(num / den);
  };
  {  // fused QKV: 64 rows of Q4_0, byte-identical to q | k | v
    BlockWeight qkv = upl.uploadFused({"q", "k", "v"});
    CHECK(qkv.N == 64 && qkv.K == K && qkv.format == DequantFormat::Q4_0 && !qkv.requantized);
    std::vector<uint8_t> all(q);
    all.insert(all.end(), k.begin(), k.end());
    all.insert(all.end(), v.begin(), v.end());
    std::vector<uint8_t> dev(all.size());
    rt->copyFromTensor(qkv.raw, dev.data(), dev.size());
    CHECK(dev == all);
    auto tC = rt->ops().matmulBlocks(tA, qkv.raw, qkv.format, qkv.N);
    std::vector<float> got(64), want(64);
    rt->copyFromTensor(tC, got.data(), got.size() * sizeof(float));
    orc_qmatmul_blocks(1, A.data(), all.data(), want.data(), nullptr, 1, K, 64, K, 64, 0, 0, 0, 0);
    CHECK(relL2(got, want) <= 1e-3);
  }
  {  // gate / up as alternating rows
    BlockWeight gu = upl.uploadPaired("gate", "up");
    CHECK(gu.N == 96 && gu.format == DequantFormat::Q4_K);
    std::vector<uint8_t> dev((size_t)96 * 2 * 144);
    rt->copyFromTensor(gu.raw, dev.data(), dev.size());
    int bad = 0;
    for (uint32_t i = 0; i < 48; ++i) {
      bad += std::memcmp(&dev[(size_t)(2 * i) * 288], &gate[(size_t)i * 288], 288) != 0;
      bad += std::memcmp(&dev[(size_t)(2 * i + 1) * 288], &up[(size_t)i * 288], 288) != 0;
    }
    CHECK(bad == 0);
    CHECK_THROWS(upl.uploadPaired("gate", "down"), "paired rows need");
  }
  {  // Q6_K: re-encoded to Q8_0 blocks on the device, the product agrees with the dense product over the exact weights
    BlockWeight d = upl.upload("down");
    CHECK(d.requantized && d.format == DequantFormat::Q8_0 && d.N == 24);
    auto tC = rt->ops().matmulBlocks(tA, d.raw, d.format, d.N);
    std::vector<float> got(24), want(24), wf((size_t)24 * K);
    rt->copyFromTensor(tC, got.data(), got.size() * sizeof(float));
    orc_dequant_rows(4, down.data(), wf.data(), 24, K, K);
    for (uint32_t n = 0; n < 24; ++n) {
      double acc = 0;
      for (uint32_t kk = 0; kk < K; ++kk) acc += (double)A[kk] * wf[(size_t)n * K + kk];
      want[n] = (float)acc;
    }
    CHECK(relL2(got, want) <= 1e-2);  // an 8-bit re-encode of 6-bit weights
    // and the fp32 form of the same tensor is the checker's dequantisation, bit for bit
    auto tF = upl.uploadF32("down");
    std::vector<float> devf((size_t)24 * K);
    rt->copyFromTensor(tF, devf.data(), devf.size() * sizeof(float));
    CHECK(std::memcmp(devf.data(), wf.data(), devf.size() * sizeof(float)) == 0);
  }
  {  // mixed formats fuse through Q8_0
    BlockWeight m = upl.uploadFused({"k", "down"});
    CHECK(m.requantized && m.format == DequantFormat::Q8_0 && m.N == 40);
    auto tC = rt->ops().matmulBlocks(tA, m.raw, m.format, m.N);
    std::vector<float> got(40);
    rt->copyFromTensor(tC, got.data(), got.size() * sizeof(float));
    std::vector<float> wantK(16);
    orc_qmatmul_blocks(1, A.data(), k.data(), wantK.data(), nullptr, 1, K, 16, K, 16, 0, 0, 0, 0);
    std::vector<float> head(got.begin(), got.begin() + 16);
    CHECK(relL2(head, wantK) <= 1e-2);
  }
  auto tN = upl.uploadF32("norm");
  std::vector<float> nf(K);
  rt->copyFromTensor(tN, nf.data(), nf.size() * sizeof(float));
  CHECK(nf == norm);
  remove(path.c_str());
}

void errorBehaviour() {
  auto a = rt->createTensor({64}, DataType::Float32);
  auto b = rt->createTensor({32, 16}, DataType::Int8);
  auto s = rt->createTensor({1, 16}, DataType::Float16);
  CHECK_THROWS(rt->ops().matmul(a, b, s), "must match A cols");
  CHECK_THROWS(rt->ops().transposeQ4(b, 3, 32), "N must be even");
  auto raw = rt->createTensor({210}, DataType::Int8);
  CHECK_THROWS(rt->ops().dequantize(raw, 9u /* not a DequantFormat */, 1, 256), "no shader");
  {  // Q6_K has a kernel: one super-block of zero quants (q = -32) with scale 1 and d = 1
    std::vector<uint8_t> blk(210, 0);
    for (int i = 192; i < 208; ++i) blk[i] = 1;
    blk[208] = 0x00, blk[209] = 0x3C;
    auto q6 = rt->createTensor({210}, DataType::Int8, blk.data());
    auto out = rt->ops().dequantize(q6, (uint32_t)DequantFormat::Q6_K, 1, 256);
    std::vector<float> v(256), want(256);
    rt->copyFromTensor(out, v.data(), v.size() * sizeof(float));
    orc_dequant_rows(4, blk.data(), want.data(), 1, 256, 256);
    for (int i = 0; i < 256; ++i) CHECK(v[i] == -32.0f && want[i] == -32.0f);
  }
  CHECK(rt->iface().caps().backend == ComputeBackend::CUDA && rt->iface().caps().cooperativeMatrix);
  CHECK(rt->iface().bufferCount() > 0 && rt->iface().deviceTotalMemoryBytes() > (size_t)100 << 30);
}

// RMSNorm through Operations::rmsNorm (cases of OpCoverageTests.cpp:146-178 and
// RuntimeTests.cpp:3182-3209: 1-D known values, weighted rows, 13 x 5120 against fp64)
void rmsNormCases() {
  auto run = [&](uint32_t rows, uint32_t dim, const std::vector<float> &x, const std::vector<float> &w, bool oneD, float rel, float abs) {
    auto a = oneD ? rt->createTensor({dim}, DataType::Float32, x.data()) : rt->createTensor({rows, dim}, DataType::Float32, x.data());
    auto wt = rt->createTensor({dim}, DataType::Float32, w.data());
    auto out = rt->ops().rmsNorm(a, wt, 1e-5f);
    std::vector<float> got(rows * dim), want(rows * dim);
    rt->copyFromTensor(out, got.data(), got.size() * sizeof(float));
    orc_rmsnorm(x.data(), w.data(), want.data(), rows, dim, dim, 1e-5f);
    int bad = 0;
    for (uint32_t r = 0; r < rows; ++r) {
      double ss = 0;
      for (uint32_t i = 0; i < dim; ++i) ss += (double)x[r * dim + i] * x[r * dim + i];
      const double sc = 1.0 / std::sqrt(ss / dim + 1e-5);
      for (uint32_t i = 0; i < dim; ++i) {
        const double e = x[r * dim + i] * sc * w[i];
        if (!(std::abs(got[r * dim + i] - e) <= std::abs(e) * rel + abs)) ++bad;
        if (!(std::abs(want[r * dim + i] - e) <= std::abs(e) * rel + abs)) ++bad;
      }
    }
    CHECK(bad == 0);
  };
  run(1, 4, {1.f, 2.f, 3.f, 4.f}, {1.f, 1.f, 1.f, 1.f}, true, 0.f, 1e-4f);
  run(2, 4, {1.f, 2.f, 3.f, 4.f, 2.f, 4.f, 6.f, 8.f}, {0.5f, 1.0f, 1.5f, 2.0f}, false, 0.f, 1e-4f);
  const uint32_t N = 13, dim = 5120;
  std::mt19937 gen(7);
  std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
  std::vector<float> hidden(N * dim), weight(dim);
  for (auto &v : hidden) v = dist(gen);
  for (auto &v : weight) v = dist(gen) * 0.1f + 1.0f;
  run(N, dim, hidden, weight, false, 1e-3f, 1e-4f);
  run(3, 10, std::vector<float>(hidden.begin(), hidden.begin() + 30), std::vector<float>(weight.begin(), weight.begin() + 10), false,
      1e-3f, 1e-4f);  // dim % 4 != 0: padded row stride
}

// Whole-tensor argmax / argmin (RuntimeTests.cpp:1207-1262) plus the tie rule of the reference's tree
void argReduceCases() {
  auto run = [&](OperatorEnum op, const std::vector<float> &v) {
    auto in = rt->createTensor({(uint32_t)v.size()}, DataType::Float32, v.data());
    auto out = rt->ops().reduce(op, in);
    float got = -1.f;
    rt->copyFromTensor(out, &got, sizeof(float));
    const float want = orc_argreduce(v.data(), v.size(), op == ReduceArgmax);
    CHECK(got == want);
    return (int)got;
  };
  CHECK(run(ReduceArgmax, {1.f, 5.f, 3.f, 9.f, 2.f, 7.f, 4.f, 6.f}) == 3);
  CHECK(run(ReduceArgmin, {5.f, 3.f, 1.f, 9.f, 2.f, 7.f, 4.f, 6.f}) == 2);
  std::mt19937 gen(42);
  std::uniform_real_distribution<float> dist(-100.f, 100.f);
  std::vector<float> big(1024);
  for (auto &v : big) v = dist(gen);
  int expect = 0;
  for (int i = 1; i < 1024; ++i)
    if (big[i] > big[expect]) expect = i;
  CHECK(run(ReduceArgmax, big) == expect);
  std::vector<float> ties(600, 0.f);
  ties[1] = ties[2] = ties[258] = 1.f;  // lanes 1, 2, 2: bit-reversed lane 2 (64) beats lane 1 (128), then the smaller index
  CHECK(run(ReduceArgmax, ties) == 2);
}

// Embedding gather through Operations::embedding (rows of a [vocab, dim] fp32 table)
void embeddingCases() {
  const uint32_t vocab = 37, dim = 10;
  std::vector<float> table(vocab * dim);
  for (size_t i = 0; i < table.size(); ++i) table[i] = (float)i * 0.25f;
  std::vector<uint32_t> idx = {36, 0, 5, 5, 17};
  auto tT = rt->createTensor({vocab, dim}, DataType::Float32, table.data());
  auto tI = rt->createTensor({(uint32_t)idx.size()}, DataType::UInt32, idx.data());
  auto out = rt->ops().embedding(tI, tT);
  CHECK(rt->getTensor(out).getShape() == (std::vector<uint32_t>{5, dim}));
  std::vector<float> got(idx.size() * dim);
  rt->copyFromTensor(out, got.data(), got.size() * sizeof(float));
  int bad = 0;
  for (size_t i = 0; i < idx.size(); ++i)
    for (uint32_t j = 0; j < dim; ++j)
      if (got[i * dim + j] != table[idx[i] * dim + j]) ++bad;
  CHECK(bad == 0);
  idx[1] = vocab;  // outside the table: zeros and an error when the batch is waited for
  auto tBad = rt->createTensor({(uint32_t)idx.size()}, DataType::UInt32, idx.data());
  auto outBad = rt->ops().embedding(tBad, tT);
  CHECK_THROWS(rt->flush(), "kernel reported");
  rt->copyFromTensor(outBad, got.data(), got.size() * sizeof(float));
  bad = 0;
  for (uint32_t j = 0; j < dim; ++j)
    if (got[dim + j] != 0.f || got[j] != table[36 * dim + j]) ++bad;
  CHECK(bad == 0);
}

// Attention through Operations::attention: the reference's two geometries (RuntimeTests.cpp:5996-6066,
// uniform [0.1, 10) data, its 1e-3 / 1e-2 absolute tolerances) against the CPU checker
void attentionCases() {
  auto run = [&](uint32_t nH, uint32_t nKv, uint32_t hd, uint32_t seq, uint32_t maxSeq, float tol) {
    const uint32_t dim = nH * hd, kvDim = nKv * hd;
    auto q = generateTestData(dim, 42), kData = generateTestData(maxSeq * kvDim, 100), vData = generateTestData(maxSeq * kvDim, 200);
    auto tq = rt->createTensor({dim}, DataType::Float32, q.data());
    auto tk = rt->createTensor({maxSeq, kvDim}, DataType::Float32, kData.data());
    auto tv = rt->createTensor({maxSeq, kvDim}, DataType::Float32, vData.data());
    uint32_t params[2] = {seq - 1, seq};
    auto tp = rt->createTensor({2}, DataType::UInt32, params);
    auto out = rt->ops().attention(tq, tk, tv, tp, nH, nKv, hd);
    std::vector<float> got(dim), want(dim);
    rt->copyFromTensor(out, got.data(), dim * sizeof(float));
    orc_attention(0, q.data(), kData.data(), vData.data(), seq, want.data(), nH, nKv, hd, kvDim, 1.0f / std::sqrt((float)hd));
    int bad = 0;
    for (uint32_t i = 0; i < dim; ++i)
      if (!(std::abs(got[i] - want[i]) <= tol)) ++bad;
    CHECK(bad == 0);
  };
  run(1, 1, 4, 3, 8, 1e-3f);
  run(4, 2, 8, 4, 16, 1e-2f);
  run(32, 8, 128, 300, 512, 1e-3f);  // the decoder's geometry: the cluster kernel
}

// Per-token chain fusedRoPEKVWrite -> attention over growing positions (the sequence of
// RuntimeTests.cpp:2231-2262, fp32 caches) against the checker's chain
void ropeCacheAttentionChain() {
  const uint32_t nH = 4, nKv = 2, hd = 16, maxSeq = 16, N = 6, qdim = nH * hd, kvdim = nKv * hd, half = hd / 2;
  std::mt19937 gen(123);
  std::uniform_real_distribution<float> dist(-1.f, 1.f);
  std::vector<float> cosT(maxSeq * half), sinT(maxSeq * half);
  for (uint32_t p = 0; p < maxSeq; ++p)
    for (uint32_t i = 0; i < half; ++i) {
      const float theta = float(p) / std::pow(10000.0f, 2.0f * i / hd);
      cosT[p * half + i] = std::cos(theta);
      sinT[p * half + i] = std::sin(theta);
    }
  auto tCos = rt->createTensor({maxSeq * half}, DataType::Float32, cosT.data());
  auto tSin = rt->createTensor({maxSeq * half}, DataType::Float32, sinT.data());
  std::vector<float> zeros(maxSeq * kvdim, 0.f), kRef(zeros), vRef(zeros);
  auto tK = rt->createTensor({maxSeq, kvdim}, DataType::Float32, zeros.data());
  auto tV = rt->createTensor({maxSeq, kvdim}, DataType::Float32, zeros.data());
  int bad = 0;
  for (uint32_t i = 0; i < N; ++i) {
    std::vector<float> q(qdim), k(kvdim), v(kvdim), qr(qdim), want(qdim), got(qdim), gotQ(qdim);
    for (auto &x : q) x = dist(gen);
    for (auto &x : k) x = dist(gen);
    for (auto &x : v) x = dist(gen);
    uint32_t params[2] = {i, i + 1};
    auto tp = rt->createTensor({2}, DataType::UInt32, params);
    auto tq = rt->createTensor({qdim}, DataType::Float32, q.data());
    auto tk = rt->createTensor({kvdim}, DataType::Float32, k.data());
    auto tv = rt->createTensor({kvdim}, DataType::Float32, v.data());
    auto roped = rt->ops().fusedRoPEKVWrite(tq, tk, tv, tp, tCos, tSin, tK, tV, hd);
    rt->ops().barrier();
    auto attn = rt->ops().attention(roped, tK, tV, tp, nH, nKv, hd);
    rt->copyFromTensor(attn, got.data(), qdim * sizeof(float));
    rt->copyFromTensor(roped, gotQ.data(), qdim * sizeof(float));
    orc_rope_kv_write(0, q.data(), k.data(), v.data(), i, cosT.data(), sinT.data(), kRef.data(), vRef.data(), qr.data(), qdim, kvdim, hd,
                      kvdim);
    orc_attention(0, qr.data(), kRef.data(), vRef.data(), i + 1, want.data(), nH, nKv, hd, kvdim, 1.0f / std::sqrt((float)hd));
    if (std::memcmp(gotQ.data(), qr.data(), qdim * sizeof(float)) != 0) ++bad;  // the rotation is bit-exact
    for (uint32_t j = 0; j < qdim; ++j)
      if (!(std::abs(got[j] - want[j]) <= std::abs(want[j]) * 1e-3f + 1e-4f)) ++bad;
  }
  CHECK(bad == 0);
  std::vector<float> kGot(maxSeq * kvdim);
  rt->copyFromTensor(tK, kGot.data(), kGot.size() * sizeof(float));
  CHECK(std::memcmp(kGot.data(), kRef.data(), kGot.size() * sizeof(float)) == 0);
}

// Batched path (batchedKVCacheWrite + batchedAttentionReadCache over a fused QKV matrix) against the per-token
// chain, row by row, with the reference's tolerance (RuntimeTests.cpp:2215-2300)
void batchedAgainstPerToken() {
  const uint32_t nH = 4, nKv = 2, hd = 16, maxSeq = 32, N = 9, qdim = nH * hd, kvdim = nKv * hd, half = hd / 2;
  const uint32_t width = qdim + 2 * kvdim;
  std::mt19937 gen(123);
  std::uniform_real_distribution<float> dist(-1.f, 1.f);
  std::vector<float> qkv(N * width);
  for (auto &x : qkv) x = dist(gen);
  std::vector<float> cosT(maxSeq * half), sinT(maxSeq * half);
  for (uint32_t p = 0; p < maxSeq; ++p)
    for (uint32_t i = 0; i < half; ++i) {
      const float theta = float(p) / std::pow(10000.0f, 2.0f * i / hd);
      cosT[p * half + i] = std::cos(theta);
      sinT[p * half + i] = std::sin(theta);
    }
  auto tCos = rt->createTensor({maxSeq * half}, DataType::Float32, cosT.data());
  auto tSin = rt->createTensor({maxSeq * half}, DataType::Float32, sinT.data());
  std::vector<float> zeros(maxSeq * kvdim, 0.f), ref(N * qdim), got(N * qdim);
  {  // per token
    auto tK = rt->createTensor({maxSeq, kvdim}, DataType::Float32, zeros.data());
    auto tV = rt->createTensor({maxSeq, kvdim}, DataType::Float32, zeros.data());
    for (uint32_t i = 0; i < N; ++i) {
      uint32_t params[2] = {i, i + 1};
      auto tp = rt->createTensor({2}, DataType::UInt32, params);
      auto tq = rt->createTensor({qdim}, DataType::Float32, &qkv[i * width]);
      auto tk = rt->createTensor({kvdim}, DataType::Float32, &qkv[i * width + qdim]);
      auto tv = rt->createTensor({kvdim}, DataType::Float32, &qkv[i * width + qdim + kvdim]);
      auto roped = rt->ops().fusedRoPEKVWrite(tq, tk, tv, tp, tCos, tSin, tK, tV, hd);
      auto attn = rt->ops().attention(roped, tK, tV, tp, nH, nKv, hd);
      rt->copyFromTensor(attn, &ref[i * qdim], qdim * sizeof(float));
    }
  }
  {  // batched, q / k / v as columns of one matrix
    auto tK = rt->createTensor({maxSeq, kvdim}, DataType::Float32, zeros.data());
    auto tV = rt->createTensor({maxSeq, kvdim}, DataType::Float32, zeros.data());
    std::vector<uint32_t> positions(N);
    for (uint32_t i = 0; i < N; ++i) positions[i] = i;
    auto tPos = rt->createTensor({N}, DataType::UInt32, positions.data());
    auto tQkv = rt->createTensor({N, width}, DataType::Float32, qkv.data());
    rt->ops().batchedKVCacheWrite(tQkv, tQkv, tK, tV, tPos, tCos, tSin, N, nKv, hd, width, width, qdim, qdim + kvdim);
    auto attn = rt->ops().batchedAttentionReadCache(tQkv, tK, tV, tPos, tCos, tSin, N, nH, nKv, hd, width, 0);
    CHECK(rt->getTensor(attn).getShape() == (std::vector<uint32_t>{N, qdim}));
    rt->copyFromTensor(attn, got.data(), got.size() * sizeof(float));
  }
  int bad = 0;
  for (size_t j = 0; j < ref.size(); ++j)
    if (!(std::abs(got[j] - ref[j]) <= std::abs(ref[j]) * 1e-3f + 1e-4f)) ++bad;
  CHECK(bad == 0);
}

}  // namespace

int main() {
  try {
    Runtime runtime(0);
    rt = &runtime;
    RUN(q8Simple);
    RUN(q8WithScales);
    RUN(q4SimpleAndWithScales);
    RUN(q8VsRegular);
    RUN(q8AllVariants);
    RUN(q4VsReference);
    RUN(q4AllVariants);
    RUN(q8ModelGeometryBatchedVsPerRow);
    RUN(dequantQ4K);
    RUN(transposeQ4NibbleBitExact);
    RUN(blocksEntryPoint);
    RUN(reusableCommandBuffer);
    RUN(reusableSurvivesWorkspaceGrowth);
    RUN(resultCopiesFollowReplaysAndWrites);
    RUN(tunedVariantRunsRowGroups);
    RUN(ggufUploadAndMatmul);
    RUN(errorBehaviour);
    RUN(rmsNormCases);
    RUN(argReduceCases);
    RUN(embeddingCases);
    RUN(attentionCases);
    RUN(ropeCacheAttentionChain);
    RUN(batchedAgainstPerToken);
  } catch (const std::exception &e) {
    std::printf("FAIL: unexpected exception: %s\n", e.what());
    return 2;
  }
  return finish();
}
