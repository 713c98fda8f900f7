// CPU tests of the host logic of the operator API slice: shape validation and
// error messages, variant choice, push constants, bindings, shader keys, kernel
// descriptors, the Dispatcher's cache and VariantSelector rules.  A recording
// ComputeInterface stands in for the device: it allocates host memory for
// buffers and records dispatches without executing anything.
#include <cstdlib>

#include "check.h"
#include "cut_api.h"
#include "gguf_upload.h"
#include "gguf_writer.h"

using namespace cut;

// This executable links the host logic only; the device backend is not part of it.
namespace cut {
std::unique_ptr<ComputeInterface> createB200Compute(int) {
  throw std::runtime_error("host_logic_test is built without the device backend");
}
}  // namespace cut

namespace {

struct HostBuffer : ComputeBuffer {
  std::vector<uint8_t> bytes;
};
struct Module : ComputeHandle::Slot {
  KernelDesc desc;
};
struct Batch : ComputeHandle::Slot {
  std::vector<ComputeDispatch> dispatches;
};

class RecordingCompute : public ComputeInterface {
public:
  RecordingCompute() {
    caps_.backend = ComputeBackend::CUDA;
    caps_.cooperativeMatrix = true;
  }
  ComputeHandle createBuffer(const std::vector<uint32_t> &shape, DataType dtype, const void *host, bool) override {
    auto b = std::make_shared<HostBuffer>();
    b->describe(shape, dtype);
    b->bytes.assign(b->size(), 0);
    b->data = b->bytes.data();
    if (host) copyActualToAligned(host, b->data, *b);
    ++buffers;
    return ComputeHandle(b);
  }
  ComputeHandle createBufferView(const ComputeHandle &, size_t, const std::vector<uint32_t> &, DataType) override {
    throw std::runtime_error("views are not part of these tests");
  }
  void copyDataToBuffer(const void *, const ComputeHandle &, size_t, size_t, size_t, bool, bool) override {}
  void copyDataFromBuffer(const ComputeHandle &src, void *dst, size_t n, size_t, size_t, bool, bool) override {
    auto *b = src.as<HostBuffer>();
    std::vector<uint8_t> dense(b->calculateActualSize());
    copyAlignedToActual(b->data, dense.data(), *b);
    std::memcpy(dst, dense.data(), n);
  }
  ComputeHandle createShaderModule(const std::vector<uint32_t> &words) override {
    auto d = KernelDesc::decode(words);
    if (!d) throw std::runtime_error("not a kernel descriptor");
    auto m = std::make_shared<Module>();
    m->desc = *d;
    ++modules;
    return ComputeHandle(m);
  }
  const ComputeBuffer &getBuffer(const ComputeHandle &h) const override {
    auto *b = h.as<HostBuffer>();
    if (!b) throw std::runtime_error("invalid buffer handle");
    return *b;
  }
  size_t bufferCount() const override { return buffers; }
  size_t buffers = 0, modules = 0;
  std::vector<ComputeDispatch> executed;

protected:
  ComputeHandle executeDispatches(std::vector<ComputeDispatch> &&d, bool) override {
    auto b = std::make_shared<Batch>();
    for (auto &x : d) executed.push_back(x);
    b->dispatches = std::move(d);
    return ComputeHandle(b);
  }
  void replay(const ComputeHandle &) override {}
  void waitFor(const ComputeHandle &) override {}
};

struct Fixture {
  RecordingCompute *raw;
  Runtime rt;
  Fixture() : raw(new RecordingCompute()), rt(std::unique_ptr<ComputeInterface>(raw)) {}
};

struct PC {
  uint32_t M, K, N, strideA, strideB, strideC, scaleStride;
};
PC pcOf(const MatMulOpNode &n) {
  PC pc;
  auto b = n.bindings();
  std::memcpy(&pc, b.back().bytes.data(), sizeof(pc));
  return pc;
}

void bufferGeometry() {
  // core/api/src/ComputeStructs.cpp:99-120: inner dim to 4 elements, bytes to 16
  CHECK(ComputeBuffer::calculateAlignedElements({3, 5}) == 3 * 8);
  CHECK(ComputeBuffer::calculateAlignedSize({3, 5}, DataType::Float32) == 96);
  CHECK(ComputeBuffer::calculateAlignedSize({2, 2}, DataType::Int8) == 16);
  CHECK(ComputeBuffer::calculateAlignedSize({5}, DataType::Float16) == 16);
  CHECK(ComputeBuffer::calculateActualSize({3, 5}, DataType::Float32) == 60);
  CHECK(dataTypeSize(DataType::Float16) == 2 && dataTypeSize(DataType::Int8) == 1);
  CHECK(widenPrecision(DataType::Float16) == DataType::Float32 && widenPrecision(DataType::Int8) == DataType::Int8);
  Fixture f;
  const float src[6] = {1, 2, 3, 4, 5, 6};
  auto t = f.rt.createTensor({2, 3}, DataType::Float32, src);
  const float *padded = (const float *)f.rt.getTensor(t).data;
  CHECK(padded[0] == 1 && padded[2] == 3 && padded[3] == 0 && padded[4] == 4 && padded[6] == 6);
  float back[6];
  f.rt.copyFromTensor(t, back, sizeof(back));
  CHECK(std::memcmp(back, src, sizeof(src)) == 0);
}

void quantFormatDetectionAndVariants() {
  Fixture f;
  auto &s = f.rt.store();
  const uint32_t K = 64;
  auto a1 = s.createTensor({K}, DataType::Float32), a4 = s.createTensor({4, K}, DataType::Float32);
  auto b8 = s.createTensor({K, 16}, DataType::Int8), b8small = s.createTensor({K, 4}, DataType::Int8);
  auto sc = s.createTensor({K / 32, 16}, DataType::Float16), scSmall = s.createTensor({K / 32, 4}, DataType::Float16);
  auto b4 = s.createTensor({K, 8}, DataType::Int8);
  auto scAff = s.createTensor({2 * K / 32, 16}, DataType::Float16);
  // Q8: B.cols == scales.cols; Q4: 2 * B.cols == scales.cols; affine: scales rows doubled (MatMulOp.cpp:309-329)
  MatMulOpNode q8(s, a1, b8, sc), q4(s, a1, b4, sc), q4a(s, a1, b4, scAff);
  CHECK(q8.format() == QuantFormat::Q8 && q8.op() == MatMulQ8 && q8.N() == 16 && q8.M() == 1 && q8.K() == K);
  CHECK(q4.format() == QuantFormat::Q4 && q4.op() == MatMulQ4 && q4.N() == 16 && !q4.affine());
  CHECK(q4a.affine());
  // variant choice (MatMulOp.cpp:335-380): M = 1 -> GemvKPar8 (N >= 8) else GemvKPar; M > 1 -> tensor-core tiled
  CHECK(*q8.spec() == 4 && *q4.spec() == 3);
  CHECK(*MatMulOpNode(s, a1, b8small, scSmall).spec() == 3);
  CHECK(*MatMulOpNode(s, a1, s.createTensor({K, 2}, DataType::Int8), scSmall).spec() == 2);  // Q4, N = 4 < 8
  auto b8w = s.createTensor({K, 32}, DataType::Int8), scw = s.createTensor({K / 32, 32}, DataType::Float16);
  CHECK(*MatMulOpNode(s, a4, b8w, scw).spec() == (uint32_t)kMatMulQ8VariantCount - 1);
  CHECK(*MatMulOpNode(s, a4, s.createTensor({K, 16}, DataType::Int8), scw).spec() == 4);  // Q4 tensor-core tiled
  CHECK(*MatMulOpNode(s, a4, b8, sc).spec() == (uint32_t)kMatMulQ8DefaultVariant);         // N % 32 != 0
  CHECK(*MatMulOpNode(s, a4, b8w, scw, 0).spec() == 0);                                    // explicit spec wins
  CHECK(std::string(getMatMulQ4VariantName(3)) == "MatMulQ4GemvKPar8");
  CHECK(std::string(getMatMulQ8VariantName(7)) == "MatMulQ8CoopMatTiled");
  CHECK(std::string(getMatMulQ8VariantName(99)) == "Unknown");
  CHECK(getCompiledMatMulQ8(4, DataType::Float32, DataType::Float16, DataType::Float32).has_value());
  CHECK(getCompiledMatMulQ8(4, DataType::Float16, DataType::Float16, DataType::Float32).has_value());
  CHECK(!getCompiledMatMulQ8(6, DataType::Float32, DataType::Float16, DataType::Float32).has_value());
  CHECK(!getCompiledMatMulQ4(5, DataType::Float32, DataType::Float16, DataType::Float32).has_value());
  CHECK(!getCompiledMatMulQ4(3, DataType::Float32, DataType::Float32, DataType::Float32).has_value());
  // output is allocated by the node: Float32 [M, N]
  CHECK(f.rt.getTensor(q8.output()).getShape() == (std::vector<uint32_t>{1, 16}));
  CHECK(f.rt.getTensor(q8.output()).getDtype() == DataType::Float32);
}

void shapeErrors() {
  Fixture f;
  auto &s = f.rt.store();
  auto a = s.createTensor({64}, DataType::Float32);
  auto b = s.createTensor({64, 16}, DataType::Int8);
  auto sc = s.createTensor({2, 16}, DataType::Float16);
  CHECK_THROWS(MatMulOpNode(s, a, s.createTensor({64}, DataType::Int8), sc), "2D B and scales");
  CHECK_THROWS(MatMulOpNode(s, s.createTensor({1, 1, 64}, DataType::Float32), b, sc), "A must be 1D or 2D");
  CHECK_THROWS(MatMulOpNode(s, s.createTensor({32}, DataType::Float32), b, sc), "must match A cols");
  CHECK_THROWS(MatMulOpNode(s, a, b, s.createTensor({2, 24}, DataType::Float16)), "cannot determine quant format");
  CHECK_THROWS(MatMulOpNode(s, a, b, sc, 42), "out of range");
  CHECK_THROWS(TransposeQ4NibbleOpNode(s, b, 3, 32), "N must be even");
  CHECK_THROWS(TransposeQ4NibbleOpNode(s, b, 4, 24), "multiple of 32");
  auto raw = s.createTensor({144}, DataType::Int8);
  CHECK_THROWS(MatMulOpNode(s, s.createTensor({256}, DataType::Float16), raw, DequantFormat::Q4_K, 2), "need");
  CHECK_THROWS(MatMulOpNode(s, a, raw, DequantFormat::Q4_K, 1), "multiple of the block size");
  CHECK_THROWS(MatMulOpNode(s, a, raw, DequantFormat::Q6_K, 1), "Q8_0, Q4_0 or Q4_K");
  CHECK_THROWS(MatMulOpNode(s, a, b, DequantFormat::Q4_0, 1), "1D Int8");
  MatMulOpNode ok(s, a, b, sc);
  CHECK_THROWS(ok.setFusion(MatMulFusion::Binary, BinaryAdd), "needs the D operand");
  CHECK_THROWS(ok.setFusion(MatMulFusion::Binary, BinaryAdd, s.createTensor({1, 8}, DataType::Float32)), "D must be");
}

void pushConstantsBindingsAndKeys() {
  Fixture f;
  auto &s = f.rt.store();
  const uint32_t M = 3, K = 96, N = 10;
  auto a = s.createTensor({M, K}, DataType::Float32);
  auto b8 = s.createTensor({K, N}, DataType::Int8), sc = s.createTensor({K / 32, N}, DataType::Float16);
  auto b4 = s.createTensor({K, N / 2}, DataType::Int8);
  MatMulOpNode q8(s, a, b8, sc), q4(s, a, b4, sc);
  // strides padded to 4 (MatMulOp.cpp:514-541)
  PC p8 = pcOf(q8), p4 = pcOf(q4);
  CHECK(p8.M == M && p8.K == K && p8.N == N && p8.strideA == 96 && p8.strideB == 12 && p8.strideC == 12 && p8.scaleStride == 12);
  CHECK(p4.strideB == 8 && p4.strideC == 12);
  // bindings: A, B, scales, dummy D (= C), C, push constants (MatMulOp.cpp:543-575)
  auto bind = q8.bindings();
  CHECK(bind.size() == 6 && bind[3].handle == q8.output() && bind[4].handle == q8.output() && !bind[5].isHandle());
  auto d = s.createTensor({M, N}, DataType::Float32);
  MatMulOpNode fused(s, a, b8, sc);
  fused.setFusion(MatMulFusion::Binary, BinaryAdd, d);
  auto fb = fused.bindings();
  CHECK(fb.size() == 6 && fb[3].handle == d && fb[4].handle == fused.output());
  // dispatch size = ceil(N / tileN) * wgX x ceil(M / tileM) * wgY (MatMulOp.cpp:507-512)
  ThreadSize ts = MatMulOpNode(s, s.createTensor({K}, DataType::Float32), b8, sc).dispatchSize();
  CHECK(ts.x == 2 * 32 && ts.y == 8 && ts.z == 1);
  // shader keys separate op, dtypes, affine, fusion and variant (MatMulOp.cpp:440-454)
  MatMulOpNode unary(s, a, b8, sc);
  unary.setFusion(MatMulFusion::Unary, UnarySilu);
  MatMulOpNode relu(s, a, b8, sc);
  relu.setFusion(MatMulFusion::Unary, UnaryRelu);
  MatMulOpNode half(s, s.createTensor({M, K}, DataType::Float16), b8, sc);
  CHECK(q8.shaderKey() != q4.shaderKey() && q8.shaderKey() != unary.shaderKey() && unary.shaderKey() != relu.shaderKey());
  CHECK(q8.shaderKey() != half.shaderKey() && q8.shaderKey() != fused.shaderKey());
  CHECK(q8.shaderKey() != MatMulOpNode(s, a, b8, sc, 0).shaderKey());
  auto scAff = s.createTensor({2 * K / 32, N}, DataType::Float16);
  CHECK(q4.shaderKey() != MatMulOpNode(s, a, b4, scAff).shaderKey());
  CHECK(q8.displayName() == "MatMulQ8" && unary.displayName() == "MatMulQ8Unary" && fused.displayName() == "MatMulQ8Binary");
  // the descriptor carries what the reference patches in as specialisation constants 1-3
  auto kd = KernelDesc::decode(*unary.shader());
  CHECK(kd && kd->op == MatMulQ8 && kd->fusionType == 1 && kd->fusionOp == UnarySilu && kd->affine == 0);
  auto ka = KernelDesc::decode(*MatMulOpNode(s, a, b4, scAff).shader());
  CHECK(ka && ka->op == MatMulQ4 && ka->affine == 1);
  CHECK(!KernelDesc::decode({1, 2, 3}).has_value());
  // Float16 activations are kept (kernels exist); D is widened
  auto r = half.resolveInputDtypes({DataType::Float16, DataType::Int8, DataType::Float16});
  CHECK(r[0] == DataType::Float16);
}

void blockNodesAndDequant() {
  Fixture f;
  auto &s = f.rt.store();
  const uint32_t K = 512, N = 6;
  auto raw = s.createTensor({N * (K / 256) * 144}, DataType::Int8);
  MatMulOpNode dec(s, s.createTensor({K}, DataType::Float16), raw, DequantFormat::Q4_K, N);
  CHECK(dec.format() == QuantFormat::Blocks && dec.op() == MatMulQBlocks && *dec.spec() == 1);  // decode mat-vec
  MatMulOpNode pre(s, s.createTensor({64, K}, DataType::Float16), raw, DequantFormat::Q4_K, N);
  CHECK(*pre.spec() == 2);  // prefill GEMM
  auto raw32 = s.createTensor({N * 3 * 18}, DataType::Int8);
  CHECK(*MatMulOpNode(s, s.createTensor({96}, DataType::Float32), raw32, DequantFormat::Q4_0, N).spec() == 0);
  auto kd = KernelDesc::decode(*dec.shader());
  CHECK(kd && kd->format == (uint32_t)DequantFormat::Q4_K && kd->variant == 1 && kd->dtypeA == (uint32_t)DataType::Float16);
  CHECK(pcOf(dec).strideB == 2 * 144);
  CHECK(dec.bindings().size() == 5);  // A, raw blocks, dummy D, C, push constants
  DequantOpNode dq(s, raw, DequantFormat::Q4_K, N, K);
  CHECK(dq.dispatchSize().x == K && dq.dispatchSize().y == N);
  CHECK(f.rt.getTensor(dq.output()).getShape() == (std::vector<uint32_t>{N, K}));
  CHECK(dq.shader().has_value() && DequantOpNode(s, raw, DequantFormat::Q6_K, N, K).shader().has_value());
  CHECK(!DequantOpNode(s, raw, static_cast<DequantFormat>(9), N, K).shader().has_value());
  TransposeQ4NibbleOpNode tq(s, s.createTensor({6, 16}, DataType::Int8), 6, 32);
  CHECK(f.rt.getTensor(tq.output()).getShape() == (std::vector<uint32_t>{32, 3}));
  struct {
    uint32_t N, K, sin, sout;
  } tp;
  auto tb = tq.bindings();
  std::memcpy(&tp, tb.back().bytes.data(), sizeof(tp));
  CHECK(tp.N == 6 && tp.K == 32 && tp.sin == 16 && tp.sout == 4);
}

// The runner's extras of the block matmul node (fused RMSNorm of A, paired gate / up rows, staging and overlap
// flags) and the GluPairs operator: descriptor words, bindings, push constants, output shapes, refusals.
void blockMatmulOptionsAndGluPairs() {
  Fixture f;
  auto &s = f.rt.store();
  const uint32_t K = 512, N = 12;
  auto raw = s.createTensor({N * (K / 32) * 18}, DataType::Int8);
  auto x = s.createTensor({K}, DataType::Float32);
  auto nw = s.createTensor({K}, DataType::Float32);
  MatMulOpNode plain(s, x, raw, DequantFormat::Q4_0, N);
  CHECK(plain.shader()->size() == 9 && plain.blockFlags() == 0);  // no options: the nine-word descriptor as before
  MatMulOpNode n1(s, x, raw, DequantFormat::Q4_0, N);
  MatMulBlockOptions o;
  o.flags = kBlockFlagRmsNorm | kBlockFlagAct16 | kBlockFlagNoOverlap;
  o.normWeight = nw;
  o.normEps = 1e-6f;
  n1.setBlockOptions(o);
  auto kd = KernelDesc::decode(*n1.shader());
  CHECK(n1.shader()->size() == 10 && kd && kd->flags == o.flags && kd->op == MatMulQBlocks);
  auto b = n1.bindings();  // A, raw blocks, the norm weight, dummy D, C, push constants (one more word: the epsilon)
  CHECK(b.size() == 6 && b[2].handle == nw && b[4].handle == n1.output() && b[5].bytes.size() == 32);
  float eps;
  std::memcpy(&eps, b[5].bytes.data() + 28, 4);
  CHECK(eps == 1e-6f);
  CHECK(n1.shaderKey() != plain.shaderKey());
  MatMulOpNode g(s, x, raw, DequantFormat::Q4_0, N);
  g.setFusion(MatMulFusion::Unary, UnarySilu);
  MatMulBlockOptions og;
  og.flags = kBlockFlagGluPairs;
  g.setBlockOptions(og);
  CHECK(g.outputShape() == (std::vector<uint32_t>{1, N / 2}) && f.rt.getTensor(g.output()).getShape() == g.outputShape());
  CHECK(pcOf(g).strideC == 8 && pcOf(g).N == N);  // the output row is N / 2 wide, padded to 4
  MatMulOpNode bad(s, x, raw, DequantFormat::Q4_0, N);
  CHECK_THROWS(bad.setBlockOptions(og), "need a unary fusion");
  MatMulBlockOptions on;
  on.flags = kBlockFlagRmsNorm;
  CHECK_THROWS(bad.setBlockOptions(on), "needs its weight");
  on.normWeight = s.createTensor({K + 4}, DataType::Float32);
  CHECK_THROWS(bad.setBlockOptions(on), "must be Float32 [K]");
  MatMulOpNode gemm(s, s.createTensor({64, K}, DataType::Float16), raw, DequantFormat::Q4_0, N);
  on.normWeight = nw;
  CHECK_THROWS(gemm.setBlockOptions(on), "decode mat-vec only");
  {
    // paired rows also run on the tensor-core GEMM (variant 2); the any-shape kernel (variant 0) has no such epilogue
    MatMulOpNode gg(s, s.createTensor({64, K}, DataType::Float16), raw, DequantFormat::Q4_0, N);
    gg.setFusion(MatMulFusion::Unary, UnarySilu);
    gg.setBlockOptions(og);
    CHECK(gg.outputShape() == (std::vector<uint32_t>{64, N / 2}));
    MatMulOpNode g0(s, x, raw, DequantFormat::Q4_0, N, 0u);
    g0.setFusion(MatMulFusion::Unary, UnarySilu);
    CHECK_THROWS(g0.setBlockOptions(og), "tensor-core GEMM only");
    // 13 to 16 fp16 rows on 16 M weights and more: the automatic choice is the GEMM; asking for the fused RMSNorm,
    // which only the mat-vec has, brings it back
    const uint32_t Kb = 4096, Nb = 4096;
    auto rawb = s.createTensor({Nb * (Kb / 32) * 18}, DataType::Int8);
    auto nwb = s.createTensor({Kb}, DataType::Float32);
    MatMulOpNode big(s, s.createTensor({16, Kb}, DataType::Float16), rawb, DequantFormat::Q4_0, Nb);
    CHECK(KernelDesc::decode(*big.shader())->variant == 2);
    MatMulOpNode small(s, s.createTensor({12, Kb}, DataType::Float16), rawb, DequantFormat::Q4_0, Nb);
    CHECK(KernelDesc::decode(*small.shader())->variant == 1);
    MatMulBlockOptions onb;
    onb.flags = kBlockFlagRmsNorm;
    onb.normWeight = nwb;
    big.setBlockOptions(onb);
    CHECK(KernelDesc::decode(*big.shader())->variant == 1);
  }
  auto fused = f.rt.ops().matmulBlocksFused(x, raw, DequantFormat::Q4_0, N, o);
  CHECK(f.rt.getTensor(fused).getShape() == (std::vector<uint32_t>{1, N}));

  GluPairsOpNode gp(s, s.createTensor({5, 14}, DataType::Float32), UnarySilu);
  CHECK(gp.op() == GluPairs && gp.outputShape() == (std::vector<uint32_t>{5, 7}) && gp.displayName() == "GluPairs");
  struct {
    uint32_t rows, colsOut, strideIn, strideOut;
  } gpc;
  auto gb = gp.bindings();
  std::memcpy(&gpc, gb.back().bytes.data(), sizeof(gpc));
  CHECK(gpc.rows == 5 && gpc.colsOut == 7 && gpc.strideIn == 16 && gpc.strideOut == 8);
  auto gkd = KernelDesc::decode(*gp.shader());
  CHECK(gkd && gkd->op == GluPairs && gkd->fusionOp == (uint32_t)UnarySilu);
  CHECK_THROWS(GluPairsOpNode(s, s.createTensor({5, 13}, DataType::Float32), UnarySilu), "even number of columns");
  CHECK_THROWS(GluPairsOpNode(s, s.createTensor({5, 14}, DataType::Float16), UnarySilu), "must be Float32");
}

void dispatcherAndOperations() {
  Fixture f;
  auto &ops = f.rt.ops();
  auto &s = f.rt.store();
  const uint32_t K = 64, N = 8;
  auto a = s.createTensor({K}, DataType::Float32);
  auto b = s.createTensor({K, N}, DataType::Int8), sc = s.createTensor({K / 32, N}, DataType::Float16);
  auto c1 = ops.matmul(a, b, sc);
  auto c2 = ops.matmul(a, b, sc);
  auto c3 = ops.matmulUnary(UnarySilu, a, b, sc);
  auto d = s.createTensor({1, N}, DataType::Float32);
  auto c4 = ops.matmulBinary(BinaryAdd, a, b, sc, d);
  CHECK(c1 != c2 && f.raw->modules == 3);  // same kernel cached by shaderKey (Dispatcher.cpp:62-75)
  CHECK(f.raw->pendingDispatches() == 4 && f.raw->executed.empty());
  ops.barrier();
  f.rt.flush();
  CHECK(f.raw->executed.size() == 5 && f.raw->executed[4].isBarrier && f.raw->executed[0].label == "MatMulQ8");
  CHECK(f.raw->executed[3].label == "MatMulQ8Binary" && f.raw->executed[3].outputHandle == c4);
  // a node without a kernel is an error, not a silent skip
  auto raw = s.createTensor({210}, DataType::Int8);
  CHECK_THROWS(ops.dequantize(raw, 9u /* not a DequantFormat */, 1, 256), "no shader");
  (void)c3;
}

void variantSelectorRules() {
  auto &vs = VariantSelector::instance();
  vs.clear();
  CHECK(vs.select("MatMulQ8", {1, 64, 16}, 4, "cuda") == 4);  // not loaded -> default
  const char *json = R"({"operators": {
      "MatMulQ8": {"default_variant": 2, "rules": [{"variant": 1, "conditions": {"total_elements_max": 2048}}],
                   "backends": {"cuda": {"default_variant": 4,
                                          "rules": [{"variant": 3, "conditions": {"shape": [1, 64, 16]}},
                                                    {"variant": 0, "conditions": {"total_elements_min": 100000}}]}}},
      "MatMulQBlocks": {"backends": {"cuda": {"default_variant": 0, "rules": []}}}}})";
  CHECK(vs.loadFromString(json) && vs.isLoaded());
  CHECK(vs.select("MatMulQ8", {1, 64, 16}, 7, "cuda") == 3);        // exact shape, backend-specific
  CHECK(vs.select("MatMulQ8", {1, 64, 8}, 7, "cuda") == 4);         // backend default
  CHECK(vs.select("MatMulQ8", {64, 64, 64}, 7, "cuda") == 0);       // total_elements_min
  CHECK(vs.select("MatMulQ8", {1, 64, 16}, 7, "vulkan") == 1);      // falls back to backend-agnostic rules
  CHECK(vs.select("MatMulQ8", {64, 64, 64}, 7, "") == 2);
  CHECK(vs.select("MatMulQ4", {1, 64, 16}, 3, "cuda") == 3);        // unknown operator -> caller's default
  {
    Fixture f;
    auto &s = f.rt.store();
    auto a = s.createTensor({64}, DataType::Float32);
    auto b = s.createTensor({64, 16}, DataType::Int8), sc = s.createTensor({2, 16}, DataType::Float16);
    CHECK(*MatMulOpNode(s, a, b, sc).spec() == 3);  // the rule overrides the built-in GemvKPar8
    auto raw = s.createTensor({2 * 144}, DataType::Int8);
    CHECK(*MatMulOpNode(s, s.createTensor({256}, DataType::Float16), raw, DequantFormat::Q4_K, 2).spec() == 0);
  }
  CHECK(!vs.loadFromString("{ not json"));
  CHECK(!vs.loadFromFile("/nonexistent/tuning_data.json"));
  vs.clear();
  CHECK(!vs.isLoaded());
}

}  // namespace

// RMSNormOpNode / EmbeddingOpNode / GlobalReduceOpNode: validation, geometry and recorded dispatches
void layerOperatorNodes() {
  Fixture f;
  TensorStore &s = f.rt.store();
  auto x1 = s.createTensor({10}, DataType::Float32), x2 = s.createTensor({3, 10}, DataType::Float32);
  auto w = s.createTensor({10}, DataType::Float32), wh = s.createTensor({10}, DataType::Float16);
  RMSNormOpNode n1(s, x1, w), n2(s, x2, w, 1e-6f);
  CHECK(n1.outputShape() == (std::vector<uint32_t>{10}) && n2.outputShape() == (std::vector<uint32_t>{3, 10}));
  CHECK(n2.dispatchSize().x == 256 && n2.dispatchSize().y == 3 && n1.dispatchSize().y == 1);
  struct {
    uint32_t dim, alignedDim;
    float eps;
  } pc;
  auto b = n2.bindings();
  CHECK(b.size() == 4 && b[2].handle == n2.output() && b[3].bytes.size() == sizeof(pc));
  std::memcpy(&pc, b[3].bytes.data(), sizeof(pc));
  CHECK(pc.dim == 10 && pc.alignedDim == 12 && pc.eps == 1e-6f);
  CHECK(n1.op() == RMSNorm && n1.displayName() == "RMSNorm" && n1.shader().has_value());
  CHECK_THROWS(RMSNormOpNode(s, s.createTensor({1, 3, 10}, DataType::Float32), w), "1D or 2D input, 1D weight");
  CHECK_THROWS(RMSNormOpNode(s, x1, x2), "1D or 2D input, 1D weight");
  CHECK_THROWS(RMSNormOpNode(s, x1, s.createTensor({12}, DataType::Float32)), "weight dimension must match");
  CHECK_THROWS(RMSNormOpNode(s, x1, wh), "same dtype");
  CHECK(RMSNormOpNode(s, s.createTensor({10}, DataType::Float16), wh).shaderKey() != n1.shaderKey());

  auto table = s.createTensor({50, 6}, DataType::Float32), idx = s.createTensor({2, 5}, DataType::UInt32);
  EmbeddingOpNode e(s, idx, table);
  CHECK(e.outputShape() == (std::vector<uint32_t>{2, 5, 6}) && e.outputDtype() == DataType::Float32);
  CHECK(e.dispatchSize().x == 256 && e.dispatchSize().y == 1);  // 10 rows x 2 vec4 -> one group of 256
  uint32_t epc[2];
  std::memcpy(epc, e.bindings().back().bytes.data(), sizeof(epc));
  CHECK(epc[0] == 10 && epc[1] == 6);
  auto pre = s.createTensor({2, 5, 6}, DataType::Float32);
  CHECK(EmbeddingOpNode(s, idx, table, pre).output() == pre);
  CHECK_THROWS(EmbeddingOpNode(s, idx, w), "weight must be 2D");
  CHECK(!EmbeddingOpNode(s, idx, s.createTensor({50, 6}, DataType::Float16)).shader().has_value());
  {  // EmbeddingColOpNode (operators/impl/memory/MemoryOp.cpp:127-202): geometry, format detection, messages
    auto head16 = s.createTensor({6, 50}, DataType::Float16);
    auto head8 = s.createTensor({64, 50}, DataType::Int8);
    auto sc8 = s.createTensor({2, 50}, DataType::Float16);
    EmbeddingColOpNode c0(s, idx, head16, head16);
    CHECK(c0.outputShape().back() == 6 && c0.outputDtype() == DataType::Float32);
    struct PC { uint32_t numIndices, embDim, vocabStride, scaleStride, outStride; } pc;
    auto bytes = c0.pushConstants();
    CHECK(bytes.size() == sizeof(pc));
    std::memcpy(&pc, bytes.data(), sizeof(pc));
    CHECK(pc.embDim == 6 && pc.vocabStride == 52 && pc.scaleStride == 52 && pc.outStride == 8);
    CHECK(KernelDesc::decode(*c0.shader())->fusionType == 0);
    EmbeddingColOpNode c1(s, idx, head8, sc8);
    CHECK(KernelDesc::decode(*c1.shader())->fusionType == 1 && KernelDesc::decode(*c1.shader())->op == EmbeddingCol);
    CHECK(c1.dispatchSize().x == (pc.numIndices * 64 + 255) / 256 * 256);
    CHECK_THROWS(EmbeddingColOpNode(s, idx, w, w), "matrix must be 2D");
    CHECK_THROWS(EmbeddingColOpNode(s, idx, s.createTensor({6, 50}, DataType::Float32), sc8), "Float16 or Int8");
  }

  GlobalReduceOpNode am(ReduceArgmax, s, s.createTensor({1, 1000}, DataType::Float32));
  CHECK(am.outputShape() == (std::vector<uint32_t>{1}) && am.dispatchSize().x == 256 && am.displayName() == "ReduceArgmax");
  uint32_t n = 0;
  CHECK(am.bindings().back().bytes.size() == 4);
  std::memcpy(&n, am.bindings().back().bytes.data(), 4);
  CHECK(n == 1000);
  CHECK(GlobalReduceOpNode(ReduceSum, s, x2).bindings().back().bytes.size() == 12);
  CHECK(am.shaderKey() != GlobalReduceOpNode(ReduceArgmin, s, x1).shaderKey());

  const size_t before = f.raw->modules;
  auto y = f.rt.ops().rmsNorm(x2, w);
  f.rt.ops().rmsNorm(x2, w);  // same kernel: one module
  auto emb = f.rt.ops().embedding(idx, table);
  auto arg = f.rt.ops().reduce(ReduceArgmin, x1);
  CHECK(f.raw->modules == before + 3);
  CHECK(f.rt.getTensor(y).getShape() == (std::vector<uint32_t>{3, 10}) && f.rt.getTensor(arg).getShape() == (std::vector<uint32_t>{1}));
  CHECK(f.rt.getTensor(emb).getShape() == (std::vector<uint32_t>{2, 5, 6}));
  CHECK_THROWS(f.rt.ops().reduce(ReduceSum, x1), "no shader");
  f.rt.flush();
  CHECK(f.raw->executed.size() == 4 && f.raw->executed[2].label == "Embedding" && f.raw->executed[3].label == "ReduceArgmin");
}

// AttentionOpNode / FusedRoPEKVWriteOpNode: geometry, push constants, keys, validation
void attentionNodes() {
  Fixture f;
  TensorStore &s = f.rt.store();
  const uint32_t nH = 8, nKv = 2, hd = 16, maxSeq = 32;
  auto q = s.createTensor({nH * hd}, DataType::Float32), k = s.createTensor({nKv * hd}, DataType::Float32);
  auto v = s.createTensor({nKv * hd}, DataType::Float32), params = s.createTensor({2}, DataType::UInt32);
  auto cosT = s.createTensor({maxSeq * hd / 2}, DataType::Float32), sinT = s.createTensor({maxSeq * hd / 2}, DataType::Float32);
  auto kc = s.createTensor({maxSeq, nKv * hd}, DataType::Float16), vc = s.createTensor({maxSeq, nKv * hd}, DataType::Float16);
  auto kc32 = s.createTensor({maxSeq, nKv * hd}, DataType::Float32), vc32 = s.createTensor({maxSeq, nKv * hd}, DataType::Float32);
  AttentionOpNode a(s, q, kc, vc, params, nH, nKv, hd);
  CHECK(a.op() == Attention && a.outputShape() == (std::vector<uint32_t>{nH * hd}) && a.outputDtype() == DataType::Float32);
  CHECK(a.dispatchSize().x == nH * 256 && a.displayName() == "Attention");
  struct {
    uint32_t nHeads, nKvHeads, headDim, kvDim, alignedKvDim, nRep;
    float scale;
  } pc;
  auto b = a.bindings();
  CHECK(b.size() == 6 && b[4].handle == a.output() && b[5].bytes.size() == sizeof(pc));
  std::memcpy(&pc, b[5].bytes.data(), sizeof(pc));
  CHECK(pc.nHeads == nH && pc.nKvHeads == nKv && pc.headDim == hd && pc.kvDim == 32 && pc.alignedKvDim == 32 && pc.nRep == 4);
  CHECK(pc.scale == 0.25f);
  CHECK(a.shaderKey() != AttentionOpNode(s, q, kc32, vc32, params, nH, nKv, hd).shaderKey());
  auto pre = s.createTensor({nH * hd}, DataType::Float32);
  CHECK(AttentionOpNode(s, q, kc, vc, params, nH, nKv, hd, pre).output() == pre);
  CHECK_THROWS(AttentionOpNode(s, q, kc, vc, params, nH, 3, hd), "multiple of nKvHeads");
  CHECK_THROWS(AttentionOpNode(s, q, kc, vc32, params, nH, nKv, hd), "share a dtype");
  CHECK(!AttentionOpNode(s, q, kc, vc, params, 18, 2, hd).shader().has_value());  // nine query heads per KV head

  FusedRoPEKVWriteOpNode r(s, q, k, v, params, cosT, sinT, kc, vc, hd);
  CHECK(r.op() == CacheWrite && r.outputShape() == (std::vector<uint32_t>{nH * hd}) && r.displayName() == "FusedRoPEKVWrite");
  CHECK(r.dispatchSize().x == 256 && r.bindings().size() == 10);  // 128 + 2 * 32 elements -> one group
  uint32_t rpc[5];
  std::memcpy(rpc, r.bindings().back().bytes.data(), sizeof(rpc));
  CHECK(rpc[0] == nH * hd && rpc[1] == nKv * hd && rpc[2] == hd && rpc[3] == hd / 2 && rpc[4] == 32);
  auto kd = KernelDesc::decode(*r.shader());
  CHECK(kd && kd->op == CacheWrite && kd->variant == FusedRoPEKVWriteOpNode::kVariant && kd->dtypeA == (uint32_t)DataType::Float16);
  CHECK(r.shaderKey() != FusedRoPEKVWriteOpNode(s, q, k, v, params, cosT, sinT, kc32, vc32, hd).shaderKey());
  CHECK_THROWS(FusedRoPEKVWriteOpNode(s, q, k, v, params, cosT, sinT, kc, vc, 6), "headDim must be even and divide");
  CHECK_THROWS(FusedRoPEKVWriteOpNode(s, q, k, q, params, cosT, sinT, kc, vc, hd), "k and v of one length");
  // prefill nodes: q / k / v as columns of one [T, 192] matrix
  const uint32_t T = 5, width = nH * hd + 2 * nKv * hd;
  auto qkv = s.createTensor({T, width}, DataType::Float32), posT = s.createTensor({T}, DataType::UInt32);
  BatchedKVCacheWriteOpNode bw(s, qkv, qkv, kc, vc, posT, cosT, sinT, T, nKv, hd, width, width, nH * hd, nH * hd + nKv * hd);
  CHECK(bw.op() == CacheWrite && bw.output() == kc && bw.dispatchSize().x == 256 && bw.dispatchSize().y == T);
  uint32_t bpc[9];
  std::memcpy(bpc, bw.bindings().back().bytes.data(), sizeof(bpc));
  CHECK(bpc[0] == T && bpc[1] == 32 && bpc[2] == 32 && bpc[3] == hd && bpc[4] == hd / 2 && bpc[5] == width && bpc[7] == nH * hd);
  CHECK(bw.shaderKey() != r.shaderKey() && KernelDesc::decode(*bw.shader())->variant == BatchedKVCacheWriteOpNode::kVariant);
  CHECK_THROWS(BatchedKVCacheWriteOpNode(s, qkv, qkv, kc, vc, posT, cosT, sinT, T, nKv, hd, 100, width, nH * hd, 0), "row stride is shorter");
  BatchedAttentionReadCacheOpNode ba(s, qkv, kc, vc, posT, cosT, sinT, T, nH, nKv, hd, width, 0);
  CHECK(ba.op() == Attention && ba.outputShape() == (std::vector<uint32_t>{T, nH * hd}) && ba.dispatchSize().y == T);
  CHECK(ba.shaderKey() != a.shaderKey() && ba.bindings().size() == 8 && ba.bindings().back().bytes.size() == 40);
  CHECK_THROWS(BatchedAttentionReadCacheOpNode(s, qkv, kc, vc, posT, cosT, sinT, T, nH, nKv, hd, 64, 0), "qStride is shorter");
  auto qr = f.rt.ops().fusedRoPEKVWrite(q, k, v, params, cosT, sinT, kc, vc, hd);
  auto out = f.rt.ops().attention(qr, kc, vc, params, nH, nKv, hd);
  f.rt.flush();
  CHECK(f.raw->executed.size() == 2 && f.raw->executed[0].label == "FusedRoPEKVWrite" && f.raw->executed[1].label == "Attention");
  CHECK(f.rt.getTensor(out).getShape() == (std::vector<uint32_t>{nH * hd}));
}

// GGUF header parsing (interface/loader/gguf/gguf_reader.cpp:15-58, 268-291): a file written here with every scalar
// metadata type, strings, arrays (skipped), a non-default alignment and three tensors.
void ggufFileParsing() {
  GGUFWriter w;
  w.put<uint32_t>(0x46554747u);
  w.put<uint32_t>(3);
  w.put<uint64_t>(3);   // tensors
  w.put<uint64_t>(9);   // metadata pairs
  w.str("general.alignment"); w.put<uint32_t>(4); w.put<uint32_t>(64);
  w.str("general.name"); w.put<uint32_t>(8); w.str("tiny");
  w.str("llama.block_count"); w.put<uint32_t>(4); w.put<uint32_t>(2);
  w.str("llama.rope.freq_base"); w.put<uint32_t>(6); w.put<float>(10000.0f);
  w.str("some.i8"); w.put<uint32_t>(1); w.put<int8_t>(-3);
  w.str("some.bool"); w.put<uint32_t>(7); w.put<uint8_t>(1);
  w.str("some.u64"); w.put<uint32_t>(10); w.put<uint64_t>(1ull << 40);
  w.str("tokens"); w.put<uint32_t>(9); w.put<uint32_t>(8); w.put<uint64_t>(3); w.str("a"); w.str("bc"); w.str("");  // array of strings
  w.str("scores"); w.put<uint32_t>(9); w.put<uint32_t>(6); w.put<uint64_t>(4); for (int i = 0; i < 4; ++i) w.put<float>(1.5f * i);
  // tensor directory: name, n_dims, dims (inner first), type, offset
  w.str("blk.0.attn_q.weight"); w.put<uint32_t>(2); w.put<uint64_t>(64); w.put<uint64_t>(3); w.put<uint32_t>(2); w.put<uint64_t>(0);     // Q4_0: 3 x 2 blocks = 108 B
  w.str("blk.0.ffn_down.weight"); w.put<uint32_t>(2); w.put<uint64_t>(256); w.put<uint64_t>(2); w.put<uint32_t>(14); w.put<uint64_t>(128);  // Q6_K: 2 x 210 B
  w.str("output_norm.weight"); w.put<uint32_t>(1); w.put<uint64_t>(8); w.put<uint32_t>(0); w.put<uint64_t>(576);                        // F32: 32 B
  const size_t dataStart = (w.b.size() + 63) / 64 * 64;
  w.b.resize(dataStart + 576 + 32);
  for (size_t i = dataStart; i < w.b.size(); ++i) w.b[i] = (uint8_t)(i * 7 + 1);
  const std::string path = "/tmp/cutb_host_logic_test.gguf";
  FILE *f = fopen(path.c_str(), "wb");
  CHECK(f != nullptr);
  fwrite(w.b.data(), 1, w.b.size(), f);
  fclose(f);

  GGUFFile g(path);
  CHECK(g.version() == 3 && g.alignment() == 64 && g.dataOffset() == dataStart && g.tensors().size() == 3);
  CHECK(*g.metaString("general.name") == "tiny" && *g.metaNumber("llama.block_count") == 2.0);
  CHECK(*g.metaNumber("llama.rope.freq_base") == 10000.0 && *g.metaNumber("some.i8") == -3.0 && *g.metaNumber("some.bool") == 1.0);
  CHECK(*g.metaNumber("some.u64") == (double)(1ull << 40) && !g.metaNumber("tokens") && !g.metaString("scores"));
  const auto &q = g.info("blk.0.attn_q.weight");
  CHECK(q.dims == (std::vector<uint64_t>{64, 3}) && q.type == 2 && q.bytes() == 108 && q.elements() == 192);
  CHECK(g.info("blk.0.ffn_down.weight").bytes() == 420 && g.info("output_norm.weight").bytes() == 32);
  const auto raw = g.readRaw("blk.0.ffn_down.weight");
  CHECK(raw.size() == 420 && raw[0] == (uint8_t)((dataStart + 128) * 7 + 1) && raw[419] == (uint8_t)((dataStart + 128 + 419) * 7 + 1));
  CHECK(g.has("output_norm.weight") && !g.has("nope"));
  CHECK_THROWS(g.info("nope"), "Tensor not found");
  CHECK(ggmlBlockGeometry(12)->second == 144 && !ggmlBlockGeometry(10) && *ggmlDequantFormat(6) == DequantFormat::Q5_0);
  // malformed files are refused
  {
    std::vector<uint8_t> bad = w.b;
    bad[0] = 'X';
    FILE *fb = fopen("/tmp/cutb_host_logic_bad.gguf", "wb");
    fwrite(bad.data(), 1, bad.size(), fb);
    fclose(fb);
    CHECK_THROWS(GGUFFile("/tmp/cutb_host_logic_bad.gguf"), "invalid magic");
    fb = fopen("/tmp/cutb_host_logic_bad.gguf", "wb");
    fwrite(w.b.data(), 1, dataStart + 100, fb);  // the second tensor would lie past the end
    fclose(fb);
    CHECK_THROWS(GGUFFile("/tmp/cutb_host_logic_bad.gguf"), "past the end");
    remove("/tmp/cutb_host_logic_bad.gguf");
  }
  remove(path.c_str());
}

int main() {
  RUN(attentionNodes);
  RUN(layerOperatorNodes);
  RUN(bufferGeometry);
  RUN(quantFormatDetectionAndVariants);
  RUN(shapeErrors);
  RUN(pushConstantsBindingsAndKeys);
  RUN(blockNodesAndDequant);
  RUN(blockMatmulOptionsAndGluPairs);
  RUN(dispatcherAndOperations);
  RUN(variantSelectorRules);
  RUN(ggufFileParsing);
  return finish();
}
