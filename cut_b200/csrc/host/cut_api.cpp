// Host logic of the operator API slice (see cut_api.h): buffer geometry, the
// three operator nodes of the quantized-matmul path, Dispatcher, VariantSelector,
// Operations and a minimal Runtime.  No CUDA in this file; the device work sits
// behind ComputeInterface (b200_compute.cpp) and, below that, the C ABI.
#include "cut_api.h"

#include <cmath>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <iterator>
#include <map>

namespace cut {

// ---------------------------------------------------------------------------
// core/api basics
// ---------------------------------------------------------------------------
size_t dataTypeSize(DataType t) {
  switch (t) {
    case DataType::Float32: case DataType::UInt32: case DataType::Int32: return 4;
    case DataType::Float16: return 2;
    case DataType::Int8: return 1;
  }
  return 4;
}

DataType widenPrecision(DataType t) { return t == DataType::Float16 ? DataType::Float32 : t; }

size_t ComputeHandle::id() const { return slot_ ? slot_->id : 0; }

size_t ComputeBuffer::calculateActualSize(const std::vector<uint32_t> &shape, DataType dtype) {
  if (shape.empty()) return 0;
  size_t n = 1;
  for (uint32_t d : shape) n *= d;
  return n * dataTypeSize(dtype);
}

// core/api/src/ComputeStructs.cpp:99-120: inner dimension to a multiple of 4 elements...
size_t ComputeBuffer::calculateAlignedElements(const std::vector<uint32_t> &shape) {
  if (shape.empty()) return 0;
  size_t n = 1;
  for (size_t i = 0; i + 1 < shape.size(); ++i) n *= shape[i];
  return n * ((shape.back() + 3u) & ~3u);
}

// ...and the byte size to a multiple of 16.
size_t ComputeBuffer::calculateAlignedSize(const std::vector<uint32_t> &shape, DataType dtype) {
  const size_t size = calculateAlignedElements(shape) * dataTypeSize(dtype);
  return (size + 15) & ~static_cast<size_t>(15);
}

void ComputeBuffer::describe(const std::vector<uint32_t> &shape, DataType dtype) {
  shape_ = shape;
  dtype_ = dtype;
  size_ = calculateAlignedSize(shape, dtype);
}

// Row-wise copies between the caller's dense layout and the padded device layout
// (core/api/src/ComputeInterface.cpp:134-145); padding is zero-filled by the caller.
void ComputeInterface::copyActualToAligned(const void *src, void *dst, const ComputeBuffer &b) {
  const auto &shape = b.getShape();
  if (shape.empty()) return;
  const size_t es = dataTypeSize(b.getDtype());
  const size_t inner = shape.back(), innerPad = (inner + 3) & ~size_t(3);
  size_t rows = 1;
  for (size_t i = 0; i + 1 < shape.size(); ++i) rows *= shape[i];
  for (size_t r = 0; r < rows; ++r)
    std::memcpy((uint8_t *)dst + r * innerPad * es, (const uint8_t *)src + r * inner * es, inner * es);
}

void ComputeInterface::copyAlignedToActual(const void *src, void *dst, const ComputeBuffer &b) {
  const auto &shape = b.getShape();
  if (shape.empty()) return;
  const size_t es = dataTypeSize(b.getDtype());
  const size_t inner = shape.back(), innerPad = (inner + 3) & ~size_t(3);
  size_t rows = 1;
  for (size_t i = 0; i + 1 < shape.size(); ++i) rows *= shape[i];
  for (size_t r = 0; r < rows; ++r)
    std::memcpy((uint8_t *)dst + r * inner * es, (const uint8_t *)src + r * innerPad * es, inner * es);
}

void ComputeInterface::encode(ComputeDispatch &&dispatch) { pending_.push_back(std::move(dispatch)); }

ComputeHandle ComputeInterface::submit() {
  std::vector<ComputeDispatch> work;
  work.swap(pending_);
  return executeDispatches(std::move(work), false);
}

ComputeHandle ComputeInterface::submitReusable() {
  std::vector<ComputeDispatch> work;
  work.swap(pending_);
  return executeDispatches(std::move(work), true);
}

void ComputeInterface::resubmit(const ComputeHandle &cb) { replay(cb); }
void ComputeInterface::wait(const ComputeHandle &cb) { waitFor(cb); }

// ---------------------------------------------------------------------------
// Kernel descriptors
// ---------------------------------------------------------------------------
std::vector<uint32_t> KernelDesc::encode() const {
  std::vector<uint32_t> w = {kMagic, op, variant, dtypeA, dtypeB, fusionType, fusionOp, affine, format};
  if (flags) w.push_back(flags);
  return w;
}

std::optional<KernelDesc> KernelDesc::decode(const std::vector<uint32_t> &w) {
  if ((w.size() != 9 && w.size() != 10) || w[0] != kMagic) return std::nullopt;
  KernelDesc d;
  d.op = w[1]; d.variant = w[2]; d.dtypeA = w[3]; d.dtypeB = w[4];
  d.fusionType = w[5]; d.fusionOp = w[6]; d.affine = w[7]; d.format = w[8];
  d.flags = w.size() == 10 ? w[9] : 0u;
  return d;
}

// ---------------------------------------------------------------------------
// Variant tables: the reference's names and indices
// (MatMulQ4Variants.generated.h:23-29, MatMulQ8Variants.generated.h:23-32).  Every
// plane-layout index is served by the same sm_100a plane kernel, so explicit
// `spec` values from reference callers and tests keep working.
// ---------------------------------------------------------------------------
const MatMulQVariantInfo kMatMulQ4Variants[kMatMulQ4VariantCount] = {
    {"MatMulQ4T16R4x4", 16, 16, 64, 64, "Q4 T16 R4x4"},
    {"MatMulQ4Gemv", 256, 1, 1, 256, "Q4 GEMV (M=1 vector)"},
    {"MatMulQ4GemvKPar", 32, 1, 1, 4, "Q4 GEMV K-parallel"},
    {"MatMulQ4GemvKPar8", 32, 8, 1, 8, "Q4 GEMV (M=1, 8 cols/WG)"},
    {"MatMulQ4CoopMatTiled", 128, 1, 32, 32, "Q4 tensor-core tiled"},
};
const MatMulQVariantInfo kMatMulQ8Variants[kMatMulQ8VariantCount] = {
    {"MatMulQ8T16R4x4", 16, 16, 64, 64, "Q8 T16 R4x4"},
    {"MatMulQ8Gemv", 256, 1, 1, 256, "Q8 GEMV (M=1 vector)"},
    {"MatMulQ8VecT16R4x4", 16, 16, 64, 64, "Q8 Vec4 T16 R4x4"},
    {"MatMulQ8GemvKPar", 32, 1, 1, 4, "Q8 GEMV K-parallel"},
    {"MatMulQ8GemvKPar8", 32, 8, 1, 8, "Q8 GEMV (M=1, 8 cols/WG)"},
    {"MatMulQ8GemvDot", 32, 1, 1, 4, "Q8 GEMV packed dot"},
    {"MatMulQ8TiledDot", 256, 1, 32, 64, "Q8 tiled packed dot"},
    {"MatMulQ8CoopMatTiled", 128, 1, 32, 32, "Q8 tensor-core tiled"},
};
const MatMulQVariantInfo kMatMulQBlocksVariants[kMatMulQBlocksVariantCount] = {
    {"QMatMulGeneric", 256, 1, 8, 8, "any shape, SIMT"},
    {"QGemvBulkMma", 544, 1, 16, 16, "decode: bulk-copy ring + int8 warp MMA, one persistent CTA per SM"},
    {"QGemmTcgen05", 192, 1, 128, 128, "prefill: tcgen05 tensor-core GEMM, accumulators in tensor memory"},
};

const char *getMatMulQ4VariantName(int i) {
  return (i < 0 || i >= kMatMulQ4VariantCount) ? "Unknown" : kMatMulQ4Variants[i].name;
}
const char *getMatMulQ8VariantName(int i) {
  return (i < 0 || i >= kMatMulQ8VariantCount) ? "Unknown" : kMatMulQ8Variants[i].name;
}

static std::optional<std::vector<uint32_t>> compiledPlane(OperatorEnum op, int variant, int count, DataType in1,
                                                          DataType scales, DataType out) {
  if (variant < 0 || variant >= count) return std::nullopt;
  // compiled combinations: activation fp32 or fp16, fp16 scales, fp32 output
  if ((in1 != DataType::Float32 && in1 != DataType::Float16) || scales != DataType::Float16 || out != DataType::Float32)
    return std::nullopt;
  KernelDesc d;
  d.op = op;
  d.variant = (uint32_t)variant;
  d.dtypeA = (uint32_t)in1;
  d.dtypeB = (uint32_t)scales;
  return d.encode();
}

std::optional<std::vector<uint32_t>> getCompiledMatMulQ4(int v, DataType in1, DataType scales, DataType out) {
  return compiledPlane(MatMulQ4, v, kMatMulQ4VariantCount, in1, scales, out);
}
std::optional<std::vector<uint32_t>> getCompiledMatMulQ8(int v, DataType in1, DataType scales, DataType out) {
  if (v == 6) return std::nullopt;  // TiledDot: known wrong in the reference (MatMulOp.cpp:343-345), not provided
  return compiledPlane(MatMulQ8, v, kMatMulQ8VariantCount, in1, scales, out);
}

// ---------------------------------------------------------------------------
// OpNode
// ---------------------------------------------------------------------------
std::vector<ComputeBinding> OpNode::bindings() const {
  std::vector<ComputeBinding> result;
  uint32_t idx = 0;
  for (const auto &h : inputs_) result.emplace_back(idx++, h);
  if (output_) result.emplace_back(idx++, output_);
  auto pc = pushConstants();
  if (!pc.empty()) result.emplace_back(idx, pc.data(), (uint32_t)pc.size());
  return result;
}

// ---------------------------------------------------------------------------
// MatMulOpNode (operators/impl/matmul/MatMulOp.cpp:271-617)
// ---------------------------------------------------------------------------
MatMulOpNode::MatMulOpNode(TensorStore &store, const Tensor &a, const Tensor &packedB, const Tensor &scalesB,
                           std::optional<uint32_t> spec)
    : OpNode(MatMul, store, spec) {
  const auto &bufA = store.getTensor(a);
  const auto &bufPB = store.getTensor(packedB);
  const auto &bufSB = store.getTensor(scalesB);
  const auto shapeA = bufA.getShape(), shapePB = bufPB.getShape(), shapeSB = bufSB.getShape();
  dtypeA_ = bufA.getDtype();
  dtypeB_ = bufSB.getDtype();
  if (shapePB.size() != 2 || shapeSB.size() != 2) throw std::runtime_error("matmul requires 2D B and scales matrices");
  if (shapeA.size() == 1) {
    M_ = 1;
    K_ = shapeA[0];
  } else if (shapeA.size() == 2) {
    M_ = shapeA[0];
    K_ = shapeA[1];
  } else {
    throw std::runtime_error("matmul: A must be 1D or 2D");
  }
  if (shapePB[0] != K_)
    throw std::runtime_error("matmul: B rows (" + std::to_string(shapePB[0]) + ") must match A cols (" +
                             std::to_string(K_) + ")");
  const uint32_t bCols = shapePB[1], sCols = shapeSB[1];
  if (bCols == sCols) {
    format_ = QuantFormat::Q8;
    N_ = bCols;
  } else if (bCols * 2 == sCols) {
    format_ = QuantFormat::Q4;
    N_ = sCols;
    q4Affine_ = (shapeSB[0] == 2u * ((K_ + 31u) / 32u));
  } else {
    throw std::runtime_error("matmul: cannot determine quant format from B cols (" + std::to_string(bCols) +
                             ") and scales cols (" + std::to_string(sCols) + ")");
  }
  op_ = format_ == QuantFormat::Q8 ? MatMulQ8 : MatMulQ4;
  autoSpec_ = !spec.has_value();
  // built-in choice, same indices as the reference (MatMulOp.cpp:335-380)
  if (format_ == QuantFormat::Q8)
    fusionFallbackSpec_ = (M_ == 1) ? ((N_ >= 8) ? 4 : 3) : (uint32_t)kMatMulQ8DefaultVariant;
  else
    fusionFallbackSpec_ = (M_ == 1) ? ((N_ >= 8) ? 3 : 2) : (uint32_t)kMatMulQ4DefaultVariant;
  uint32_t builtin = fusionFallbackSpec_;
  const bool tc = M_ > 1 && store.caps().cooperativeMatrix && dtypeB_ == DataType::Float16 && K_ % 16 == 0 && N_ % 32 == 0;
  if (tc) builtin = format_ == QuantFormat::Q8 ? (uint32_t)kMatMulQ8VariantCount - 1 : 4u;
  if (spec.has_value()) {
    spec_ = *spec;
  } else {
    // tuning_data.json rules win over the built-in choice when present
    const char *name = format_ == QuantFormat::Q8 ? "MatMulQ8" : "MatMulQ4";
    spec_ = (uint32_t)VariantSelector::instance().select(name, {M_, K_, N_}, (int)builtin,
                                                          backendName(store.caps().backend));
  }
  const int count = format_ == QuantFormat::Q8 ? kMatMulQ8VariantCount : kMatMulQ4VariantCount;
  if ((int)*spec_ >= count) throw std::runtime_error("matmul: variant index " + std::to_string(*spec_) + " out of range");
  inputs_ = {a, packedB, scalesB};
  output_ = store.createTensorEmpty(outputShape(), outputDtype());
}

static uint32_t blockElems(DequantFormat f) { return f == DequantFormat::Q4_K ? 256u : 32u; }
static uint32_t blockBytes(DequantFormat f) {
  return f == DequantFormat::Q8_0 ? 34u : (f == DequantFormat::Q4_0 ? 18u : 144u);
}
static bool isBlockFormat(DequantFormat f) {
  return f == DequantFormat::Q8_0 || f == DequantFormat::Q4_0 || f == DequantFormat::Q4_K;
}

MatMulOpNode::MatMulOpNode(TensorStore &store, const Tensor &a, const Tensor &rawB, DequantFormat blockFormat, uint32_t N,
                           std::optional<uint32_t> spec)
    : OpNode(MatMulQBlocks, store, spec), format_(QuantFormat::Blocks), blockFormat_(blockFormat) {
  if (!isBlockFormat(blockFormat)) throw std::runtime_error("matmul: block format must be Q8_0, Q4_0 or Q4_K");
  const auto &bufA = store.getTensor(a);
  const auto &bufB = store.getTensor(rawB);
  const auto shapeA = bufA.getShape();
  dtypeA_ = bufA.getDtype();
  dtypeB_ = DataType::Float16;
  if (shapeA.size() == 1) {
    M_ = 1;
    K_ = shapeA[0];
  } else if (shapeA.size() == 2) {
    M_ = shapeA[0];
    K_ = shapeA[1];
  } else {
    throw std::runtime_error("matmul: A must be 1D or 2D");
  }
  N_ = N;
  if (bufB.getShape().size() != 1 || bufB.getDtype() != DataType::Int8)
    throw std::runtime_error("matmul: raw block weights must be a 1D Int8 tensor");
  if (K_ % blockElems(blockFormat) != 0)
    throw std::runtime_error("matmul: A cols (" + std::to_string(K_) + ") must be a multiple of the block size (" +
                             std::to_string(blockElems(blockFormat)) + ")");
  const size_t need = (size_t)N_ * (K_ / blockElems(blockFormat)) * blockBytes(blockFormat);
  if (bufB.getShape()[0] < need)
    throw std::runtime_error("matmul: raw block tensor holds " + std::to_string(bufB.getShape()[0]) + " bytes, " +
                             std::to_string(N_) + " rows of " + std::to_string(K_) + " weights need " +
                             std::to_string(need));
  autoSpec_ = !spec.has_value();
  // decode shapes -> bulk-copy MMA mat-vec, prefill shapes -> tensor-core GEMM, the rest -> SIMT
  const uint32_t vrows = dtypeA_ == DataType::Float32 ? 2 * M_ : M_;
  uint32_t builtin = 0;
  if (K_ % 256 == 0 && vrows <= 16) builtin = 1;
  else if (K_ % 256 == 0 && M_ > 1 && store.caps().cooperativeMatrix) builtin = 2;
  // 13 to 16 fp16 rows on 16 M weights or more: the tensor-core GEMM for few tokens beats the mat-vec's fourth
  // column tile (the library's own automatic choice makes the same cut)
  if (builtin == 1 && dtypeA_ == DataType::Float16 && M_ >= 13 && (uint64_t)K_ * N_ >= (1ull << 24) &&
      store.caps().cooperativeMatrix)
    builtin = 2;
  fusionFallbackSpec_ = builtin;
  if (spec.has_value()) spec_ = *spec;
  else
    spec_ = (uint32_t)VariantSelector::instance().select("MatMulQBlocks", {M_, K_, N_}, (int)builtin,
                                                          backendName(store.caps().backend));
  if ((int)*spec_ >= kMatMulQBlocksVariantCount)
    throw std::runtime_error("matmul: variant index " + std::to_string(*spec_) + " out of range");
  inputs_ = {a, rawB};
  output_ = store.createTensorEmpty(outputShape(), outputDtype());
}

void MatMulOpNode::setFusion(MatMulFusion fusion, OperatorEnum fusionOp, const Tensor &d) {
  fusion_ = fusion;
  fusionOp_ = fusionOp;
  if (fusion == MatMulFusion::Binary) {
    if (!d) throw std::runtime_error("matmul: binary fusion needs the D operand");
    const auto &bd = store_->getTensor(d);
    const auto sd = bd.getShape();
    const bool ok = (sd.size() == 2 && sd[0] == M_ && sd[1] == N_) || (sd.size() == 1 && M_ == 1 && sd[0] == N_);
    if (!ok || bd.getDtype() != DataType::Float32) throw std::runtime_error("matmul: D must be Float32 [M, N]");
    inputs_.push_back(d);
  }
  // every variant of this backend has the fused epilogue: no fallback needed
  // (the reference falls back for float cooperative-matrix variants only, MatMulOp.cpp:400-417)
}

void MatMulOpNode::setBlockOptions(const MatMulBlockOptions &opt) {
  if (format_ != QuantFormat::Blocks) throw std::runtime_error("matmul: block options need the raw-block constructor");
  if (opt.flags & ~(kBlockFlagNoOverlap | kBlockFlagAct16 | kBlockFlagRmsNorm | kBlockFlagGluPairs))
    throw std::runtime_error("matmul: unknown block option bits");
  if (opt.flags & kBlockFlagRmsNorm) {
    // only the decode mat-vec has it (variant 1: K % 256 == 0, at most 16 virtual activation rows); an automatic
    // choice that went elsewhere for speed comes back to it
    const uint32_t vrows = dtypeA_ == DataType::Float32 ? 2 * M_ : M_;
    if (*spec_ != 1 && autoSpec_ && K_ % 256 == 0 && vrows <= 16) spec_ = 1;
    if (*spec_ != 1) throw std::runtime_error("matmul: the fused RMSNorm exists in the decode mat-vec only");
  }
  if ((opt.flags & kBlockFlagGluPairs) && *spec_ != 1 && *spec_ != 2)
    throw std::runtime_error("matmul: paired rows exist in the decode mat-vec and the tensor-core GEMM only");
  if (opt.flags & kBlockFlagGluPairs) {
    if (fusion_ != MatMulFusion::Unary) throw std::runtime_error("matmul: paired gate/up rows need a unary fusion");
    if (N_ % 2) throw std::runtime_error("matmul: paired gate/up rows need an even N");
  }
  if (opt.flags & kBlockFlagRmsNorm) {
    if (!opt.normWeight) throw std::runtime_error("matmul: fused RMSNorm needs its weight");
    const auto &w = store_->getTensor(opt.normWeight);
    if (w.getDtype() != DataType::Float32 || w.getShape().size() != 1 || w.getShape()[0] != K_)
      throw std::runtime_error("matmul: the RMSNorm weight must be Float32 [K]");
    inputs_.push_back(opt.normWeight);  // binds after D
    normEps_ = opt.normEps;
  }
  blockFlags_ = opt.flags;
  if (opt.flags & kBlockFlagGluPairs) output_ = store_->createTensorEmpty(outputShape(), outputDtype());
}

size_t MatMulOpNode::shaderKey() const {
  size_t key = static_cast<size_t>(op_);
  key |= (static_cast<size_t>(dtypeA_) & 0xF) << 16;
  key |= (static_cast<size_t>(dtypeB_) & 0xF) << 20;
  if (format_ == QuantFormat::Blocks) key |= (static_cast<size_t>(blockFormat_) & 0x1F) << 24;
  key |= (static_cast<size_t>(blockFlags_) & 0xF) << 29;
  key |= (static_cast<size_t>(q4Affine_ ? 1 : 0)) << 35;
  key |= (static_cast<size_t>(fusion_) & 0xF) << 36;
  if (fusion_ != MatMulFusion::None) key |= (static_cast<size_t>(fusionOp_) & 0xFF) << 40;
  key |= static_cast<size_t>(spec_.value_or(0)) << 48;
  return key;
}

std::optional<std::vector<uint32_t>> MatMulOpNode::shader() const {
  std::optional<std::vector<uint32_t>> compiled;
  if (format_ == QuantFormat::Q8) compiled = getCompiledMatMulQ8((int)*spec_, dtypeA_, dtypeB_, DataType::Float32);
  else if (format_ == QuantFormat::Q4) compiled = getCompiledMatMulQ4((int)*spec_, dtypeA_, dtypeB_, DataType::Float32);
  else {
    KernelDesc d;
    d.op = MatMulQBlocks;
    d.variant = *spec_;
    d.dtypeA = (uint32_t)dtypeA_;
    d.dtypeB = (uint32_t)dtypeB_;
    d.format = (uint32_t)blockFormat_;
    compiled = d.encode();
  }
  if (!compiled) return compiled;
  // the specialisation constants of the reference (1, 2: fusion; 3: affine) live in the descriptor
  auto d = *KernelDesc::decode(*compiled);
  d.fusionType = (uint32_t)fusion_;
  d.fusionOp = fusion_ != MatMulFusion::None ? (uint32_t)fusionOp_ : 0u;
  d.affine = q4Affine_ ? 1u : 0u;
  d.flags = blockFlags_;
  return d.encode();
}

ThreadSize MatMulOpNode::dispatchSize() const {
  const MatMulQVariantInfo &vi = format_ == QuantFormat::Q8   ? kMatMulQ8Variants[*spec_]
                                 : format_ == QuantFormat::Q4 ? kMatMulQ4Variants[*spec_]
                                                              : kMatMulQBlocksVariants[*spec_];
  const uint32_t gridX = ((N_ + vi.effTileN - 1) / vi.effTileN) * vi.wgX;
  const uint32_t gridY = ((M_ + vi.effTileM - 1) / vi.effTileM) * vi.wgY;
  return {gridX, gridY, 1};
}

std::vector<uint8_t> MatMulOpNode::pushConstants() const {
  // {M, K, N, strideA, strideB, strideC, scaleStride}, strides padded to 4 (MatMulOp.cpp:507-541)
  const uint32_t strideA = (K_ + 3) & ~3u;
  uint32_t strideB = (N_ + 3) & ~3u;
  if (format_ == QuantFormat::Q4) strideB = (N_ / 2 + 3) & ~3u;
  if (format_ == QuantFormat::Blocks) strideB = (K_ / blockElems(blockFormat_)) * blockBytes(blockFormat_);
  const uint32_t nOut = (blockFlags_ & kBlockFlagGluPairs) ? N_ / 2 : N_;
  const uint32_t strideC = (nOut + 3) & ~3u, scaleStride = (N_ + 3) & ~3u;
  struct {
    uint32_t M, K, N, strideA, strideB, strideC, scaleStride;
  } pc{M_, K_, N_, strideA, strideB, strideC, scaleStride};
  if (blockFlags_ & kBlockFlagRmsNorm) {  // one more word: the epsilon
    struct {
      uint32_t M, K, N, strideA, strideB, strideC, scaleStride;
      float normEps;
    } pcn{M_, K_, N_, strideA, strideB, strideC, scaleStride, normEps_};
    return toBytes(pcn);
  }
  return toBytes(pc);
}

std::vector<ComputeBinding> MatMulOpNode::bindings() const {
  // (A, packedB, [scalesB], D or a dummy, C, push constants) as in MatMulOp.cpp:543-575
  std::vector<ComputeBinding> result;
  uint32_t idx = 0;
  for (const auto &h : inputs_) result.emplace_back(idx++, h);
  if (fusion_ != MatMulFusion::Binary) result.emplace_back(idx++, output_);
  result.emplace_back(idx++, output_);
  auto pc = pushConstants();
  result.emplace_back(idx, pc.data(), (uint32_t)pc.size());
  return result;
}

std::string MatMulOpNode::displayName() const {
  std::string name = format_ == QuantFormat::Q8 ? "MatMulQ8" : format_ == QuantFormat::Q4 ? "MatMulQ4" : "MatMulQBlocks";
  if (fusion_ == MatMulFusion::Unary) name += "Unary";
  if (fusion_ == MatMulFusion::Binary) name += "Binary";
  return name;
}

std::vector<DataType> MatMulOpNode::resolveInputDtypes(const std::vector<DataType> &in) const {
  // Float16 activations have compiled kernels here, so nothing is widened except D
  std::vector<DataType> out = in;
  const size_t dIdx = format_ == QuantFormat::Blocks ? 2 : 3;
  if (fusion_ == MatMulFusion::Binary && out.size() > dIdx) out[dIdx] = widenPrecision(out[dIdx]);
  return out;
}

// ---------------------------------------------------------------------------
// DequantOpNode / TransposeQ4NibbleOpNode
// ---------------------------------------------------------------------------
DequantOpNode::DequantOpNode(TensorStore &store, const Tensor &rawData, DequantFormat format, uint32_t rows, uint32_t cols,
                             std::optional<uint32_t> spec)
    : OpNode(Dequantize, store, spec), format_(format), rows_(rows), cols_(cols) {
  outputStride_ = (cols_ + 3) & ~3u;
  inputs_ = {rawData};
  output_ = store.createTensorEmpty({rows_, cols_}, DataType::Float32);
}

RequantQ8BlocksOpNode::RequantQ8BlocksOpNode(TensorStore &store, const Tensor &rawData, DequantFormat format, uint32_t rows,
                                             uint32_t cols, std::optional<uint32_t> spec)
    : OpNode(RequantQ8Blocks, store, spec), format_(format), rows_(rows), cols_(cols) {
  const auto &raw = store.getTensor(rawData);
  if (raw.getDtype() != DataType::Int8 || raw.getShape().size() != 1)
    throw std::runtime_error("requantQ8Blocks: raw data must be a 1D Int8 tensor");
  if (cols % 32 != 0) throw std::runtime_error("requantQ8Blocks: cols must be a multiple of 32");
  inputs_ = {rawData};
  output_ = store.createTensorEmpty(outputShape(), DataType::Int8);
}

std::optional<std::vector<uint32_t>> RequantQ8BlocksOpNode::shader() const {
  switch (format_) {
    case DequantFormat::BF16: case DequantFormat::Q4_K: case DequantFormat::Q5_K: case DequantFormat::Q6_K:
    case DequantFormat::Q8_0: case DequantFormat::Q4_0: case DequantFormat::Q4_1: case DequantFormat::Q5_0: break;
    default: return std::nullopt;
  }
  KernelDesc d;
  d.op = RequantQ8Blocks;
  d.format = (uint32_t)format_;
  d.dtypeA = d.dtypeB = (uint32_t)DataType::Int8;
  return d.encode();
}

std::vector<uint8_t> RequantQ8BlocksOpNode::pushConstants() const {
  struct {
    uint32_t rows, cols;
  } pc{rows_, cols_};
  return toBytes(pc);
}

GluPairsOpNode::GluPairsOpNode(TensorStore &store, const Tensor &in, OperatorEnum unaryOp, std::optional<uint32_t> spec)
    : OpNode(GluPairs, store, spec), unaryOp_(unaryOp) {
  const auto &b = store.getTensor(in);
  const auto sh = b.getShape();
  if (b.getDtype() != DataType::Float32 || sh.empty() || sh.size() > 2) throw std::runtime_error("gluPairs: input must be Float32 [rows, 2F]");
  rows_ = sh.size() == 2 ? sh[0] : 1;
  const uint32_t colsIn = sh.back();
  if (colsIn % 2) throw std::runtime_error("gluPairs: the input needs an even number of columns");
  colsOut_ = colsIn / 2;
  strideIn_ = b.innerDimPadded();
  strideOut_ = (colsOut_ + 3) & ~3u;
  inputs_ = {in};
  output_ = store.createTensorEmpty(outputShape(), DataType::Float32);
}

std::optional<std::vector<uint32_t>> GluPairsOpNode::shader() const {
  KernelDesc d;
  d.op = GluPairs;
  d.fusionType = (uint32_t)MatMulFusion::Unary;
  d.fusionOp = (uint32_t)unaryOp_;
  d.dtypeA = d.dtypeB = (uint32_t)DataType::Float32;
  return d.encode();
}

std::vector<uint8_t> GluPairsOpNode::pushConstants() const {
  struct {
    uint32_t rows, colsOut, strideIn, strideOut;
  } pc{rows_, colsOut_, strideIn_, strideOut_};
  return toBytes(pc);
}

size_t DequantOpNode::shaderKey() const {
  return static_cast<size_t>(op_) | ((static_cast<size_t>(format_) & 0x1F) << 16);
}

std::optional<std::vector<uint32_t>> DequantOpNode::shader() const {
  switch (format_) {  // the reference's DequantFormat set plus the 32-weight block formats
    case DequantFormat::BF16: case DequantFormat::Q4_K: case DequantFormat::Q5_K: case DequantFormat::Q6_K:
    case DequantFormat::Q8_0: case DequantFormat::Q4_0: case DequantFormat::Q4_1: case DequantFormat::Q5_0: break;
    default: return std::nullopt;
  }
  KernelDesc d;
  d.op = Dequantize;
  d.format = (uint32_t)format_;
  d.dtypeA = (uint32_t)DataType::Int8;
  d.dtypeB = (uint32_t)DataType::Float32;
  return d.encode();
}

std::vector<uint8_t> DequantOpNode::pushConstants() const {
  struct {
    uint32_t rows, cols, outputStride;
  } pc{rows_, cols_, outputStride_};
  return toBytes(pc);
}

TransposeQ4NibbleOpNode::TransposeQ4NibbleOpNode(TensorStore &store, const Tensor &packedInput, uint32_t N, uint32_t K,
                                                 std::optional<uint32_t> spec)
    : OpNode(TransposeQ4, store, spec), N_(N), K_(K) {
  if (N_ % 2 != 0) throw std::runtime_error("TransposeQ4: N must be even");
  if (K_ % 32 != 0) throw std::runtime_error("TransposeQ4: K must be a multiple of 32");
  strideInHalf_ = (K_ / 2 + 3) & ~3u;
  strideOutHalf_ = (N_ / 2 + 3) & ~3u;
  inputs_ = {packedInput};
  output_ = store.createTensorEmpty({K_, N_ / 2}, DataType::Int8);
}

std::optional<std::vector<uint32_t>> TransposeQ4NibbleOpNode::shader() const {
  KernelDesc d;
  d.op = TransposeQ4;
  d.dtypeA = d.dtypeB = (uint32_t)DataType::Int8;
  return d.encode();
}

ThreadSize TransposeQ4NibbleOpNode::dispatchSize() const {
  const uint32_t wordsPerRow = (N_ / 2 + 3) / 4;
  return {((wordsPerRow + 63) / 64) * 64, ((K_ + 3) / 4) * 4, 1};
}

std::vector<uint8_t> TransposeQ4NibbleOpNode::pushConstants() const {
  struct {
    uint32_t N, K, strideInHalf, strideOutHalf;
  } pc{N_, K_, strideInHalf_, strideOutHalf_};
  return toBytes(pc);
}

// ---------------------------------------------------------------------------
// RMSNormOpNode / EmbeddingOpNode / GlobalReduceOpNode: the layer operators next to the matmul
// ---------------------------------------------------------------------------
RMSNormOpNode::RMSNormOpNode(TensorStore &store, const Tensor &x, const Tensor &weight, float eps,
                             std::optional<uint32_t> spec)
    : OpNode(RMSNorm, store, spec), eps_(eps) {
  const auto &bx = store.getTensor(x);
  const auto &bw = store.getTensor(weight);
  const auto &sx = bx.getShape();
  const auto &sw = bw.getShape();
  dtype_ = bx.getDtype();
  if (sx.empty() || sx.size() > 2 || sw.size() != 1) throw std::runtime_error("RMSNorm requires 1D or 2D input, 1D weight");
  batchSize_ = sx.size() == 2 ? sx[0] : 1;
  dim_ = sx.back();
  if (sw[0] != dim_) throw std::runtime_error("RMSNorm: weight dimension must match input");
  if (bw.getDtype() != dtype_) throw std::runtime_error("RMSNorm: weight must have same dtype as input");
  alignedDim_ = (dim_ + 3) & ~3u;
  inputs_ = {x, weight};
  output_ = store.createTensorEmpty(outputShape(), dtype_);
}

std::vector<uint32_t> RMSNormOpNode::outputShape() const {
  if (batchSize_ > 1) return {batchSize_, dim_};
  return {dim_};
}

std::optional<std::vector<uint32_t>> RMSNormOpNode::shader() const {
  if (dtype_ != DataType::Float32 && dtype_ != DataType::Float16) return std::nullopt;
  KernelDesc d;
  d.op = RMSNorm;
  d.dtypeA = d.dtypeB = (uint32_t)dtype_;
  return d.encode();
}

std::vector<uint8_t> RMSNormOpNode::pushConstants() const {
  struct {
    uint32_t dim, alignedDim;
    float eps;
  } pc{dim_, alignedDim_, eps_};
  return toBytes(pc);
}

EmbeddingOpNode::EmbeddingOpNode(TensorStore &store, const Tensor &indices, const Tensor &weight,
                                 const Tensor &preallocOutput, std::optional<uint32_t> spec)
    : OpNode(Embedding, store, spec) {
  const auto &bi = store.getTensor(indices);
  const auto &bw = store.getTensor(weight);
  dtype_ = bw.getDtype();
  if (bw.getShape().size() != 2)
    throw std::runtime_error("embedding: weight must be 2D [num_embeddings, embedding_dim]");
  embDim_ = bw.getShape()[1];
  for (uint32_t d : bi.getShape()) numIndices_ *= d;
  outShape_ = bi.getShape();
  outShape_.push_back(embDim_);
  inputs_ = {indices, weight};
  output_ = preallocOutput ? preallocOutput : store.createTensorEmpty(outShape_, dtype_);
}

std::optional<std::vector<uint32_t>> EmbeddingOpNode::shader() const {
  if (dtype_ != DataType::Float32) return std::nullopt;  // the table kernel gathers fp32 rows
  KernelDesc d;
  d.op = Embedding;
  d.dtypeA = d.dtypeB = (uint32_t)dtype_;
  return d.encode();
}

ThreadSize EmbeddingOpNode::dispatchSize() const {
  const uint32_t vec4PerRow = ((embDim_ + 3) & ~3u) / 4;
  return {(numIndices_ * vec4PerRow + 255) / 256 * 256, 1, 1};
}

std::vector<uint8_t> EmbeddingOpNode::pushConstants() const {
  struct {
    uint32_t numIndices, embDim;
  } pc{numIndices_, embDim_};
  return toBytes(pc);
}

EmbeddingColOpNode::EmbeddingColOpNode(TensorStore &store, const Tensor &indices, const Tensor &matrix, const Tensor &scales,
                                       const Tensor &preallocOutput, std::optional<uint32_t> spec)
    : OpNode(EmbeddingCol, store, spec) {
  const auto &bi = store.getTensor(indices);
  const auto &bm = store.getTensor(matrix);
  const auto &bs = store.getTensor(scales);
  if (bm.getShape().size() != 2) throw std::runtime_error("embeddingCol: matrix must be 2D [dim, vocab]");
  embDim_ = bm.getShape()[0];
  vocabStride_ = (bm.getShape()[1] + 3) & ~3u;
  scaleStride_ = bs.getShape().size() == 2 ? ((bs.getShape()[1] + 3) & ~3u) : vocabStride_;
  outStride_ = (embDim_ + 3) & ~3u;
  for (uint32_t d : bi.getShape()) numIndices_ *= d;
  format_ = bm.getDtype() == DataType::Int8 ? 1 : 0;
  if (bm.getDtype() != DataType::Float16 && bm.getDtype() != DataType::Int8)
    throw std::runtime_error("embeddingCol: matrix must be Float16 or Int8");
  outShape_ = bi.getShape();
  outShape_.push_back(embDim_);
  inputs_ = {indices, matrix, scales};
  output_ = preallocOutput ? preallocOutput : store.createTensorEmpty(outShape_, DataType::Float32);
}

std::optional<std::vector<uint32_t>> EmbeddingColOpNode::shader() const {
  KernelDesc d;
  d.op = EmbeddingCol;
  d.dtypeA = (uint32_t)DataType::UInt32;
  d.dtypeB = (uint32_t)DataType::Float32;
  d.fusionType = format_;  // specialisation constant 1, as in the reference: 0 = fp16 matrix, 1 = int8 + fp16 scales
  return d.encode();
}

ThreadSize EmbeddingColOpNode::dispatchSize() const {
  const uint32_t total = numIndices_ * embDim_;
  return {(total + 255) / 256 * 256, 1, 1};
}

std::vector<uint8_t> EmbeddingColOpNode::pushConstants() const {
  struct {
    uint32_t numIndices, embDim, vocabStride, scaleStride, outStride;
  } pc{numIndices_, embDim_, vocabStride_, scaleStride_, outStride_};
  return toBytes(pc);
}

GlobalReduceOpNode::GlobalReduceOpNode(OperatorEnum op, TensorStore &store, const Tensor &a, std::optional<uint32_t> spec)
    : OpNode(op, store, spec) {
  const auto &b = store.getTensor(a);
  dtype_ = b.getDtype();
  numElements_ = 1;
  for (uint32_t d : b.getShape()) numElements_ *= d;
  actualInner_ = b.innerDimSize();
  alignedInner_ = b.innerDimPadded();
  inputs_ = {a};
  output_ = store.createTensorEmpty({1}, dtype_);
}

std::optional<std::vector<uint32_t>> GlobalReduceOpNode::shader() const {
  if ((op_ != ReduceArgmax && op_ != ReduceArgmin) || dtype_ != DataType::Float32) return std::nullopt;
  KernelDesc d;
  d.op = op_;
  d.dtypeA = d.dtypeB = (uint32_t)dtype_;
  return d.encode();
}

std::vector<uint8_t> GlobalReduceOpNode::pushConstants() const {
  if (op_ == ReduceArgmax || op_ == ReduceArgmin) return toBytes(static_cast<uint32_t>(numElements_));
  struct {
    uint32_t numElements, actualInner, alignedInner;
  } pc{static_cast<uint32_t>(numElements_), actualInner_, alignedInner_};
  return toBytes(pc);
}

std::string GlobalReduceOpNode::displayName() const {
  switch (op_) {
    case ReduceArgmax: return "ReduceArgmax";
    case ReduceArgmin: return "ReduceArgmin";
    case ReduceSum: return "ReduceSum";
    case ReduceMean: return "ReduceMean";
    case ReduceMin: return "ReduceMin";
    case ReduceMax: return "ReduceMax";
    default: return "Reduce";
  }
}

AttentionOpNode::AttentionOpNode(TensorStore &store, const Tensor &q, const Tensor &kCache, const Tensor &vCache,
                                 const Tensor &runtimeParams, uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim,
                                 const Tensor &preallocOutput, std::optional<uint32_t> spec)
    : OpNode(Attention, store, spec), nHeads_(nHeads), nKvHeads_(nKvHeads), headDim_(headDim) {
  if (nHeads == 0 || nKvHeads == 0 || headDim == 0 || nHeads % nKvHeads != 0)
    throw std::runtime_error("attention: nHeads must be a positive multiple of nKvHeads and headDim positive");
  dtype_ = store.getTensor(kCache).getDtype();
  if (store.getTensor(vCache).getDtype() != dtype_) throw std::runtime_error("attention: K and V caches must share a dtype");
  kvDim_ = nKvHeads * headDim;
  alignedKvDim_ = (kvDim_ + 3) & ~3u;
  nRep_ = nHeads / nKvHeads;
  scale_ = 1.0f / std::sqrt(static_cast<float>(headDim));
  inputs_ = {q, kCache, vCache, runtimeParams};
  output_ = preallocOutput ? preallocOutput : store.createTensorEmpty({nHeads * headDim}, DataType::Float32);
}

std::optional<std::vector<uint32_t>> AttentionOpNode::shader() const {
  if (dtype_ != DataType::Float32 && dtype_ != DataType::Float16) return std::nullopt;
  if (headDim_ > 128 || nRep_ > 8) return std::nullopt;  // the kernels' limits (the reference's shared query holds 128 floats)
  KernelDesc d;
  d.op = Attention;
  d.dtypeA = d.dtypeB = (uint32_t)dtype_;
  return d.encode();
}

std::vector<uint8_t> AttentionOpNode::pushConstants() const {
  struct {
    uint32_t nHeads, nKvHeads, headDim, kvDim, alignedKvDim, nRep;
    float scale;
  } pc{nHeads_, nKvHeads_, headDim_, kvDim_, alignedKvDim_, nRep_, scale_};
  return toBytes(pc);
}

FusedRoPEKVWriteOpNode::FusedRoPEKVWriteOpNode(TensorStore &store, const Tensor &q, const Tensor &k, const Tensor &v,
                                               const Tensor &runtimeParams, const Tensor &cosTable, const Tensor &sinTable,
                                               const Tensor &kCache, const Tensor &vCache, uint32_t headDim,
                                               std::optional<uint32_t> spec)
    : OpNode(CacheWrite, store, spec), headDim_(headDim) {
  const auto &sq = store.getTensor(q).getShape();
  const auto &sk = store.getTensor(k).getShape();
  if (sq.empty() || sk.empty() || store.getTensor(v).getShape() != sk)
    throw std::runtime_error("fusedRoPEKVWrite: q, k and v must be vectors, k and v of one length");
  qDim_ = sq[0];
  kvDim_ = sk[0];
  if (headDim == 0 || headDim % 2 != 0 || qDim_ % headDim != 0 || kvDim_ % headDim != 0)
    throw std::runtime_error("fusedRoPEKVWrite: headDim must be even and divide the q and k lengths");
  cacheDtype_ = store.getTensor(kCache).getDtype();
  if (store.getTensor(vCache).getDtype() != cacheDtype_) throw std::runtime_error("fusedRoPEKVWrite: K and V caches must share a dtype");
  halfDim_ = headDim / 2;
  alignedKvDim_ = (kvDim_ + 3) & ~3u;
  inputs_ = {q, k, v, runtimeParams, cosTable, sinTable, kCache, vCache};
  output_ = store.createTensorEmpty({qDim_}, DataType::Float32);
}

std::optional<std::vector<uint32_t>> FusedRoPEKVWriteOpNode::shader() const {
  if (cacheDtype_ != DataType::Float32 && cacheDtype_ != DataType::Float16) return std::nullopt;
  KernelDesc d;
  d.op = CacheWrite;
  d.variant = kVariant;
  d.dtypeA = d.dtypeB = (uint32_t)cacheDtype_;
  return d.encode();
}

std::vector<uint8_t> FusedRoPEKVWriteOpNode::pushConstants() const {
  struct {
    uint32_t qDim, kvDim, headDim, halfDim, alignedKvDim;
  } pc{qDim_, kvDim_, headDim_, halfDim_, alignedKvDim_};
  return toBytes(pc);
}

BatchedKVCacheWriteOpNode::BatchedKVCacheWriteOpNode(TensorStore &store, const Tensor &k, const Tensor &v, const Tensor &kCache,
                                                     const Tensor &vCache, const Tensor &positions, const Tensor &cosTable,
                                                     const Tensor &sinTable, uint32_t batchSize, uint32_t nKvHeads, uint32_t headDim,
                                                     uint32_t kStride, uint32_t vStride, uint32_t kOffset, uint32_t vOffset,
                                                     std::optional<uint32_t> spec)
    : OpNode(CacheWrite, store, spec), batchSize_(batchSize), headDim_(headDim), kStride_(kStride), vStride_(vStride),
      kOffset_(kOffset), vOffset_(vOffset) {
  if (headDim == 0 || headDim % 2 != 0 || nKvHeads == 0) throw std::runtime_error("batchedKVCacheWrite: headDim must be even, nKvHeads positive");
  kvDim_ = nKvHeads * headDim;
  if (kStride < kOffset + kvDim_ || vStride < vOffset + kvDim_)
    throw std::runtime_error("batchedKVCacheWrite: a row stride is shorter than offset + kvDim");
  alignedKvDim_ = (kvDim_ + 3) & ~3u;
  cacheDtype_ = store.getTensor(kCache).getDtype();
  if (store.getTensor(vCache).getDtype() != cacheDtype_) throw std::runtime_error("batchedKVCacheWrite: K and V caches must share a dtype");
  inputs_ = {k, v, kCache, vCache, positions, cosTable, sinTable};
  output_ = kCache;
}

std::optional<std::vector<uint32_t>> BatchedKVCacheWriteOpNode::shader() const {
  if (cacheDtype_ != DataType::Float32 && cacheDtype_ != DataType::Float16) return std::nullopt;
  KernelDesc d;
  d.op = CacheWrite;
  d.variant = kVariant;
  d.dtypeA = d.dtypeB = (uint32_t)cacheDtype_;
  return d.encode();
}

std::vector<uint8_t> BatchedKVCacheWriteOpNode::pushConstants() const {
  struct {
    uint32_t batchSize, kvDim, alignedKvDim, headDim, halfDim, kStride, vStride, kOffset, vOffset;
  } pc{batchSize_, kvDim_, alignedKvDim_, headDim_, headDim_ / 2, kStride_, vStride_, kOffset_, vOffset_};
  return toBytes(pc);
}

BatchedAttentionReadCacheOpNode::BatchedAttentionReadCacheOpNode(TensorStore &store, const Tensor &q, const Tensor &kCache,
                                                                 const Tensor &vCache, const Tensor &positions, const Tensor &cosTable,
                                                                 const Tensor &sinTable, uint32_t batchSize, uint32_t nHeads,
                                                                 uint32_t nKvHeads, uint32_t headDim, uint32_t qStride, uint32_t qOffset,
                                                                 const Tensor &preallocOutput, std::optional<uint32_t> spec)
    : OpNode(Attention, store, spec), batchSize_(batchSize), nHeads_(nHeads), nKvHeads_(nKvHeads), headDim_(headDim), qStride_(qStride),
      qOffset_(qOffset) {
  if (nHeads == 0 || nKvHeads == 0 || headDim == 0 || headDim % 2 != 0 || nHeads % nKvHeads != 0)
    throw std::runtime_error("batchedAttentionReadCache: nHeads must be a positive multiple of nKvHeads and headDim even");
  if (qStride < qOffset + nHeads * headDim) throw std::runtime_error("batchedAttentionReadCache: qStride is shorter than qOffset + nHeads * headDim");
  dtype_ = store.getTensor(kCache).getDtype();
  alignedKvDim_ = (nKvHeads * headDim + 3) & ~3u;
  nRep_ = nHeads / nKvHeads;
  scale_ = 1.0f / std::sqrt(static_cast<float>(headDim));
  inputs_ = {q, kCache, vCache, positions, cosTable, sinTable};
  output_ = preallocOutput ? preallocOutput : store.createTensorEmpty({batchSize, nHeads * headDim}, DataType::Float32);
}

std::optional<std::vector<uint32_t>> BatchedAttentionReadCacheOpNode::shader() const {
  if (dtype_ != DataType::Float32 && dtype_ != DataType::Float16) return std::nullopt;
  if (headDim_ > 128 || nRep_ > 8) return std::nullopt;
  KernelDesc d;
  d.op = Attention;
  d.variant = kVariant;
  d.dtypeA = d.dtypeB = (uint32_t)dtype_;
  return d.encode();
}

std::vector<uint8_t> BatchedAttentionReadCacheOpNode::pushConstants() const {
  struct {
    uint32_t batchSize, nHeads, nKvHeads, headDim, alignedKvDim, nRep;
    float scale;
    uint32_t halfDim, qStride, qOffset;
  } pc{batchSize_, nHeads_, nKvHeads_, headDim_, alignedKvDim_, nRep_, scale_, headDim_ / 2, qStride_, qOffset_};
  return toBytes(pc);
}

// ---------------------------------------------------------------------------
// VariantSelector (runtime/VariantSelector.cpp:242-428) with a small JSON reader
// ---------------------------------------------------------------------------
namespace {
struct Json {
  enum Type { Null, Bool, Number, String, Array, Object } type = Null;
  double num = 0;
  bool b = false;
  std::string str;
  std::vector<Json> arr;
  std::map<std::string, Json> obj;
  const Json *get(const std::string &k) const {
    auto it = obj.find(k);
    return (type == Object && it != obj.end()) ? &it->second : nullptr;
  }
};

class JsonReader {
public:
  explicit JsonReader(const std::string &s) : s_(s) {}
  Json parse() {
    Json v = value();
    ws();
    if (p_ != s_.size()) throw std::runtime_error("trailing characters in JSON");
    return v;
  }

private:
  const std::string &s_;
  size_t p_ = 0;
  void ws() {
    while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) ++p_;
  }
  char peek() {
    ws();
    if (p_ >= s_.size()) throw std::runtime_error("unexpected end of JSON");
    return s_[p_];
  }
  void expect(char c) {
    if (peek() != c) throw std::runtime_error(std::string("expected '") + c + "' in JSON");
    ++p_;
  }
  std::string string() {
    expect('"');
    std::string out;
    while (p_ < s_.size() && s_[p_] != '"') {
      if (s_[p_] == '\\' && p_ + 1 < s_.size()) ++p_;
      out += s_[p_++];
    }
    if (p_ >= s_.size()) throw std::runtime_error("unterminated JSON string");
    ++p_;
    return out;
  }
  Json value() {
    Json v;
    const char c = peek();
    if (c == '{') {
      v.type = Json::Object;
      ++p_;
      if (peek() == '}') { ++p_; return v; }
      for (;;) {
        std::string k = string();
        expect(':');
        v.obj[k] = value();
        if (peek() == ',') { ++p_; continue; }
        expect('}');
        return v;
      }
    }
    if (c == '[') {
      v.type = Json::Array;
      ++p_;
      if (peek() == ']') { ++p_; return v; }
      for (;;) {
        v.arr.push_back(value());
        if (peek() == ',') { ++p_; continue; }
        expect(']');
        return v;
      }
    }
    if (c == '"') {
      v.type = Json::String;
      v.str = string();
      return v;
    }
    if (s_.compare(p_, 4, "true") == 0) { p_ += 4; v.type = Json::Bool; v.b = true; return v; }
    if (s_.compare(p_, 5, "false") == 0) { p_ += 5; v.type = Json::Bool; return v; }
    if (s_.compare(p_, 4, "null") == 0) { p_ += 4; return v; }
    size_t used = 0;
    v.num = std::stod(s_.substr(p_), &used);
    if (used == 0) throw std::runtime_error("bad JSON value");
    p_ += used;
    v.type = Json::Number;
    return v;
  }
};
}  // namespace

VariantSelector &VariantSelector::instance() {
  static VariantSelector inst;
  return inst;
}

void VariantSelector::clear() {
  operators_.clear();
  loaded_ = false;
}

bool VariantSelector::loadTuningData() {
  if (const char *env = std::getenv("CUT_TUNING_DATA"))
    if (loadFromFile(env)) return true;
  if (loadFromFile("tuning_data.json")) return true;
  if (const char *home = std::getenv("HOME"))
    if (loadFromFile(std::string(home) + "/.cut/tuning_data.json")) return true;
  return false;
}

bool VariantSelector::loadFromFile(const std::string &path) {
  std::ifstream f(path);
  if (!f) return false;
  std::string content((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  return loadFromString(content);
}

bool VariantSelector::loadFromString(const std::string &content) {
  try {
    JsonReader reader(content);
    Json root = reader.parse();
    const Json *ops = root.get("operators");
    if (!ops || ops->type != Json::Object) return false;
    auto parseRules = [](const Json &o) {
      OperatorRules r;
      if (const Json *dv = o.get("default_variant"); dv && dv->type == Json::Number) r.defaultVariant = (int)dv->num;
      if (const Json *rules = o.get("rules"); rules && rules->type == Json::Array)
        for (const Json &rv : rules->arr) {
          Rule rule;
          if (const Json *v = rv.get("variant"); v && v->type == Json::Number) rule.variant = (int)v->num;
          if (const Json *c = rv.get("conditions"); c && c->type == Json::Object) {
            if (const Json *mn = c->get("total_elements_min"); mn && mn->type == Json::Number)
              rule.totalElementsMin = (int64_t)mn->num;
            if (const Json *mx = c->get("total_elements_max"); mx && mx->type == Json::Number)
              rule.totalElementsMax = (int64_t)mx->num;
            if (const Json *sh = c->get("shape"); sh && sh->type == Json::Array)
              for (const Json &d : sh->arr)
                if (d.type == Json::Number) rule.shape.push_back((int64_t)d.num);
          }
          r.rules.push_back(rule);
        }
      return r;
    };
    operators_.clear();
    for (const auto &[name, val] : ops->obj) {
      if (const Json *backends = val.get("backends"); backends && backends->type == Json::Object)
        for (const auto &[bname, bval] : backends->obj) operators_[name + "@" + bname] = parseRules(bval);
      if (val.get("default_variant") || val.get("rules")) operators_[name] = parseRules(val);
    }
    loaded_ = true;
    return true;
  } catch (const std::exception &e) {
    std::cerr << "VariantSelector: cannot parse tuning data: " << e.what() << std::endl;
    return false;
  }
}

int VariantSelector::select(const std::string &op, const std::vector<uint32_t> &shape, int defaultVariant,
                            const std::string &backend) const {
  if (!loaded_) return defaultVariant;
  auto eval = [&shape, defaultVariant](const OperatorRules &r) {
    int64_t total = 1;
    for (uint32_t d : shape) total *= d;
    for (const Rule &rule : r.rules) {
      bool shapeOk = rule.shape.empty();
      if (!shapeOk && shape.size() == rule.shape.size()) {
        shapeOk = true;
        for (size_t i = 0; i < shape.size(); ++i)
          if ((int64_t)shape[i] != rule.shape[i]) shapeOk = false;
      }
      const bool minOk = rule.totalElementsMin < 0 || total >= rule.totalElementsMin;
      const bool maxOk = rule.totalElementsMax < 0 || total < rule.totalElementsMax;
      if (shapeOk && minOk && maxOk) return rule.variant;  // first match wins
    }
    // (a negative default_variant in the file leaves the caller's own choice in place: for the quantized matmuls
    // that choice depends on the shape, so one fixed fallback index would be wrong for most of them)
    return r.defaultVariant < 0 ? defaultVariant : r.defaultVariant;
  };
  if (!backend.empty())
    if (auto it = operators_.find(op + "@" + backend); it != operators_.end()) return eval(it->second);
  if (auto it = operators_.find(op); it != operators_.end()) return eval(it->second);
  return defaultVariant;
}

// ---------------------------------------------------------------------------
// Dispatcher (runtime/Dispatcher.cpp:18-75)
// ---------------------------------------------------------------------------
Dispatcher::Dispatcher(TensorStore *store) : store_(store), iface_(store->iface()) {}

bool Dispatcher::encode(OpNode &node) {
  if (!iface_) throw std::runtime_error("Dispatcher::encode: ComputeInterface is null");
  Tensor shader = getOrCreateShader(node);
  ComputeDispatch dispatch(shader, node.dispatchSize(), node.bindings());
  dispatch.label = node.displayName();
  dispatch.outputHandle = node.output();
  iface_->encode(std::move(dispatch));
  return true;
}

void Dispatcher::encodeBarrier() { iface_->encode(ComputeDispatch::createBarrier()); }

Tensor Dispatcher::getOrCreateShader(const OpNode &node) {
  const size_t key = node.shaderKey();
  if (auto it = shaderCache_.find(key); it != shaderCache_.end()) return it->second;
  auto words = node.shader();
  if (!words.has_value()) throw std::runtime_error("Dispatcher: node returned no shader");
  Tensor handle = iface_->createShaderModule(*words);
  shaderCache_[key] = handle;
  return handle;
}

// ---------------------------------------------------------------------------
// Operations / Runtime
// ---------------------------------------------------------------------------
Tensor Operations::dispatch(std::unique_ptr<OpNode> node) {
  Tensor out = node->output();
  dispatcher_->encode(*node);
  return out;
}

Tensor Operations::matmul(const Tensor &a, const Tensor &packedB, const Tensor &scales, std::optional<uint32_t> spec) {
  return dispatch(std::make_unique<MatMulOpNode>(*store_, a, packedB, scales, spec));
}

Tensor Operations::matmulUnary(OperatorEnum unaryOp, const Tensor &a, const Tensor &packedB, const Tensor &scales,
                               std::optional<uint32_t> spec) {
  auto node = std::make_unique<MatMulOpNode>(*store_, a, packedB, scales, spec);
  node->setFusion(MatMulFusion::Unary, unaryOp);
  return dispatch(std::move(node));
}

Tensor Operations::matmulBinary(OperatorEnum binaryOp, const Tensor &a, const Tensor &packedB, const Tensor &scales,
                                const Tensor &d, std::optional<uint32_t> spec) {
  auto node = std::make_unique<MatMulOpNode>(*store_, a, packedB, scales, spec);
  node->setFusion(MatMulFusion::Binary, binaryOp, d);
  return dispatch(std::move(node));
}

Tensor Operations::matmulBlocks(const Tensor &a, const Tensor &raw, DequantFormat f, uint32_t N,
                                std::optional<uint32_t> spec) {
  return dispatch(std::make_unique<MatMulOpNode>(*store_, a, raw, f, N, spec));
}

Tensor Operations::matmulBlocksUnary(OperatorEnum unaryOp, const Tensor &a, const Tensor &raw, DequantFormat f, uint32_t N,
                                     std::optional<uint32_t> spec) {
  auto node = std::make_unique<MatMulOpNode>(*store_, a, raw, f, N, spec);
  node->setFusion(MatMulFusion::Unary, unaryOp);
  return dispatch(std::move(node));
}

Tensor Operations::matmulBlocksBinary(OperatorEnum binaryOp, const Tensor &a, const Tensor &raw, DequantFormat f,
                                      uint32_t N, const Tensor &d, std::optional<uint32_t> spec) {
  auto node = std::make_unique<MatMulOpNode>(*store_, a, raw, f, N, spec);
  node->setFusion(MatMulFusion::Binary, binaryOp, d);
  return dispatch(std::move(node));
}

Tensor Operations::matmulBlocksFused(const Tensor &a, const Tensor &raw, DequantFormat f, uint32_t N, const MatMulBlockOptions &opt,
                                     MatMulFusion fusion, OperatorEnum fusionOp, const Tensor &d) {
  auto node = std::make_unique<MatMulOpNode>(*store_, a, raw, f, N, std::nullopt);
  if (fusion != MatMulFusion::None) node->setFusion(fusion, fusionOp, d);
  node->setBlockOptions(opt);
  return dispatch(std::move(node));
}

Tensor Operations::gluPairs(const Tensor &in, OperatorEnum unaryOp) {
  return dispatch(std::make_unique<GluPairsOpNode>(*store_, in, unaryOp));
}

Tensor Operations::transposeQ4(const Tensor &packedInput, uint32_t N, uint32_t K) {
  return dispatch(std::make_unique<TransposeQ4NibbleOpNode>(*store_, packedInput, N, K));
}

Tensor Operations::dequantize(const Tensor &rawData, uint32_t format, uint32_t rows, uint32_t cols) {
  return dispatch(std::make_unique<DequantOpNode>(*store_, rawData, static_cast<DequantFormat>(format), rows, cols));
}

Tensor Operations::requantQ8Blocks(const Tensor &rawData, DequantFormat format, uint32_t rows, uint32_t cols) {
  return dispatch(std::make_unique<RequantQ8BlocksOpNode>(*store_, rawData, format, rows, cols));
}

Tensor Operations::rmsNorm(const Tensor &x, const Tensor &weight, float eps, std::optional<uint32_t> spec) {
  return dispatch(std::make_unique<RMSNormOpNode>(*store_, x, weight, eps, spec));
}

Tensor Operations::embedding(const Tensor &indices, const Tensor &weight, const Tensor &preallocOutput,
                             std::optional<uint32_t> spec) {
  return dispatch(std::make_unique<EmbeddingOpNode>(*store_, indices, weight, preallocOutput, spec));
}

Tensor Operations::embeddingCol(const Tensor &indices, const Tensor &matrix, const Tensor &scales, const Tensor &preallocOutput,
                                std::optional<uint32_t> spec) {
  return dispatch(std::make_unique<EmbeddingColOpNode>(*store_, indices, matrix, scales, preallocOutput, spec));
}

Tensor Operations::reduce(OperatorEnum op, const Tensor &a, std::optional<uint32_t> spec) {
  return dispatch(std::make_unique<GlobalReduceOpNode>(op, *store_, a, spec));
}

Tensor Operations::attention(const Tensor &q, const Tensor &kCache, const Tensor &vCache, const Tensor &runtimeParams,
                             uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, const Tensor &preallocOutput) {
  return dispatch(std::make_unique<AttentionOpNode>(*store_, q, kCache, vCache, runtimeParams, nHeads, nKvHeads, headDim, preallocOutput));
}

void Operations::batchedKVCacheWrite(const Tensor &k, const Tensor &v, const Tensor &kCache, const Tensor &vCache,
                                     const Tensor &positions, const Tensor &cosTable, const Tensor &sinTable, uint32_t batchSize,
                                     uint32_t nKvHeads, uint32_t headDim, uint32_t kStride, uint32_t vStride, uint32_t kOffset,
                                     uint32_t vOffset) {
  dispatch(std::make_unique<BatchedKVCacheWriteOpNode>(*store_, k, v, kCache, vCache, positions, cosTable, sinTable, batchSize, nKvHeads,
                                                       headDim, kStride, vStride, kOffset, vOffset));
}

Tensor Operations::batchedAttentionReadCache(const Tensor &q, const Tensor &kCache, const Tensor &vCache, const Tensor &positions,
                                             const Tensor &cosTable, const Tensor &sinTable, uint32_t batchSize, uint32_t nHeads,
                                             uint32_t nKvHeads, uint32_t headDim, uint32_t qStride, uint32_t qOffset,
                                             const Tensor &preallocOutput) {
  return dispatch(std::make_unique<BatchedAttentionReadCacheOpNode>(*store_, q, kCache, vCache, positions, cosTable, sinTable, batchSize,
                                                                   nHeads, nKvHeads, headDim, qStride, qOffset, preallocOutput));
}

Tensor Operations::fusedRoPEKVWrite(const Tensor &q, const Tensor &k, const Tensor &v, const Tensor &runtimeParams,
                                    const Tensor &cosTable, const Tensor &sinTable, const Tensor &kCache, const Tensor &vCache,
                                    uint32_t headDim) {
  return dispatch(std::make_unique<FusedRoPEKVWriteOpNode>(*store_, q, k, v, runtimeParams, cosTable, sinTable, kCache, vCache, headDim));
}

Runtime::Runtime(std::unique_ptr<ComputeInterface> iface)
    : iface_(std::move(iface)), store_(iface_.get()), dispatcher_(&store_), ops_(&store_, &dispatcher_) {}

Runtime::Runtime(int device) : Runtime(createB200Compute(device)) {}

void Runtime::flush() {
  if (iface_->pendingDispatches() == 0) return;
  ComputeHandle cb = iface_->submit();
  iface_->wait(cb);
}

void Runtime::copyFromTensor(const Tensor &t, void *dst, size_t bytes) {
  flush();
  iface_->copyDataFromBuffer(t, dst, bytes, 0, 0, false, true);
}

void Runtime::copyToTensor(const Tensor &t, const void *src, size_t bytes) {
  flush();
  iface_->copyDataToBuffer(src, t, bytes, 0, 0, false, true);
}

}  // namespace cut
