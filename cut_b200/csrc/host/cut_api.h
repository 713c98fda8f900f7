// Host side of the B200 backend: the slice of CUT's operator API that the GGUF
// quantized-matmul path crosses, with the reference's names, argument meaning
// and error behaviour, sitting on top of the C ABI in include/cutb.h.
//
//   Operations::matmul / matmulUnary / matmulBinary / transposeQ4 / dequantize
//       (runtime/Operations.h:65-93, 459, 467)
//   MatMulOpNode, DequantOpNode, TransposeQ4NibbleOpNode and the OpNode base
//       (operators/impl/matmul/MatMulOp.h, operators/impl/dequant/DequantOp.h,
//        operators/impl/q4transpose/TransposeQ4NibbleOp.h, operators/runtime/OpNode.h:64-166)
//   Dispatcher (runtime/Dispatcher.h:25-63), VariantSelector (runtime/VariantSelector.h)
//   ComputeInterface / ComputeBuffer / ComputeDispatch / ComputeBinding
//       (core/api/include/ComputeInterface.h:17-312, ComputeStructs.h:154-432)
//   B200Compute: the backend that stands where core/backends/cuda/CudaCompute stands.
//
// Differences from the reference, all deliberate:
//   * OpNode::shader() returns a small kernel descriptor (magic word, op,
//     variant, dtypes, specialisation constants) instead of SPIR-V; the backend
//     decodes it in createShaderModule() and binds it to a precompiled sm_100a
//     kernel behind the C ABI.  A descriptor no kernel covers is an error (the
//     reference skips such dispatches silently).
//   * Quantized matmul accepts Float16 activations directly (no cast dispatch).
//   * A fourth quant format, raw GGUF blocks (QuantFormat::Blocks), enters
//     through Operations::matmulBlocks(); the plane layouts the reference's
//     loader produces keep working through the three-input overloads.
//   * The variant choice goes through VariantSelector ("MatMulQ4" / "MatMulQ8" /
//     "MatMulQBlocks", backend "cuda") with the built-in choice as the default.
// Everything is single-threaded by contract, as in the reference.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace cut {

// ---- core/api: common types ---------------------------------------------------
enum class DataType { Float32, Float16, UInt32, Int32, Int8 };
size_t dataTypeSize(DataType t);
DataType widenPrecision(DataType t);

enum class ComputeBackend { Vulkan, CUDA };
inline const char *backendName(ComputeBackend b) { return b == ComputeBackend::CUDA ? "cuda" : "vulkan"; }

struct DeviceCaps {
  bool cooperativeMatrix = false;
  bool integerDotProduct = false;
  uint32_t subgroupSize = 32;
  ComputeBackend backend = ComputeBackend::Vulkan;
};

struct ThreadSize {
  uint32_t x = 0, y = 0, z = 0;
};

// Operator codes of the path (operators/runtime/ComputeOpsShared.h).
enum OperatorEnum : uint32_t {
  BinaryAdd = 0, BinarySub = 1, BinaryMul = 2, BinaryDiv = 3, BinaryMod = 4, BinaryPow = 5, BinaryFloorDiv = 6,
  BinaryMin = 13, BinaryMax = 14,
  MatMul = 64,
  UnaryNeg = 100, UnaryAbs = 101, UnarySqrt = 102, UnarySquare = 103, UnaryReciprocal = 104, UnaryExp = 106,
  UnaryLog = 109, UnaryTanh = 121, UnaryFloor = 122, UnaryCeil = 123, UnaryRound = 124, UnaryRelu = 130,
  UnarySigmoid = 131, UnaryGelu = 132, UnarySilu = 133, UnarySoftplus = 134, UnaryRelu6 = 137, UnaryMish = 141,
  UnaryHardswish = 142, UnaryHardsigmoid = 143, UnaryRsqrt = 148,
  ReduceSum = 208, ReduceMean = 209, ReduceMin = 210, ReduceMax = 211, ReduceArgmax = 214, ReduceArgmin = 215,
  RMSNorm = 312, Embedding = 320, EmbeddingCol = 321,
  CacheWrite = 360, Attention = 361,
  MatMulQ8 = 371, MatMulQ4 = 374,
  MatMulQBlocks = 375,  // new: weights as raw GGUF blocks
  Dequantize = 390,
  RequantQ8Blocks = 391,  // new: any block format -> Q8_0 GGUF blocks on the device
  GluPairs = 392,         // new: out[r, i] = unary(in[r, 2i]) * in[r, 2i + 1] (gate / up stored as row pairs)
  TransposeQ4 = 401,
};

// ---- handles and buffers -------------------------------------------------------
class ComputeInterface;

/// Reference-counted handle to a backend object (buffer, kernel, command buffer);
/// the last copy releases the object (core/api/include/ComputeHandle.h).
class ComputeHandle final {
public:
  ComputeHandle() = default;
  explicit operator bool() const { return static_cast<bool>(slot_); }
  bool operator==(const ComputeHandle &o) const { return slot_ == o.slot_; }
  bool operator!=(const ComputeHandle &o) const { return slot_ != o.slot_; }
  void reset() { slot_.reset(); }
  size_t id() const;

  struct Slot {
    size_t id = 0;
    virtual ~Slot() = default;
  };
  explicit ComputeHandle(std::shared_ptr<Slot> s) : slot_(std::move(s)) {}
  template <typename T> T *as() const { return dynamic_cast<T *>(slot_.get()); }

private:
  std::shared_ptr<Slot> slot_;
};
using Tensor = ComputeHandle;

/// Buffer description: the innermost dimension is padded to 4 elements and the
/// byte size to 16 (core/api/src/ComputeStructs.cpp:99-120).
struct ComputeBuffer : ComputeHandle::Slot {
  void *data = nullptr;  ///< device pointer
  const std::vector<uint32_t> &getShape() const { return shape_; }
  DataType getDtype() const { return dtype_; }
  size_t size() const { return size_; }
  uint32_t innerDimSize() const { return shape_.empty() ? 0 : shape_.back(); }
  uint32_t innerDimPadded() const { return (innerDimSize() + 3u) & ~3u; }
  size_t calculateActualSize() const { return calculateActualSize(shape_, dtype_); }
  static size_t calculateActualSize(const std::vector<uint32_t> &shape, DataType dtype);
  static size_t calculateAlignedSize(const std::vector<uint32_t> &shape, DataType dtype);
  static size_t calculateAlignedElements(const std::vector<uint32_t> &shape);
  void describe(const std::vector<uint32_t> &shape, DataType dtype);

private:
  std::vector<uint32_t> shape_;
  DataType dtype_ = DataType::Float32;
  size_t size_ = 0;
};

/// One shader argument: a buffer handle or an owned byte blob (push constants).
struct ComputeBinding {
  uint32_t index = 0;
  ComputeHandle handle;
  std::vector<uint8_t> bytes;
  ComputeBinding(uint32_t i, const ComputeHandle &h) : index(i), handle(h) {}
  ComputeBinding(uint32_t i, const void *p, uint32_t n) : index(i), bytes((const uint8_t *)p, (const uint8_t *)p + n) {}
  bool isHandle() const { return static_cast<bool>(handle); }
};

/// One recorded kernel launch (core/api/include/ComputeStructs.h:304-432).
struct ComputeDispatch {
  ComputeHandle shader;
  ThreadSize size;
  std::vector<ComputeBinding> bindings;
  std::string label;
  ComputeHandle outputHandle;
  bool isBarrier = false;
  ComputeDispatch() = default;
  ComputeDispatch(const ComputeHandle &s, const ThreadSize &ts, std::vector<ComputeBinding> b)
      : shader(s), size(ts), bindings(std::move(b)) {}
  static ComputeDispatch createBarrier() {
    ComputeDispatch d;
    d.isBarrier = true;
    return d;
  }
};

/// Kernel descriptor carried where the reference carries SPIR-V words.
struct KernelDesc {
  static constexpr uint32_t kMagic = 0x42545543u;  // "CUTB"
  uint32_t op = 0;        ///< OperatorEnum
  uint32_t variant = 0;   ///< index into the op's variant table
  uint32_t dtypeA = 0;    ///< DataType of the activation
  uint32_t dtypeB = 0;    ///< DataType of the scales plane
  uint32_t fusionType = 0, fusionOp = 0;  ///< specialisation constants 1 and 2
  uint32_t affine = 0;    ///< specialisation constant 3
  uint32_t format = 0;    ///< block format (Blocks / Dequantize)
  uint32_t flags = 0;     ///< MatMulQBlocks: kBlockFlag* bits (a tenth word, present only when non-zero)
  std::vector<uint32_t> encode() const;
  static std::optional<KernelDesc> decode(const std::vector<uint32_t> &words);
};

// ---- ComputeInterface ------------------------------------------------------------
class ComputeInterface {
public:
  ComputeInterface() = default;
  virtual ~ComputeInterface() = default;
  ComputeInterface(const ComputeInterface &) = delete;
  ComputeInterface(ComputeInterface &&) = delete;

  virtual ComputeHandle createBuffer(const std::vector<uint32_t> &shape, DataType dtype,
                                     const void *hostSourcePtr = nullptr, bool immutable = false) = 0;
  virtual ComputeHandle createBufferMapped(const std::vector<uint32_t> &shape, DataType dtype,
                                           const void *hostSourcePtr = nullptr, bool preferHost = false) {
    (void)preferHost;
    return createBuffer(shape, dtype, hostSourcePtr, false);
  }
  virtual ComputeHandle createBufferView(const ComputeHandle &parent, size_t byteOffset,
                                         const std::vector<uint32_t> &shape, DataType dtype) = 0;
  virtual void copyDataToBuffer(const void *hostSourcePtr, const ComputeHandle &dest, size_t copySize,
                                size_t srcOffset, size_t destOffset, bool useStagingBuffer = false,
                                bool waitForCompletion = false) = 0;
  virtual void copyDataFromBuffer(const ComputeHandle &src, void *hostDestPtr, size_t copySize, size_t srcOffset,
                                  size_t destOffset, bool useStagingBuffer = false,
                                  bool waitForCompletion = false) = 0;
  virtual ComputeHandle createShaderModule(const std::vector<uint32_t> &words) = 0;
  virtual const ComputeBuffer &getBuffer(const ComputeHandle &h) const = 0;
  virtual size_t bufferCount() const = 0;
  virtual size_t activeBufferMemoryBytes() const { return 0; }
  virtual size_t bufferOffsetAlignment() const { return 256; }
  virtual uint32_t maxSharedMemoryPerBlock() const { return 49152; }
  virtual size_t deviceTotalMemoryBytes() const { return 0; }
  virtual void releaseLoadingResources() {}
  virtual void flushTransfers() {}
  const DeviceCaps &caps() const { return caps_; }

  // Command recording (ComputeInterface.cpp:15-82): encode() appends to the
  // active command buffer, submit() runs it, submitReusable() keeps it for
  // resubmit() (a CUDA graph on this backend).
  void encode(ComputeDispatch &&dispatch);
  ComputeHandle submit();
  ComputeHandle submitReusable();
  void resubmit(const ComputeHandle &commandBuffer);
  void wait(const ComputeHandle &commandBuffer);
  size_t pendingDispatches() const { return pending_.size(); }

protected:
  // Backend hooks behind the non-virtual recording calls above.
  virtual ComputeHandle executeDispatches(std::vector<ComputeDispatch> &&dispatches, bool reusable) = 0;
  virtual void replay(const ComputeHandle &commandBuffer) = 0;
  virtual void waitFor(const ComputeHandle &commandBuffer) = 0;
  static void copyActualToAligned(const void *src, void *dst, const ComputeBuffer &buffer);
  static void copyAlignedToActual(const void *src, void *dst, const ComputeBuffer &buffer);
  DeviceCaps caps_;

private:
  std::vector<ComputeDispatch> pending_;
};

/// Creates the sm_100a backend on `device` (throws std::runtime_error without a CUDA device).
std::unique_ptr<ComputeInterface> createB200Compute(int device = 0);

// ---- TensorStore -----------------------------------------------------------------
class TensorStore {
public:
  explicit TensorStore(ComputeInterface *iface) : iface_(iface) {}
  ComputeInterface *iface() const { return iface_; }
  const ComputeBuffer &getTensor(const Tensor &h) const { return iface_->getBuffer(h); }
  Tensor createTensor(const std::vector<uint32_t> &shape, DataType dtype, const void *src = nullptr) {
    return iface_->createBuffer(shape, dtype, src, false);
  }
  Tensor createTensorEmpty(const std::vector<uint32_t> &shape, DataType dtype) {
    return iface_->createBuffer(shape, dtype, nullptr, false);
  }
  const DeviceCaps &caps() const { return iface_->caps(); }

private:
  ComputeInterface *iface_;
};

// ---- variant tables (same names and indices as the reference's generated tables) ---
struct MatMulQVariantInfo {
  const char *name;
  uint32_t wgX, wgY, effTileM, effTileN;
  const char *description;
};
inline constexpr int kMatMulQ4VariantCount = 5;
inline constexpr int kMatMulQ4DefaultVariant = 0;
extern const MatMulQVariantInfo kMatMulQ4Variants[kMatMulQ4VariantCount];
inline constexpr int kMatMulQ8VariantCount = 8;
inline constexpr int kMatMulQ8DefaultVariant = 2;
extern const MatMulQVariantInfo kMatMulQ8Variants[kMatMulQ8VariantCount];
/// Variants over raw GGUF blocks: the cutb_qmatmul variants (include/cutb.h).
inline constexpr int kMatMulQBlocksVariantCount = 3;
extern const MatMulQVariantInfo kMatMulQBlocksVariants[kMatMulQBlocksVariantCount];
const char *getMatMulQ4VariantName(int i);
const char *getMatMulQ8VariantName(int i);
/// Kernel descriptor for a variant and dtype triple, nullopt if no kernel is compiled for it
/// (MatMulQ4Variants.generated.h:50, MatMulQ8Variants.generated.h:59).
std::optional<std::vector<uint32_t>> getCompiledMatMulQ4(int variant, DataType input1 = DataType::Float32,
                                                         DataType scales = DataType::Float32,
                                                         DataType output = DataType::Float32);
std::optional<std::vector<uint32_t>> getCompiledMatMulQ8(int variant, DataType input1 = DataType::Float32,
                                                         DataType scales = DataType::Float32,
                                                         DataType output = DataType::Float32);

// ---- OpNode and the three operators of the path --------------------------------------
template <typename T> inline std::vector<uint8_t> toBytes(const T &v) {
  std::vector<uint8_t> b(sizeof(T));
  std::memcpy(b.data(), &v, sizeof(T));
  return b;
}

class OpNode {
public:
  virtual ~OpNode() = default;
  OperatorEnum op() const { return op_; }
  const Tensor &output() const { return output_; }
  const std::vector<Tensor> &inputs() const { return inputs_; }
  virtual std::optional<std::vector<uint32_t>> shader() const = 0;
  virtual size_t shaderKey() const = 0;
  virtual std::vector<uint32_t> outputShape() const = 0;
  virtual DataType outputDtype() const = 0;
  virtual std::vector<DataType> resolveInputDtypes(const std::vector<DataType> &in) const { return in; }
  virtual ThreadSize dispatchSize() const = 0;
  virtual std::vector<ComputeBinding> bindings() const;
  virtual std::string displayName() const = 0;
  virtual std::vector<uint8_t> pushConstants() const = 0;
  std::optional<uint32_t> spec() const { return spec_; }

protected:
  OpNode(OperatorEnum op, TensorStore &store, std::optional<uint32_t> spec = {}) : op_(op), store_(&store), spec_(spec) {}
  OperatorEnum op_;
  TensorStore *store_;
  std::optional<uint32_t> spec_;
  std::vector<Tensor> inputs_{};
  Tensor output_{};
};

enum class QuantFormat { None, Q8, Q4, Blocks };
enum class MatMulFusion { None, Unary, Binary };
/// Formats of DequantOpNode; the reference's values (operators/impl/dequant/DequantOp.h:8-13)
/// plus the 32-weight block formats it only dequantises on the CPU (gguf_reader.cpp:541-660, 826-850).
enum class DequantFormat : uint32_t { BF16 = 0, Q4_K = 1, Q5_K = 2, Q6_K = 3, Q8_0 = 16, Q4_0 = 17, Q4_1 = 18, Q5_0 = 19 };

/// Extras of the block-layout decode mat-vec that a runner's per-token step uses (bit values = the C ABI's
/// CUTB_FLAG_*): kBlockFlagNoOverlap -- the launch does not prefetch under its predecessor; kBlockFlagAct16 -- fp32
/// activations staged at one 16-bit level per 32-k block; kBlockFlagRmsNorm -- the RMSNorm in front of the
/// projection applied while the activations are staged (needs normWeight); kBlockFlagGluPairs -- rows stored as
/// (gate_i, up_i) pairs, C[m, i] = unary(acc[2i]) * acc[2i + 1] (needs a unary fusion; output [M, N / 2]).
enum : uint32_t { kBlockFlagNoOverlap = 1, kBlockFlagAct16 = 2, kBlockFlagRmsNorm = 4, kBlockFlagGluPairs = 8 };
struct MatMulBlockOptions {
  uint32_t flags = 0;
  Tensor normWeight;       ///< Float32 [K], with kBlockFlagRmsNorm
  float normEps = 1e-5f;
};

class MatMulOpNode : public OpNode {
public:
  /// Quantized matmul over the reference's plane layout; detects Q8 / Q4 / affine Q4 from the
  /// shapes and throws std::runtime_error on bad shapes (operators/impl/matmul/MatMulOp.cpp:271-383).
  MatMulOpNode(TensorStore &store, const Tensor &a, const Tensor &packedB, const Tensor &scalesB,
               std::optional<uint32_t> spec = {});
  /// Quantized matmul over raw GGUF blocks: rawB is a 1-D Int8 tensor of N rows of blocks along K.
  MatMulOpNode(TensorStore &store, const Tensor &a, const Tensor &rawB, DequantFormat blockFormat, uint32_t N,
               std::optional<uint32_t> spec = {});
  QuantFormat format() const { return format_; }
  MatMulFusion fusion() const { return fusion_; }
  bool affine() const { return q4Affine_; }
  void setFusion(MatMulFusion fusion, OperatorEnum fusionOp = {}, const Tensor &d = {});
  /// Block layout only, after setFusion(); throws std::runtime_error on combinations no kernel has.
  void setBlockOptions(const MatMulBlockOptions &opt);
  uint32_t blockFlags() const { return blockFlags_; }
  DataType outputDtype() const override { return DataType::Float32; }
  size_t shaderKey() const override;
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override {
    return {M_, (blockFlags_ & kBlockFlagGluPairs) ? N_ / 2 : N_};
  }
  ThreadSize dispatchSize() const override;
  std::vector<uint8_t> pushConstants() const override;
  std::vector<ComputeBinding> bindings() const override;
  std::string displayName() const override;
  std::vector<DataType> resolveInputDtypes(const std::vector<DataType> &in) const override;
  uint32_t M() const { return M_; }
  uint32_t K() const { return K_; }
  uint32_t N() const { return N_; }
  DequantFormat blockFormat() const { return blockFormat_; }

private:
  QuantFormat format_ = QuantFormat::None;
  MatMulFusion fusion_ = MatMulFusion::None;
  OperatorEnum fusionOp_{};
  DataType dtypeA_ = DataType::Float32, dtypeB_ = DataType::Float16;
  uint32_t M_ = 0, K_ = 0, N_ = 0;
  bool autoSpec_ = false, q4Affine_ = false;
  uint32_t fusionFallbackSpec_ = 0;
  DequantFormat blockFormat_ = DequantFormat::Q4_K;
  uint32_t blockFlags_ = 0;
  float normEps_ = 0.f;
};

class DequantOpNode : public OpNode {
public:
  DequantOpNode(TensorStore &store, const Tensor &rawData, DequantFormat format, uint32_t rows, uint32_t cols,
                std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return DataType::Float32; }
  size_t shaderKey() const override;
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return {rows_, cols_}; }
  ThreadSize dispatchSize() const override { return {cols_, rows_, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "Dequantize"; }

private:
  DequantFormat format_;
  uint32_t rows_, cols_, outputStride_;
};

/// Raw blocks of any DequantFormat -> Q8_0 GGUF blocks [rows * cols / 32 * 34 bytes], what the runner does on the
/// CPU for the formats its matmul does not take (interface/runner/llama/llama.cpp:488-505, 750-767).
class RequantQ8BlocksOpNode : public OpNode {
public:
  RequantQ8BlocksOpNode(TensorStore &store, const Tensor &rawData, DequantFormat format, uint32_t rows, uint32_t cols,
                        std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return DataType::Int8; }
  size_t shaderKey() const override { return static_cast<size_t>(op_) | ((static_cast<size_t>(format_) & 0x1F) << 16); }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return {rows_ * (cols_ / 32) * 34}; }
  ThreadSize dispatchSize() const override { return {cols_ / 32, rows_, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "RequantQ8Blocks"; }

private:
  DequantFormat format_;
  uint32_t rows_, cols_;
};

/// The gated activation over a matmul whose weight rows are (gate_i, up_i) pairs: [rows, 2F] -> [rows, F],
/// out[r, i] = unary(in[r, 2i]) * in[r, 2i + 1] (SiLU for the llama feed-forward, interface/runner/llama/llama.cpp:2455-2470).
class GluPairsOpNode : public OpNode {
public:
  GluPairsOpNode(TensorStore &store, const Tensor &in, OperatorEnum unaryOp, std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return DataType::Float32; }
  size_t shaderKey() const override { return static_cast<size_t>(op_) | (static_cast<size_t>(unaryOp_) << 16); }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return {rows_, colsOut_}; }
  ThreadSize dispatchSize() const override { return {colsOut_, rows_, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "GluPairs"; }

private:
  OperatorEnum unaryOp_;
  uint32_t rows_ = 0, colsOut_ = 0, strideIn_ = 0, strideOut_ = 0;
};

class TransposeQ4NibbleOpNode : public OpNode {
public:
  TransposeQ4NibbleOpNode(TensorStore &store, const Tensor &packedInput, uint32_t N, uint32_t K,
                          std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return DataType::Int8; }
  size_t shaderKey() const override { return static_cast<size_t>(op_); }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return {K_, N_ / 2}; }
  ThreadSize dispatchSize() const override;
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "TransposeQ4"; }

private:
  uint32_t N_, K_, strideInHalf_, strideOutHalf_;
};

/// Row-wise RMS normalisation with a weight vector (operators/impl/rmsnorm/RMSNormOp.cpp:7-76):
/// x is [dim] or [batch, dim], weight [dim] of the same dtype; one 256-thread group per row.
class RMSNormOpNode : public OpNode {
public:
  RMSNormOpNode(TensorStore &store, const Tensor &x, const Tensor &weight, float eps = 1e-5f,
                std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return dtype_; }
  size_t shaderKey() const override { return static_cast<size_t>(op_) | (static_cast<size_t>(dtype_) << 16); }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override;
  ThreadSize dispatchSize() const override { return {256, batchSize_, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "RMSNorm"; }

private:
  DataType dtype_ = DataType::Float32;
  uint32_t batchSize_ = 1, dim_ = 0, alignedDim_ = 0;
  float eps_;
};

/// Row gather out[i, :] = weight[indices[i], :] (operators/impl/memory/MemoryOp.cpp:68-125).
class EmbeddingOpNode : public OpNode {
public:
  EmbeddingOpNode(TensorStore &store, const Tensor &indices, const Tensor &weight, const Tensor &preallocOutput = {},
                  std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return dtype_; }
  size_t shaderKey() const override { return static_cast<size_t>(op_) | (static_cast<size_t>(dtype_) << 16); }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return outShape_; }
  ThreadSize dispatchSize() const override;
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "Embedding"; }

private:
  DataType dtype_ = DataType::Float32;
  uint32_t embDim_ = 0, numIndices_ = 1;
  std::vector<uint32_t> outShape_;
};

/// Column gather out[i, d] = matrix[d, indices[i]] from a [dim, vocab] matrix in the matmul's orientation:
/// the embedding read out of a tied LM head, fp16 or int8 + fp16 scales (operators/impl/memory/MemoryOp.cpp:127-202).
class EmbeddingColOpNode : public OpNode {
public:
  EmbeddingColOpNode(TensorStore &store, const Tensor &indices, const Tensor &matrix, const Tensor &scales,
                     const Tensor &preallocOutput = {}, std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return DataType::Float32; }
  size_t shaderKey() const override { return static_cast<size_t>(op_) | (static_cast<size_t>(format_) << 16); }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return outShape_; }
  ThreadSize dispatchSize() const override;
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "EmbeddingCol"; }

private:
  uint32_t embDim_ = 0, numIndices_ = 1, vocabStride_ = 0, scaleStride_ = 0, outStride_ = 0, format_ = 0;
  std::vector<uint32_t> outShape_;
};

/// Whole-tensor reduction to one element (operators/impl/reduce/ReduceOp.cpp:29-91).  Only the two
/// index reductions the sampler uses have a kernel here; the others construct but have no shader.
class GlobalReduceOpNode : public OpNode {
public:
  GlobalReduceOpNode(OperatorEnum op, TensorStore &store, const Tensor &a, std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return dtype_; }
  size_t shaderKey() const override { return static_cast<size_t>(op_) | (static_cast<size_t>(dtype_) << 16); }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return {1}; }
  ThreadSize dispatchSize() const override { return {256, 1, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override;

private:
  DataType dtype_ = DataType::Float32;
  size_t numElements_ = 0;
  uint32_t actualInner_ = 0, alignedInner_ = 0;
};

/// Decode attention of one roped query over the populated KV cache with grouped-query heads
/// (operators/impl/attention/AttentionOp.cpp:57-122).  runtimeParams is the device buffer
/// {pos, seqLen}; the cache dtype (Float32 or Float16) selects the kernel, q and the output stay fp32.
class AttentionOpNode : public OpNode {
public:
  AttentionOpNode(TensorStore &store, const Tensor &q, const Tensor &kCache, const Tensor &vCache, const Tensor &runtimeParams,
                  uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, const Tensor &preallocOutput = {},
                  std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return DataType::Float32; }
  size_t shaderKey() const override { return static_cast<size_t>(op_) | ((static_cast<size_t>(dtype_) & 0xF) << 56); }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return {nHeads_ * headDim_}; }
  ThreadSize dispatchSize() const override { return {nHeads_ * 256, 1, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "Attention"; }

private:
  DataType dtype_ = DataType::Float32;
  uint32_t nHeads_, nKvHeads_, headDim_, kvDim_, alignedKvDim_, nRep_;
  float scale_;
};

/// Half-split RoPE of q and k at runtimeParams[0] fused with the write of the roped k and of v
/// into row pos of the caches; the output is the roped q
/// (operators/impl/attention/AttentionOp.cpp:553-612).
class FusedRoPEKVWriteOpNode : public OpNode {
public:
  static constexpr uint32_t kVariant = 1;  ///< KernelDesc::variant of this user of the CacheWrite op code
  FusedRoPEKVWriteOpNode(TensorStore &store, const Tensor &q, const Tensor &k, const Tensor &v, const Tensor &runtimeParams,
                         const Tensor &cosTable, const Tensor &sinTable, const Tensor &kCache, const Tensor &vCache,
                         uint32_t headDim, std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return DataType::Float32; }
  size_t shaderKey() const override {
    return static_cast<size_t>(op_) | (size_t{1} << 34) | ((static_cast<size_t>(cacheDtype_) & 0xF) << 56);
  }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return {qDim_}; }
  ThreadSize dispatchSize() const override { return {(qDim_ + 2 * kvDim_ + 255) / 256 * 256, 1, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "FusedRoPEKVWrite"; }

private:
  DataType cacheDtype_ = DataType::Float32;
  uint32_t qDim_, kvDim_, headDim_, halfDim_, alignedKvDim_;
};

/// Prefill: roped k and v of a batch of tokens into the cache rows positions[i]; k and v may be columns
/// (offset, row stride) of a wider matrix.  The node's output is the K cache itself
/// (operators/impl/attention/AttentionOp.cpp:295-372).
class BatchedKVCacheWriteOpNode : public OpNode {
public:
  static constexpr uint32_t kVariant = 2;
  BatchedKVCacheWriteOpNode(TensorStore &store, const Tensor &k, const Tensor &v, const Tensor &kCache, const Tensor &vCache,
                            const Tensor &positions, const Tensor &cosTable, const Tensor &sinTable, uint32_t batchSize,
                            uint32_t nKvHeads, uint32_t headDim, uint32_t kStride, uint32_t vStride, uint32_t kOffset,
                            uint32_t vOffset, std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return cacheDtype_; }
  size_t shaderKey() const override {
    return static_cast<size_t>(op_) | (size_t{1} << 33) | ((static_cast<size_t>(cacheDtype_) & 0xF) << 56);
  }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return store_->getTensor(output_).getShape(); }
  ThreadSize dispatchSize() const override { return {256, batchSize_, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "BatchedKVCacheWrite"; }

private:
  DataType cacheDtype_ = DataType::Float32;
  uint32_t batchSize_, kvDim_, alignedKvDim_, headDim_, kStride_, vStride_, kOffset_, vOffset_;
};

/// Prefill attention over the populated cache: token i's query (rotated by the kernel) attends rows
/// [0, positions[i]] (operators/impl/attention/AttentionOp.cpp:374-450).
class BatchedAttentionReadCacheOpNode : public OpNode {
public:
  static constexpr uint32_t kVariant = 2;
  BatchedAttentionReadCacheOpNode(TensorStore &store, const Tensor &q, const Tensor &kCache, const Tensor &vCache,
                                  const Tensor &positions, const Tensor &cosTable, const Tensor &sinTable, uint32_t batchSize,
                                  uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint32_t qStride, uint32_t qOffset,
                                  const Tensor &preallocOutput = {}, std::optional<uint32_t> spec = {});
  DataType outputDtype() const override { return DataType::Float32; }
  size_t shaderKey() const override {
    return static_cast<size_t>(op_) | (size_t{1} << 33) | ((static_cast<size_t>(dtype_) & 0xF) << 56);
  }
  std::optional<std::vector<uint32_t>> shader() const override;
  std::vector<uint32_t> outputShape() const override { return {batchSize_, nHeads_ * headDim_}; }
  ThreadSize dispatchSize() const override { return {nHeads_ * 256, batchSize_, 1}; }
  std::vector<uint8_t> pushConstants() const override;
  std::string displayName() const override { return "BatchedAttentionReadCache"; }

private:
  DataType dtype_ = DataType::Float32;
  uint32_t batchSize_, nHeads_, nKvHeads_, headDim_, alignedKvDim_, nRep_, qStride_, qOffset_;
  float scale_;
};

// ---- VariantSelector: tuning_data.json rules (runtime/VariantSelector.cpp:242-428) ----------
class VariantSelector {
public:
  static VariantSelector &instance();
  bool loadTuningData();  ///< $CUT_TUNING_DATA, ./tuning_data.json, ~/.cut/tuning_data.json
  bool loadFromFile(const std::string &path);
  bool loadFromString(const std::string &json);
  void clear();
  int select(const std::string &operatorName, const std::vector<uint32_t> &shape, int defaultVariant,
             const std::string &backend = "") const;
  bool isLoaded() const { return loaded_; }

private:
  VariantSelector() = default;
  struct Rule {
    int variant = 0;
    int64_t totalElementsMin = -1, totalElementsMax = -1;
    std::vector<int64_t> shape;
  };
  struct OperatorRules {
    int defaultVariant = 0;
    std::vector<Rule> rules;
  };
  bool loaded_ = false;
  std::unordered_map<std::string, OperatorRules> operators_;
};

// ---- Dispatcher ----------------------------------------------------------------------
class Dispatcher {
public:
  explicit Dispatcher(TensorStore *store);
  bool encode(std::unique_ptr<OpNode> node) { return encode(*node); }
  bool encode(OpNode &node);
  void encodeBarrier();
  size_t cachedShaders() const { return shaderCache_.size(); }

private:
  TensorStore *store_;
  ComputeInterface *iface_;
  std::unordered_map<size_t, Tensor> shaderCache_;
  Tensor getOrCreateShader(const OpNode &node);
};

// ---- Operations (the methods of the path and of its neighbours in a layer) and a minimal Runtime ---------------------
class Operations {
public:
  Operations(TensorStore *store, Dispatcher *dispatcher) : store_(store), dispatcher_(dispatcher) {}
  Tensor matmul(const Tensor &a, const Tensor &packedB, const Tensor &scales, std::optional<uint32_t> spec = {});
  Tensor matmulUnary(OperatorEnum unaryOp, const Tensor &a, const Tensor &packedB, const Tensor &scales,
                     std::optional<uint32_t> spec = {});
  Tensor matmulBinary(OperatorEnum binaryOp, const Tensor &a, const Tensor &packedB, const Tensor &scales,
                      const Tensor &d, std::optional<uint32_t> spec = {});
  /// C = A * dequant(rawBlocks): rawBlocks is a 1-D Int8 tensor holding N rows of GGUF blocks.
  Tensor matmulBlocks(const Tensor &a, const Tensor &rawBlocks, DequantFormat format, uint32_t N,
                      std::optional<uint32_t> spec = {});
  Tensor matmulBlocksUnary(OperatorEnum unaryOp, const Tensor &a, const Tensor &rawBlocks, DequantFormat format,
                           uint32_t N, std::optional<uint32_t> spec = {});
  Tensor matmulBlocksBinary(OperatorEnum binaryOp, const Tensor &a, const Tensor &rawBlocks, DequantFormat format,
                            uint32_t N, const Tensor &d, std::optional<uint32_t> spec = {});
  /// The block-layout matmul with a runner's extras (fused RMSNorm of A, paired gate / up rows, staging and
  /// overlap flags); `fusion` / `fusionOp` / `d` as in matmulBlocksUnary / matmulBlocksBinary.
  Tensor matmulBlocksFused(const Tensor &a, const Tensor &rawBlocks, DequantFormat format, uint32_t N,
                           const MatMulBlockOptions &opt, MatMulFusion fusion = MatMulFusion::None, OperatorEnum fusionOp = {},
                           const Tensor &d = {});
  /// out[r, i] = unary(in[r, 2i]) * in[r, 2i + 1] for a Float32 [rows, 2F] input.
  Tensor gluPairs(const Tensor &in, OperatorEnum unaryOp);
  Tensor transposeQ4(const Tensor &packedInput, uint32_t N, uint32_t K);
  Tensor dequantize(const Tensor &rawData, uint32_t format, uint32_t rows, uint32_t cols);
  /// Raw blocks of `format` -> Q8_0 GGUF blocks (a 1-D Int8 tensor matmulBlocks takes with DequantFormat::Q8_0).
  Tensor requantQ8Blocks(const Tensor &rawData, DequantFormat format, uint32_t rows, uint32_t cols);
  Tensor rmsNorm(const Tensor &x, const Tensor &weight, float eps = 1e-5f, std::optional<uint32_t> spec = {});
  Tensor embedding(const Tensor &indices, const Tensor &weight, const Tensor &preallocOutput = {},
                   std::optional<uint32_t> spec = {});
  /// Embedding gathered from a [dim, vocab] head (runtime/Operations.cpp:1044-1052).
  Tensor embeddingCol(const Tensor &indices, const Tensor &matrix, const Tensor &scales, const Tensor &preallocOutput = {},
                      std::optional<uint32_t> spec = {});
  /// Whole-tensor reduction (the reference's per-dimension form is outside this path).
  Tensor reduce(OperatorEnum op, const Tensor &a, std::optional<uint32_t> spec = {});
  Tensor attention(const Tensor &q, const Tensor &kCache, const Tensor &vCache, const Tensor &runtimeParams, uint32_t nHeads,
                   uint32_t nKvHeads, uint32_t headDim, const Tensor &preallocOutput = {});
  void batchedKVCacheWrite(const Tensor &k, const Tensor &v, const Tensor &kCache, const Tensor &vCache, const Tensor &positions,
                           const Tensor &cosTable, const Tensor &sinTable, uint32_t batchSize, uint32_t nKvHeads, uint32_t headDim,
                           uint32_t kStride, uint32_t vStride, uint32_t kOffset, uint32_t vOffset);
  Tensor batchedAttentionReadCache(const Tensor &q, const Tensor &kCache, const Tensor &vCache, const Tensor &positions,
                                   const Tensor &cosTable, const Tensor &sinTable, uint32_t batchSize, uint32_t nHeads,
                                   uint32_t nKvHeads, uint32_t headDim, uint32_t qStride, uint32_t qOffset,
                                   const Tensor &preallocOutput = {});
  Tensor fusedRoPEKVWrite(const Tensor &q, const Tensor &k, const Tensor &v, const Tensor &runtimeParams, const Tensor &cosTable,
                          const Tensor &sinTable, const Tensor &kCache, const Tensor &vCache, uint32_t headDim);
  void barrier() { dispatcher_->encodeBarrier(); }

private:
  Tensor dispatch(std::unique_ptr<OpNode> node);
  TensorStore *store_;
  Dispatcher *dispatcher_;
};

class Runtime {
public:
  explicit Runtime(std::unique_ptr<ComputeInterface> iface);
  explicit Runtime(int device = 0);  ///< B200 backend on `device`
  Tensor createTensor(const std::vector<uint32_t> &shape, DataType dtype, const void *src = nullptr) {
    return store_.createTensor(shape, dtype, src);
  }
  const ComputeBuffer &getTensor(const Tensor &t) const { return store_.getTensor(t); }
  /// Flushes pending dispatches, then copies `bytes` unpadded bytes of `t` to host memory.
  void copyFromTensor(const Tensor &t, void *dst, size_t bytes);
  void copyToTensor(const Tensor &t, const void *src, size_t bytes);
  void flush();
  Operations &ops() { return ops_; }
  TensorStore &store() { return store_; }
  ComputeInterface &iface() { return *iface_; }

private:
  std::unique_ptr<ComputeInterface> iface_;
  TensorStore store_;
  Dispatcher dispatcher_;
  Operations ops_;
};

}  // namespace cut
