// GGUF file -> device weights, without the CPU detour.
//
// The reference reads a tensor into a std::vector, dequantises or plane-splits it on one CPU thread
// and uploads the result (interface/loader/gguf/gguf_reader.cpp:15-58, 326-501;
// interface/runner/llama/llama.cpp:831-866, 934-1027).  Here the header is parsed on the host, the raw
// blocks of a tensor go to the device as they lie in the file, and whatever re-encoding is still
// needed runs there: the quantized matmul reads Q8_0 / Q4_0 / Q4_K blocks directly, every other
// block format is turned into Q8_0 blocks by a device kernel (the runner's own Q8 path), fused
// QKV / gate+up weights are concatenations of raw rows.
#pragma once

#include <cstdint>
#include <map>
#include <optional>
#include <string>
#include <vector>

#include "cut_api.h"

namespace cut {

/// GGML tensor types the loader knows (interface/loader/gguf/gguf_types.hpp:17-53).
enum class GGMLType : uint32_t { F32 = 0, F16 = 1, Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q8_0 = 8, Q4_K = 12, Q5_K = 13, Q6_K = 14, BF16 = 30 };

struct GGUFTensorInfo {
  std::string name;
  std::vector<uint64_t> dims;  ///< innermost first: {K, N} for a weight of N rows
  uint32_t type = 0;           ///< GGMLType code as stored
  uint64_t offset = 0;         ///< from the start of the tensor data section
  uint64_t elements() const;
  uint64_t bytes() const;      ///< 0 for a type whose block geometry is unknown here
};

/// Header, metadata scalars and tensor directory of a little-endian GGUF v2 / v3 file
/// (gguf_reader.cpp:15-58, 268-291).  Tensor bytes are read on demand.
class GGUFFile {
public:
  explicit GGUFFile(const std::string &path);  ///< throws std::runtime_error on a malformed file
  uint32_t version() const { return version_; }
  uint32_t alignment() const { return alignment_; }
  uint64_t dataOffset() const { return dataOffset_; }
  const std::vector<GGUFTensorInfo> &tensors() const { return tensors_; }
  bool has(const std::string &name) const { return index_.count(name) != 0; }
  const GGUFTensorInfo &info(const std::string &name) const;
  /// Scalar metadata (integers, floats and bools widened; arrays are skipped, strings kept apart).
  std::optional<double> metaNumber(const std::string &key) const;
  std::optional<std::string> metaString(const std::string &key) const;
  /// The tensor's bytes as stored (GGUFReader::read_tensor_raw).
  std::vector<uint8_t> readRaw(const std::string &name) const;

private:
  std::string path_;
  uint32_t version_ = 0, alignment_ = 32;
  uint64_t dataOffset_ = 0, fileSize_ = 0;
  std::vector<GGUFTensorInfo> tensors_;
  std::map<std::string, size_t> index_;
  std::map<std::string, double> numbers_;
  std::map<std::string, std::string> strings_;
};

/// Block geometry {weights per block, bytes per block} of a GGML type, or nullopt.
std::optional<std::pair<uint32_t, uint32_t>> ggmlBlockGeometry(uint32_t type);
/// The dequant / matmul format code of a GGML block type, or nullopt (F32 / F16 are not block formats).
std::optional<DequantFormat> ggmlDequantFormat(uint32_t type);

/// A weight on the device in the form Operations::matmulBlocks takes.
struct BlockWeight {
  Tensor raw;            ///< 1-D Int8 tensor: N rows of blocks along K
  DequantFormat format;  ///< Q8_0, Q4_0 or Q4_K
  uint32_t N = 0, K = 0;
  bool requantized = false;  ///< the file's format was re-encoded to Q8_0 on the device
};

class GGUFUploader {
public:
  GGUFUploader(Runtime &rt, const GGUFFile &file) : rt_(rt), file_(file) {}
  /// One 2-D weight.  Q8_0 / Q4_0 / Q4_K blocks are uploaded as they are; Q4_1 / Q5_0 / Q5_K / Q6_K / BF16 are
  /// uploaded raw and re-encoded to Q8_0 blocks on the device.
  BlockWeight upload(const std::string &name);
  /// Several weights that share K as one weight of the summed rows, in the order given (fused QKV:
  /// llama.cpp:831-866).  Same matmul-native format everywhere: a byte concatenation; otherwise every part
  /// goes through the Q8_0 re-encode first, as the reference's fused path does.
  BlockWeight uploadFused(const std::vector<std::string> &names);
  /// Gate and up projections as one weight whose rows alternate (gate_i, up_i): the layout of the
  /// paired-row mat-vec (SiLU(gate) * up in its epilogue).  Both must have the same native format and shape.
  BlockWeight uploadPaired(const std::string &gate, const std::string &up);
  /// Any tensor as fp32 [rows, cols] on the device (block formats through the dequant operator; F32 as is,
  /// F16 widened on the host).
  Tensor uploadF32(const std::string &name);

private:
  BlockWeight fromRaw(std::vector<uint8_t> &&bytes, uint32_t type, uint32_t N, uint32_t K);
  Runtime &rt_;
  const GGUFFile &file_;
};

}  // namespace cut
