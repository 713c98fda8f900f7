// GGUF header parsing and weight upload (see gguf_upload.h).
#include "gguf_upload.h"

#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace cut {
namespace {

constexpr uint32_t kMagic = 0x46554747u;  // "GGUF", little-endian

// gguf_types.hpp:56-70
enum ValueType : uint32_t { U8 = 0, I8 = 1, U16 = 2, I16 = 3, U32 = 4, I32 = 5, F32v = 6, BOOLv = 7, STR = 8, ARR = 9, U64 = 10, I64 = 11, F64 = 12 };

struct Reader {
  FILE *f;
  uint64_t pos = 0, size = 0;
  void need(uint64_t n) const {
    if (pos + n > size) throw std::runtime_error("GGUF: file ends inside the header");
  }
  void bytes(void *dst, uint64_t n) {
    need(n);
    if (n && fread(dst, 1, n, f) != n) throw std::runtime_error("GGUF: read error");
    pos += n;
  }
  void skip(uint64_t n) {
    need(n);
    if (fseek(f, (long)n, SEEK_CUR) != 0) throw std::runtime_error("GGUF: seek error");
    pos += n;
  }
  template <typename T> T get() {
    T v;
    bytes(&v, sizeof(T));
    return v;
  }
  std::string str() {
    const uint64_t n = get<uint64_t>();
    if (n > (1u << 24)) throw std::runtime_error("GGUF: implausible string length");
    std::string s(n, '\0');
    bytes(s.data(), n);
    return s;
  }
};

uint64_t scalarSize(uint32_t t) {
  switch (t) {
    case U8: case I8: case BOOLv: return 1;
    case U16: case I16: return 2;
    case U32: case I32: case F32v: return 4;
    case U64: case I64: case F64: return 8;
    default: return 0;
  }
}

// Reads one value; numbers are returned widened, strings through `s`, arrays are skipped.
bool readValue(Reader &r, uint32_t type, double &num, std::string &s, bool &isString) {
  isString = false;
  switch (type) {
    case U8: num = r.get<uint8_t>(); return true;
    case I8: num = r.get<int8_t>(); return true;
    case U16: num = r.get<uint16_t>(); return true;
    case I16: num = r.get<int16_t>(); return true;
    case U32: num = r.get<uint32_t>(); return true;
    case I32: num = r.get<int32_t>(); return true;
    case F32v: num = r.get<float>(); return true;
    case BOOLv: num = r.get<uint8_t>() != 0; return true;
    case U64: num = (double)r.get<uint64_t>(); return true;
    case I64: num = (double)r.get<int64_t>(); return true;
    case F64: num = r.get<double>(); return true;
    case STR: s = r.str(); isString = true; return true;
    case ARR: {
      const uint32_t et = r.get<uint32_t>();
      const uint64_t n = r.get<uint64_t>();
      if (et == STR) {
        for (uint64_t i = 0; i < n; ++i) r.skip(r.get<uint64_t>());
      } else if (et == ARR) {
        throw std::runtime_error("GGUF: nested arrays are not supported");
      } else {
        const uint64_t es = scalarSize(et);
        if (!es) throw std::runtime_error("GGUF: unsupported array element type");
        r.skip(n * es);
      }
      return false;
    }
    default: throw std::runtime_error("GGUF: unsupported metadata value type " + std::to_string(type));
  }
}

}  // namespace

std::optional<std::pair<uint32_t, uint32_t>> ggmlBlockGeometry(uint32_t type) {
  switch (static_cast<GGMLType>(type)) {  // gguf_types.hpp:109-150
    case GGMLType::F32: return {{1u, 4u}};
    case GGMLType::F16: return {{1u, 2u}};
    case GGMLType::BF16: return {{1u, 2u}};
    case GGMLType::Q4_0: return {{32u, 18u}};
    case GGMLType::Q4_1: return {{32u, 20u}};
    case GGMLType::Q5_0: return {{32u, 22u}};
    case GGMLType::Q8_0: return {{32u, 34u}};
    case GGMLType::Q4_K: return {{256u, 144u}};
    case GGMLType::Q5_K: return {{256u, 176u}};
    case GGMLType::Q6_K: return {{256u, 210u}};
    default: return std::nullopt;
  }
}

std::optional<DequantFormat> ggmlDequantFormat(uint32_t type) {
  switch (static_cast<GGMLType>(type)) {
    case GGMLType::BF16: return DequantFormat::BF16;
    case GGMLType::Q4_0: return DequantFormat::Q4_0;
    case GGMLType::Q4_1: return DequantFormat::Q4_1;
    case GGMLType::Q5_0: return DequantFormat::Q5_0;
    case GGMLType::Q8_0: return DequantFormat::Q8_0;
    case GGMLType::Q4_K: return DequantFormat::Q4_K;
    case GGMLType::Q5_K: return DequantFormat::Q5_K;
    case GGMLType::Q6_K: return DequantFormat::Q6_K;
    default: return std::nullopt;
  }
}

uint64_t GGUFTensorInfo::elements() const {
  uint64_t n = 1;
  for (uint64_t d : dims) n *= d;
  return n;
}

uint64_t GGUFTensorInfo::bytes() const {
  const auto g = ggmlBlockGeometry(type);
  if (!g) return 0;
  const uint64_t n = elements();
  return (n + g->first - 1) / g->first * g->second;
}

GGUFFile::GGUFFile(const std::string &path) : path_(path) {
  FILE *f = fopen(path.c_str(), "rb");
  if (!f) throw std::runtime_error("GGUF: cannot open " + path);
  struct Closer {
    FILE *f;
    ~Closer() { fclose(f); }
  } closer{f};
  fseek(f, 0, SEEK_END);
  fileSize_ = (uint64_t)ftell(f);
  fseek(f, 0, SEEK_SET);
  Reader r{f, 0, fileSize_};
  if (r.get<uint32_t>() != kMagic) throw std::runtime_error("GGUF: invalid magic number");  // big-endian files are not read
  version_ = r.get<uint32_t>();
  if (version_ < 2 || version_ > 3) throw std::runtime_error("GGUF: unsupported version " + std::to_string(version_));
  const uint64_t nTensors = r.get<uint64_t>(), nMeta = r.get<uint64_t>();
  if (nTensors > (1u << 20) || nMeta > (1u << 20)) throw std::runtime_error("GGUF: implausible header counts");
  for (uint64_t i = 0; i < nMeta; ++i) {
    const std::string key = r.str();
    const uint32_t type = r.get<uint32_t>();
    double num = 0;
    std::string s;
    bool isString = false;
    if (readValue(r, type, num, s, isString)) {
      if (isString) strings_[key] = std::move(s);
      else numbers_[key] = num;
    }
  }
  tensors_.reserve(nTensors);
  for (uint64_t i = 0; i < nTensors; ++i) {
    GGUFTensorInfo t;
    t.name = r.str();
    const uint32_t nd = r.get<uint32_t>();
    if (nd > 8) throw std::runtime_error("GGUF: tensor " + t.name + " has " + std::to_string(nd) + " dimensions");
    t.dims.resize(nd);
    for (uint32_t d = 0; d < nd; ++d) t.dims[d] = r.get<uint64_t>();
    t.type = r.get<uint32_t>();
    t.offset = r.get<uint64_t>();
    index_[t.name] = tensors_.size();
    tensors_.push_back(std::move(t));
  }
  if (auto a = metaNumber("general.alignment")) alignment_ = (uint32_t)*a;
  if (alignment_ == 0 || (alignment_ & (alignment_ - 1))) throw std::runtime_error("GGUF: alignment must be a power of two");
  dataOffset_ = (r.pos + alignment_ - 1) / alignment_ * alignment_;
  for (const auto &t : tensors_) {
    const uint64_t b = t.bytes();
    if (b && dataOffset_ + t.offset + b > fileSize_) throw std::runtime_error("GGUF: tensor " + t.name + " extends past the end of the file");
  }
}

const GGUFTensorInfo &GGUFFile::info(const std::string &name) const {
  auto it = index_.find(name);
  if (it == index_.end()) throw std::runtime_error("Tensor not found: " + name);
  return tensors_[it->second];
}

std::optional<double> GGUFFile::metaNumber(const std::string &key) const {
  auto it = numbers_.find(key);
  if (it == numbers_.end()) return std::nullopt;
  return it->second;
}

std::optional<std::string> GGUFFile::metaString(const std::string &key) const {
  auto it = strings_.find(key);
  if (it == strings_.end()) return std::nullopt;
  return it->second;
}

std::vector<uint8_t> GGUFFile::readRaw(const std::string &name) const {
  const GGUFTensorInfo &t = info(name);
  const uint64_t n = t.bytes();
  if (!n) throw std::runtime_error("GGUF: tensor " + name + " has a type this loader does not know (" + std::to_string(t.type) + ")");
  std::vector<uint8_t> out(n);
  FILE *f = fopen(path_.c_str(), "rb");
  if (!f) throw std::runtime_error("GGUF: cannot reopen " + path_);
  const bool ok = fseek(f, (long)(dataOffset_ + t.offset), SEEK_SET) == 0 && fread(out.data(), 1, n, f) == n;
  fclose(f);
  if (!ok) throw std::runtime_error("GGUF: short read of tensor " + name);
  return out;
}

// ---- upload ---------------------------------------------------------------------------------

namespace {
bool matmulNative(uint32_t type) {
  const auto t = static_cast<GGMLType>(type);
  return t == GGMLType::Q8_0 || t == GGMLType::Q4_0 || t == GGMLType::Q4_K;
}
void shape2d(const GGUFTensorInfo &t, uint32_t &N, uint32_t &K) {
  if (t.dims.size() != 2) throw std::runtime_error("GGUF upload: tensor " + t.name + " is not 2-D");
  K = (uint32_t)t.dims[0];
  N = (uint32_t)t.dims[1];
}
}  // namespace

BlockWeight GGUFUploader::fromRaw(std::vector<uint8_t> &&bytes, uint32_t type, uint32_t N, uint32_t K) {
  const auto fmt = ggmlDequantFormat(type);
  if (!fmt) throw std::runtime_error("GGUF upload: type " + std::to_string(type) + " is not a block format");
  const auto geo = *ggmlBlockGeometry(type);
  if (K % geo.first != 0) throw std::runtime_error("GGUF upload: K is not a whole number of blocks");
  BlockWeight w;
  w.N = N;
  w.K = K;
  Tensor raw = rt_.createTensor({(uint32_t)bytes.size()}, DataType::Int8, bytes.data());
  if (matmulNative(type)) {
    w.raw = raw;
    w.format = *fmt;
  } else {
    w.raw = rt_.ops().requantQ8Blocks(raw, *fmt, N, K);
    w.format = DequantFormat::Q8_0;
    w.requantized = true;
  }
  return w;
}

BlockWeight GGUFUploader::upload(const std::string &name) {
  const GGUFTensorInfo &t = file_.info(name);
  uint32_t N, K;
  shape2d(t, N, K);
  return fromRaw(file_.readRaw(name), t.type, N, K);
}

BlockWeight GGUFUploader::uploadFused(const std::vector<std::string> &names) {
  if (names.empty()) throw std::runtime_error("GGUF upload: no tensors to fuse");
  uint32_t K = 0, total = 0;
  bool sameNative = true;
  const uint32_t type0 = file_.info(names[0]).type;
  for (const auto &n : names) {
    uint32_t rows, cols;
    shape2d(file_.info(n), rows, cols);
    if (K && cols != K) throw std::runtime_error("GGUF upload: fused tensors must share K");
    K = cols;
    total += rows;
    sameNative = sameNative && file_.info(n).type == type0 && matmulNative(type0);
  }
  if (sameNative) {  // rows are contiguous runs of blocks: concatenating tensors concatenates rows
    std::vector<uint8_t> all;
    for (const auto &n : names) {
      auto part = file_.readRaw(n);
      all.insert(all.end(), part.begin(), part.end());
    }
    return fromRaw(std::move(all), type0, total, K);
  }
  // mixed formats: each part becomes Q8_0 blocks on the device (native Q8_0 parts stay as they are), then one
  // device buffer receives them back to back
  BlockWeight w;
  w.N = total;
  w.K = K;
  w.format = DequantFormat::Q8_0;
  w.requantized = true;
  const uint64_t rowBytes = (uint64_t)(K / 32) * 34;
  std::vector<uint8_t> host((size_t)total * rowBytes);
  uint64_t at = 0;
  for (const auto &n : names) {
    const GGUFTensorInfo &t = file_.info(n);
    uint32_t rows, cols;
    shape2d(t, rows, cols);
    const auto fmt = ggmlDequantFormat(t.type);
    if (!fmt) throw std::runtime_error("GGUF upload: tensor " + n + " is not a block format");
    auto bytes = file_.readRaw(n);
    Tensor raw = rt_.createTensor({(uint32_t)bytes.size()}, DataType::Int8, bytes.data());
    Tensor q8 = static_cast<GGMLType>(t.type) == GGMLType::Q8_0 ? raw : rt_.ops().requantQ8Blocks(raw, *fmt, rows, cols);
    rt_.copyFromTensor(q8, host.data() + at, (size_t)rows * rowBytes);
    at += (uint64_t)rows * rowBytes;
  }
  w.raw = rt_.createTensor({(uint32_t)host.size()}, DataType::Int8, host.data());
  return w;
}

BlockWeight GGUFUploader::uploadPaired(const std::string &gate, const std::string &up) {
  const GGUFTensorInfo &g = file_.info(gate), &u = file_.info(up);
  uint32_t N, K, N2, K2;
  shape2d(g, N, K);
  shape2d(u, N2, K2);
  if (N != N2 || K != K2 || g.type != u.type || !matmulNative(g.type))
    throw std::runtime_error("GGUF upload: paired rows need two tensors of one matmul-native format and shape");
  const auto geo = *ggmlBlockGeometry(g.type);
  const uint64_t rowBytes = (uint64_t)(K / geo.first) * geo.second;
  const auto a = file_.readRaw(gate), b = file_.readRaw(up);
  std::vector<uint8_t> both((size_t)2 * N * rowBytes);
  for (uint32_t i = 0; i < N; ++i) {
    std::memcpy(both.data() + (size_t)(2 * i) * rowBytes, a.data() + (size_t)i * rowBytes, rowBytes);
    std::memcpy(both.data() + (size_t)(2 * i + 1) * rowBytes, b.data() + (size_t)i * rowBytes, rowBytes);
  }
  return fromRaw(std::move(both), g.type, 2 * N, K);
}

Tensor GGUFUploader::uploadF32(const std::string &name) {
  const GGUFTensorInfo &t = file_.info(name);
  const uint32_t cols = (uint32_t)t.dims.at(0);
  uint64_t rows64 = 1;
  for (size_t d = 1; d < t.dims.size(); ++d) rows64 *= t.dims[d];
  const uint32_t rows = (uint32_t)rows64;
  auto bytes = file_.readRaw(name);
  const auto type = static_cast<GGMLType>(t.type);
  if (type == GGMLType::F32) return rt_.createTensor({rows, cols}, DataType::Float32, bytes.data());
  if (type == GGMLType::F16) {  // widened on the host with the loader's own conversion (gguf_reader.cpp:515-539)
    std::vector<float> f((size_t)rows * cols);
    const uint16_t *h = reinterpret_cast<const uint16_t *>(bytes.data());
    for (size_t i = 0; i < f.size(); ++i) {
      const uint32_t s = (h[i] >> 15) & 1u, e = (h[i] >> 10) & 0x1Fu, m = h[i] & 0x3FFu;
      uint32_t bits;
      if (e == 0) {
        if (m == 0) {
          bits = s << 31;
        } else {  // subnormal: renormalise
          uint32_t mm = m, ee = 113;
          while (!(mm & 0x400u)) mm <<= 1, --ee;
          bits = (s << 31) | (ee << 23) | ((mm & 0x3FFu) << 13);
        }
      } else if (e == 31) {
        bits = (s << 31) | 0x7F800000u | (m << 13);
      } else {
        bits = (s << 31) | ((e + 112) << 23) | (m << 13);
      }
      std::memcpy(&f[i], &bits, 4);
    }
    return rt_.createTensor({rows, cols}, DataType::Float32, f.data());
  }
  const auto fmt = ggmlDequantFormat(t.type);
  if (!fmt) throw std::runtime_error("GGUF upload: tensor " + name + " has no dequantiser here");
  Tensor raw = rt_.createTensor({(uint32_t)bytes.size()}, DataType::Int8, bytes.data());
  return rt_.ops().dequantize(raw, (uint32_t)*fmt, rows, cols);
}

}  // namespace cut
