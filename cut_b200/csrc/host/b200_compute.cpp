// B200Compute: the ComputeInterface backend that stands where the reference's
// core/backends/cuda/CudaCompute stands (CudaCompute.cpp:56-330,
// CudaCommandBuffer.cpp:128-360), rebuilt for precompiled sm_100a kernels:
//   * createShaderModule() decodes a kernel descriptor and binds it to a C ABI
//     entry point -- no SPIR-V hashing, no NVRTC;
//   * buffers are plain cudaMalloc allocations that honour the reference's
//     padding rule (inner dimension to 4 elements, size to 16 bytes) and are
//     zero-filled so padding never holds garbage;
//   * a command buffer is the recorded dispatch list; submit() launches it on the
//     backend's stream, submitReusable() captures it into a CUDA graph that
//     resubmit() replays with one launch;
//   * a dispatch whose descriptor no kernel covers throws (the reference logs and
//     skips it).
// Errors surface as std::runtime_error, like the reference's logErr.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <string>
#include <unordered_map>

#include "../../../include/cutb.h"
#include "cut_api.h"

namespace cut {
namespace {

void cudaCheck(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

void cutbCheck(int rc, const char *what) {
  if (rc != CUTB_OK) throw std::runtime_error(std::string(what) + ": " + cutb_last_error());
}

struct DeviceBuffer : ComputeBuffer {
  ~DeviceBuffer() override {
    if (owned && data) {
      if (mapped) cudaFreeHost(hostPtr);
      else cudaFree(data);
    }
    if (counter) *counter -= size();
    if (count) --*count;
  }
  bool owned = true, mapped = false;
  void *hostPtr = nullptr;
  ComputeHandle parent;  // keeps the parent of a view alive
  size_t *counter = nullptr, *count = nullptr;
};

struct ShaderModule : ComputeHandle::Slot {
  KernelDesc desc;
};

// A block of device scratch.  Command buffers share the current block; a recorded CUDA graph has the
// block's address baked into its kernel arguments, so the block lives as long as any command buffer
// that was built on it (a bigger request allocates a new block instead of replacing this one).
struct Scratch {
  explicit Scratch(size_t n, bool zero) : bytes(n) {
    cudaCheck(cudaMalloc(&ptr, n), "cudaMalloc(scratch)");
    if (zero) cudaCheck(cudaMemset(ptr, 0, n), "cudaMemset(scratch)");
  }
  ~Scratch() { cudaFree(ptr); }  // cudaFree waits for work that still uses the block
  Scratch(const Scratch &) = delete;
  Scratch &operator=(const Scratch &) = delete;
  void *ptr = nullptr;
  size_t bytes = 0;
};

struct CommandBufferObj : ComputeHandle::Slot {
  ~CommandBufferObj() override {
    if (gatherHost) cudaFreeHost(gatherHost);
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
  }
  std::vector<ComputeDispatch> dispatches;  // keeps every bound buffer alive until the work is done
  std::shared_ptr<Scratch> workspace, attnWs;  // the scratch blocks its launches (and its graph) point into
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  // Results of a reusable command buffer -- outputs no later dispatch of it consumes -- are copied to pinned host
  // memory right behind every replay, back to back in stream order, so that reading them costs one wait for the
  // step instead of one device round trip per tensor: {buffer, bytes, offset in the pinned block}.
  struct Shadow {
    const void *dev;
    size_t bytes, off;
  };
  std::unordered_map<const void *, Shadow> shadows;  // keyed by the buffer object
  uint64_t shadowEpoch = 0;                         // the backend epoch at which the pinned copies were requested
  // with more than one result: {result -> its place in the backend's device block}, read by one gather launch
  // (host-mapped pinned memory), followed by a single download of the block
  cutb_copy_range *gatherHost = nullptr, *gatherDev = nullptr;
  uint32_t gatherCount = 0;
  size_t gatherBytes = 0, gatherMax = 0;
};

int cutbFormat(uint32_t f) {
  switch (static_cast<DequantFormat>(f)) {
    case DequantFormat::Q8_0: return CUTB_Q8_0;
    case DequantFormat::Q4_0: return CUTB_Q4_0;
    case DequantFormat::Q4_K: return CUTB_Q4_K;
    case DequantFormat::Q5_K: return CUTB_Q5_K;  // dequant only; the matmul entry point rejects them
    case DequantFormat::Q6_K: return CUTB_Q6_K;
    case DequantFormat::BF16: return CUTB_BF16;
    case DequantFormat::Q4_1: return CUTB_Q4_1;
    case DequantFormat::Q5_0: return CUTB_Q5_0;
    default: throw std::runtime_error("B200Compute: block format has no kernel");
  }
}

class B200Compute final : public ComputeInterface {
public:
  explicit B200Compute(int device) : device_(device) {
    int n = 0;
    cudaCheck(cudaGetDeviceCount(&n), "cudaGetDeviceCount");
    if (device < 0 || device >= n) throw std::runtime_error("B200Compute: no such CUDA device");
    cudaCheck(cudaSetDevice(device), "cudaSetDevice");
    cudaDeviceProp prop;
    cudaCheck(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    if (prop.major < 10)
      throw std::runtime_error("B200Compute: kernels are built for sm_100a; device is sm_" + std::to_string(prop.major) +
                               std::to_string(prop.minor));
    totalMem_ = prop.totalGlobalMem;
    smemOptin_ = (uint32_t)prop.sharedMemPerBlockOptin;
    cudaCheck(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    cudaCheck(cudaMalloc(&status_, sizeof(int)), "cudaMalloc(status)");
    cudaCheck(cudaMemsetAsync(status_, 0, sizeof(int), stream_), "cudaMemset(status)");
    cudaCheck(cudaHostAlloc((void **)&stage_, kStageBytes, cudaHostAllocDefault), "cudaHostAlloc(staging)");
    cudaCheck(cudaHostAlloc((void **)&shadowStage_, kShadowBytes + 256, cudaHostAllocDefault), "cudaHostAlloc(results)");
    cudaCheck(cudaMalloc((void **)&devStage_, kStageBytes), "cudaMalloc(upload block)");
    cudaCheck(cudaMalloc((void **)&devResults_, kShadowBytes), "cudaMalloc(result block)");
    cudaCheck(cudaHostAlloc((void **)&tableHost_, kTableEntries * sizeof(cutb_copy_range), cudaHostAllocMapped), "cudaHostAlloc(table)");
    cudaCheck(cudaHostGetDevicePointer((void **)&tableDev_, tableHost_, 0), "cudaHostGetDevicePointer");
    caps_.backend = ComputeBackend::CUDA;
    caps_.cooperativeMatrix = true;  // tensor-core variants exist
    caps_.integerDotProduct = true;
    caps_.subgroupSize = 32;
  }
  ~B200Compute() override {
    cudaStreamSynchronize(stream_);
    lastReplayed_ = nullptr;
    lastReplayedHandle_.reset();
    pendingUploads_.clear();
    cudaFree(devStage_);
    cudaFree(devResults_);
    cudaFreeHost(tableHost_);
    workspace_.reset();
    attnWs_.reset();
    cudaFree(status_);
    cudaFreeHost(stage_);
    cudaFreeHost(shadowStage_);
    cudaStreamDestroy(stream_);
  }

  ComputeHandle createBuffer(const std::vector<uint32_t> &shape, DataType dtype, const void *host, bool) override {
    auto buf = std::make_shared<DeviceBuffer>();
    buf->describe(shape, dtype);
    buf->id = ++nextId_;
    const size_t bytes = buf->size() ? buf->size() : 16;
    cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
    cudaCheck(cudaMalloc(&buf->data, bytes), "cudaMalloc");
    buf->counter = &activeBytes_;
    buf->count = &bufferCount_;
    activeBytes_ += buf->size();
    ++bufferCount_;
    ComputeHandle h(buf);
    if (!host || buf->size() != buf->calculateActualSize())
      cudaCheck(cudaMemsetAsync(buf->data, 0, bytes, stream_), "cudaMemsetAsync");  // padding reads as zero
    if (host) upload(h, *buf, host);
    return h;
  }

  ComputeHandle createBufferMapped(const std::vector<uint32_t> &shape, DataType dtype, const void *host, bool) override {
    auto buf = std::make_shared<DeviceBuffer>();
    buf->describe(shape, dtype);
    buf->id = ++nextId_;
    buf->mapped = true;
    const size_t bytes = buf->size() ? buf->size() : 16;
    cudaCheck(cudaHostAlloc(&buf->hostPtr, bytes, cudaHostAllocMapped), "cudaHostAlloc");
    std::memset(buf->hostPtr, 0, bytes);
    cudaCheck(cudaHostGetDevicePointer(&buf->data, buf->hostPtr, 0), "cudaHostGetDevicePointer");
    if (host) copyActualToAligned(host, buf->hostPtr, *buf);
    buf->counter = &activeBytes_;
    buf->count = &bufferCount_;
    activeBytes_ += buf->size();
    ++bufferCount_;
    return ComputeHandle(buf);
  }

  ComputeHandle createBufferView(const ComputeHandle &parent, size_t byteOffset, const std::vector<uint32_t> &shape,
                                 DataType dtype) override {
    auto *p = parent.as<DeviceBuffer>();
    if (!p) throw std::runtime_error("createBufferView: parent is not a buffer");
    if (byteOffset % bufferOffsetAlignment() != 0) throw std::runtime_error("createBufferView: offset must be a multiple of 256");
    auto buf = std::make_shared<DeviceBuffer>();
    buf->describe(shape, dtype);
    if (byteOffset + buf->size() > p->size()) throw std::runtime_error("createBufferView: view exceeds the parent buffer");
    buf->id = ++nextId_;
    buf->owned = false;
    buf->parent = parent;
    buf->data = (uint8_t *)p->data + byteOffset;
    return ComputeHandle(buf);
  }

  void copyDataToBuffer(const void *host, const ComputeHandle &dest, size_t copySize, size_t srcOffset, size_t destOffset,
                        bool, bool) override {
    auto *b = dest.as<DeviceBuffer>();
    if (!b) throw std::runtime_error("copyDataToBuffer: not a buffer");
    if (lastReplayed_ && lastReplayed_->shadows.count(b)) ++epoch_;  // a result buffer is overwritten: its pinned copy is stale
    if (srcOffset == 0 && destOffset == 0 && copySize == b->calculateActualSize()) {
      upload(dest, *b, host);
      return;
    }
    if (b->innerDimSize() != b->innerDimPadded()) throw std::runtime_error("copyDataToBuffer: partial copy into a padded buffer");
    if (destOffset + copySize > b->size()) throw std::runtime_error("copyDataToBuffer: out of range");
    uploadBytes(dest, (uint8_t *)b->data + destOffset, (const uint8_t *)host + srcOffset, copySize);
  }

  void copyDataFromBuffer(const ComputeHandle &src, void *host, size_t copySize, size_t srcOffset, size_t destOffset, bool,
                          bool) override {
    auto *b = src.as<DeviceBuffer>();
    if (!b) throw std::runtime_error("copyDataFromBuffer: not a buffer");
    flushUploads();
    if (lastReplayed_ && lastReplayed_->shadowEpoch == epoch_) {
      auto it = lastReplayed_->shadows.find(b);
      if (it != lastReplayed_->shadows.end() && srcOffset + copySize <= it->second.bytes) {
        cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");  // (already drained after wait())
        std::memcpy((uint8_t *)host + destOffset, shadowStage_ + it->second.off + srcOffset, copySize);
        return;
      }
    }
    if (b->innerDimSize() == b->innerDimPadded() || b->getShape().size() <= 1) {
      if (srcOffset + copySize > b->size()) throw std::runtime_error("copyDataFromBuffer: out of range");
      if (copySize <= kStageBytes) {
        // through the pinned block: a device-to-host copy into pageable memory is staged by the driver with an
        // extra round trip per call
        cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");  // staged uploads have left the block
        stageUsed_ = 0;
        cudaCheck(cudaMemcpyAsync(stage_, (const uint8_t *)b->data + srcOffset, copySize, cudaMemcpyDeviceToHost, stream_),
                  "cudaMemcpyAsync(D2H)");
        cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
        std::memcpy((uint8_t *)host + destOffset, stage_, copySize);
        return;
      }
      cudaCheck(cudaMemcpyAsync((uint8_t *)host + destOffset, (const uint8_t *)b->data + srcOffset, copySize,
                                cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync(D2H)");
      cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
      return;
    }
    if (srcOffset != 0 || copySize > b->calculateActualSize())
      throw std::runtime_error("copyDataFromBuffer: partial copy out of a padded buffer");
    std::vector<uint8_t> bounce(b->size()), dense(b->calculateActualSize());
    cudaCheck(cudaMemcpyAsync(bounce.data(), b->data, b->size(), cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync(D2H)");
    cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    copyAlignedToActual(bounce.data(), dense.data(), *b);
    std::memcpy((uint8_t *)host + destOffset, dense.data(), copySize);
  }

  ComputeHandle createShaderModule(const std::vector<uint32_t> &words) override {
    auto desc = KernelDesc::decode(words);
    if (!desc) throw std::runtime_error("B200Compute: not a kernel descriptor");
    switch (desc->op) {
      case MatMulQ8: case MatMulQ4: case MatMulQBlocks: case Dequantize: case RequantQ8Blocks: case TransposeQ4: case GluPairs: break;
      case RMSNorm: case Embedding: case EmbeddingCol: case ReduceArgmax: case ReduceArgmin: case Attention: break;
      case CacheWrite:
        if (desc->variant != FusedRoPEKVWriteOpNode::kVariant && desc->variant != BatchedKVCacheWriteOpNode::kVariant) throw std::runtime_error("B200Compute: no kernel for this CacheWrite operator");
        break;
      default: throw std::runtime_error("B200Compute: no kernel for operator " + std::to_string(desc->op));
    }
    if (desc->op == Dequantize || desc->op == MatMulQBlocks) (void)cutbFormat(desc->format);
    auto m = std::make_shared<ShaderModule>();
    m->desc = *desc;
    m->id = ++nextId_;
    return ComputeHandle(m);
  }

  const ComputeBuffer &getBuffer(const ComputeHandle &h) const override {
    auto *b = h.as<DeviceBuffer>();
    if (!b) throw std::runtime_error("getBuffer: invalid buffer handle");
    return *b;
  }
  size_t bufferCount() const override { return bufferCount_; }
  size_t activeBufferMemoryBytes() const override { return activeBytes_; }
  uint32_t maxSharedMemoryPerBlock() const override { return smemOptin_; }
  size_t deviceTotalMemoryBytes() const override { return totalMem_; }
  void flushTransfers() override {
    flushUploads();
    cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
  }

protected:
  ComputeHandle executeDispatches(std::vector<ComputeDispatch> &&dispatches, bool reusable) override {
    auto cb = std::make_shared<CommandBufferObj>();
    cb->id = ++nextId_;
    cb->dispatches = std::move(dispatches);
    cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
    flushUploads();
    // scratch is sized before anything is launched or captured
    size_t need = 0;
    std::vector<cutb_qmatmul_desc> descs(cb->dispatches.size());
    for (size_t i = 0; i < cb->dispatches.size(); ++i)
      if (isMatmul(cb->dispatches[i])) {
        descs[i] = matmulDesc(cb->dispatches[i]);
        const size_t w = cutb_qmatmul_workspace_bytes(&descs[i]);
        need = w > need ? w : need;
      }
    ensureWorkspace(need);
    size_t attnNeed = 0;
    for (const auto &d : cb->dispatches)
      if (!d.isBarrier && descOf(d).op == Attention && descOf(d).variant == 0) {
        const AttnPC pc = pushConstants<AttnPC>(d);
        const size_t w = cutb_attention_workspace_bytes(pc.nHeads, pc.nKvHeads, pc.headDim, buf(d, 1).getShape()[0]);
        attnNeed = w > attnNeed ? w : attnNeed;
      }
    ensureAttnWorkspace(attnNeed);
    cb->workspace = workspace_;
    cb->attnWs = attnWs_;
    ++epoch_;  // device buffers change: pinned copies of earlier results are stale
    statusShadowed_ = false;
    if (reusable) {
      // results: dense outputs of at most 256 KB that no later dispatch binds, while they fit the pinned block
      size_t off = 0;
      for (size_t i = 0; i < cb->dispatches.size(); ++i) {
        const ComputeDispatch &d = cb->dispatches[i];
        if (d.isBarrier || !d.outputHandle) continue;
        auto *ob = d.outputHandle.as<DeviceBuffer>();
        if (!ob || ob->size() == 0 || ob->size() > (256u << 10)) continue;
        if (ob->innerDimSize() != ob->innerDimPadded() && ob->getShape().size() > 1) continue;
        // (a view and its parent are one allocation: compare the roots)
        auto root = [](const DeviceBuffer *b) {
          while (b->parent)
            if (auto *up = b->parent.as<DeviceBuffer>()) b = up;
            else break;
          return b;
        };
        bool consumed = false;
        for (size_t j = i + 1; j < cb->dispatches.size() && !consumed; ++j)
          for (const auto &bnd : cb->dispatches[j].bindings)
            if (bnd.isHandle())
              if (auto *other = bnd.handle.as<DeviceBuffer>())
                if (root(other) == root(ob)) consumed = true;
        const size_t need = (ob->size() + 255) & ~size_t(255);
        if (consumed || off + need > kShadowBytes || cb->shadows.size() >= 64) continue;
        cb->shadows[ob] = CommandBufferObj::Shadow{ob->data, ob->size(), off};
        off += need;
      }
      if (cb->shadows.size() > 1) {
        cudaCheck(cudaHostAlloc((void **)&cb->gatherHost, cb->shadows.size() * sizeof(cutb_copy_range), cudaHostAllocMapped),
                  "cudaHostAlloc(gather table)");
        cudaCheck(cudaHostGetDevicePointer((void **)&cb->gatherDev, cb->gatherHost, 0), "cudaHostGetDevicePointer");
        for (const auto &kv : cb->shadows) {
          cb->gatherHost[cb->gatherCount++] = cutb_copy_range{kv.second.dev, devResults_ + kv.second.off, kv.second.bytes};
          cb->gatherMax = std::max(cb->gatherMax, kv.second.bytes);
        }
        cb->gatherBytes = off;
      }
      // warm launch outside capture (first-use kernel attributes), then capture the same list
      launchAll(*cb, descs);
      cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
      cudaCheck(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
      try {
        launchAll(*cb, descs);
      } catch (...) {
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(stream_, &g);
        if (g) cudaGraphDestroy(g);
        throw;
      }
      cudaCheck(cudaStreamEndCapture(stream_, &cb->graph), "cudaStreamEndCapture");
      cudaCheck(cudaGraphInstantiate(&cb->exec, cb->graph, 0), "cudaGraphInstantiate");
    } else {
      launchAll(*cb, descs);
    }
    return ComputeHandle(cb);
  }

  void replay(const ComputeHandle &h) override {
    auto *cb = h.as<CommandBufferObj>();
    if (!cb || !cb->exec) throw std::runtime_error("resubmit: not a reusable command buffer");
    flushUploads();
    cudaCheck(cudaGraphLaunch(cb->exec, stream_), "cudaGraphLaunch");
    ++epoch_;
    if (cb->gatherCount > 1) {  // one gather launch into the device block, one download of the block
      cutbCheck(cutb_copy_batch(cb->gatherDev, cb->gatherCount, cb->gatherMax, stream_), "result gather");
      cudaCheck(cudaMemcpyAsync(shadowStage_, devResults_, cb->gatherBytes, cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync(results)");
    } else {
      for (const auto &kv : cb->shadows)
        cudaCheck(cudaMemcpyAsync(shadowStage_ + kv.second.off, kv.second.dev, kv.second.bytes, cudaMemcpyDeviceToHost, stream_),
                  "cudaMemcpyAsync(results)");
    }
    cudaCheck(cudaMemcpyAsync(shadowStage_ + kShadowBytes, status_, sizeof(int), cudaMemcpyDeviceToHost, stream_),
              "cudaMemcpyAsync(status)");
    statusShadowed_ = true;
    cb->shadowEpoch = epoch_;
    lastReplayedHandle_ = h;  // keeps the command buffer (and its shadow plan) alive
    lastReplayed_ = cb;
  }

  void waitFor(const ComputeHandle &) override {
    flushUploads();
    cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    int st = 0;
    if (statusShadowed_) std::memcpy(&st, shadowStage_ + kShadowBytes, sizeof(int));  // copied behind the replay
    else cudaCheck(cudaMemcpy(&st, status_, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
    if (st != 0) {
      statusShadowed_ = false;
      cudaMemset(status_, 0, sizeof(int));
      throw std::runtime_error(std::string("B200Compute: kernel reported ") + cutb_status_string(st));
    }
  }

private:
  // Host bytes -> device.  Small transfers (a decode step's activations, token ids, positions) are copied into a
  // pinned block at once -- the caller's memory is free again when the call returns -- and sent LATER, together:
  // everything that is pending when the stream is next used (a submit or replay, a download, a flush) goes out as
  // ONE host-to-device copy of the pinned range into a device block, followed by one launch that moves every piece
  // to its tensor.  A step that uploads 32 activations pays one transfer, not 32.  The pinned block is reused from
  // the start once it is full and the stream has drained.  (`keep` holds the destination alive until then.)
  void uploadBytes(const ComputeHandle &keep, void *dev, const void *host, size_t bytes) {
    if (bytes <= kStageBytes / 4 && reinterpret_cast<uintptr_t>(dev) % 16 == 0) {
      const size_t need = (bytes + 255) & ~size_t(255);
      if (stageUsed_ + need > kStageBytes) {
        flushUploads();
        cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
        stageUsed_ = 0;
      }
      std::memcpy(stage_ + stageUsed_, host, bytes);
      pendingUploads_.push_back(Pending{keep, dev, stageUsed_, bytes});
      stageUsed_ += need;
      return;
    }
    flushUploads();  // keep the order of writes to one buffer
    cudaCheck(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync(H2D)");
    cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
  }

  // Sends what uploadBytes() has collected; called before anything else is put on the stream.
  void flushUploads() {
    if (pendingUploads_.empty()) return;
    if (pendingUploads_.size() <= 2) {  // (one or two pieces: a copy each is cheaper than a copy and a launch)
      for (const Pending &u : pendingUploads_)
        cudaCheck(cudaMemcpyAsync(u.dev, stage_ + u.off, u.bytes, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync(H2D)");
    } else {
      const size_t first = pendingUploads_.front().off;
      const size_t last = pendingUploads_.back().off + ((pendingUploads_.back().bytes + 255) & ~size_t(255));
      cudaCheck(cudaMemcpyAsync(devStage_ + first, stage_ + first, last - first, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync(H2D)");
      const size_t n = pendingUploads_.size();
      if (n > kTableEntries) throw std::runtime_error("B200Compute: too many pending uploads");
      if (tableUsed_ + n > kTableEntries) {  // the table is read by launches that may still be queued
        cudaCheck(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
        tableUsed_ = 0;
      }
      uint64_t maxBytes = 0;
      for (size_t i = 0; i < n; ++i) {
        const Pending &u = pendingUploads_[i];
        tableHost_[tableUsed_ + i] = cutb_copy_range{devStage_ + u.off, u.dev, u.bytes};
        maxBytes = std::max<uint64_t>(maxBytes, u.bytes);
      }
      cutbCheck(cutb_copy_batch(tableDev_ + tableUsed_, (uint32_t)n, maxBytes, stream_), "upload scatter");
      tableUsed_ += n;
    }
    pendingUploads_.clear();
  }

  void upload(const ComputeHandle &keep, DeviceBuffer &b, const void *host) {
    if (b.innerDimSize() == b.innerDimPadded() || b.getShape().size() <= 1) {
      uploadBytes(keep, b.data, host, std::min(b.size(), b.calculateActualSize()));
      return;
    }
    std::vector<uint8_t> bounce(b.size(), 0);
    copyActualToAligned(host, bounce.data(), b);
    uploadBytes(keep, b.data, bounce.data(), b.size());
  }

  // Scratch only grows, and never in place: command buffers recorded earlier keep the block they
  // were built on (their graphs replay with its address), new work gets a new, larger block.
  void ensureWorkspace(size_t need) {
    if (workspace_ && need <= workspace_->bytes) return;
    if (need == 0) return;
    workspace_ = std::make_shared<Scratch>(need, false);
  }

  void ensureAttnWorkspace(size_t need) {
    if (attnWs_ && need <= attnWs_->bytes) return;
    if (need == 0) return;
    attnWs_ = std::make_shared<Scratch>(need, true);  // its arrival counters start at zero
  }
  void *wsPtr() const { return workspace_ ? workspace_->ptr : nullptr; }
  size_t wsBytes() const { return workspace_ ? workspace_->bytes : 0; }
  void *attnPtr() const { return attnWs_ ? attnWs_->ptr : nullptr; }
  size_t attnBytes() const { return attnWs_ ? attnWs_->bytes : 0; }

  struct AttnPC {
    uint32_t nHeads, nKvHeads, headDim, kvDim, alignedKvDim, nRep;
    float scale;
  };

  static const KernelDesc &descOf(const ComputeDispatch &d) {
    auto *m = d.shader.as<ShaderModule>();
    if (!m) throw std::runtime_error("B200Compute: dispatch without a kernel");
    return m->desc;
  }
  static bool isMatmul(const ComputeDispatch &d) {
    if (d.isBarrier) return false;
    const uint32_t op = descOf(d).op;
    return op == MatMulQ8 || op == MatMulQ4 || op == MatMulQBlocks;
  }

  const DeviceBuffer &buf(const ComputeDispatch &d, size_t i) const {
    if (i >= d.bindings.size() || !d.bindings[i].isHandle()) throw std::runtime_error("B200Compute: missing buffer binding");
    auto *b = d.bindings[i].handle.as<DeviceBuffer>();
    if (!b) throw std::runtime_error("B200Compute: binding is not a buffer");
    return *b;
  }
  template <typename T> static T pushConstants(const ComputeDispatch &d) {
    for (const auto &b : d.bindings)
      if (!b.isHandle() && b.bytes.size() == sizeof(T)) {
        T v;
        std::memcpy(&v, b.bytes.data(), sizeof(T));
        return v;
      }
    throw std::runtime_error("B200Compute: dispatch without push constants");
  }

  // bindings (A, packedB, [scalesB], D, C, push constants) -> C ABI descriptor
  cutb_qmatmul_desc matmulDesc(const ComputeDispatch &d) const {
    const KernelDesc &k = descOf(d);
    struct PC {
      uint32_t M, K, N, strideA, strideB, strideC, scaleStride;
    } pc;
    struct PCN {  // with the fused RMSNorm: one more word
      uint32_t M, K, N, strideA, strideB, strideC, scaleStride;
      float normEps;
    };
    const bool blocks = k.op == MatMulQBlocks;
    float normEps = 0.f;
    if (blocks && (k.flags & kBlockFlagRmsNorm)) {
      const PCN n = pushConstants<PCN>(d);
      std::memcpy(&pc, &n, sizeof(pc));
      normEps = n.normEps;
    } else {
      pc = pushConstants<PC>(d);
    }
    cutb_qmatmul_desc q{};
    const DeviceBuffer &A = buf(d, 0), &W = buf(d, 1);
    size_t i = 2;
    q.layout = blocks ? CUTB_LAYOUT_GGUF_BLOCKS : CUTB_LAYOUT_KN_PLANES;
    q.format = blocks ? cutbFormat(k.format) : (k.op == MatMulQ8 ? CUTB_Q8_0 : CUTB_Q4_0);
    q.affine = (int32_t)k.affine;
    q.a_dtype = A.getDtype() == DataType::Float16 ? CUTB_F16 : CUTB_F32;
    if (A.getDtype() != DataType::Float16 && A.getDtype() != DataType::Float32)
      throw std::runtime_error("matmul: A must be Float32 or Float16");
    q.M = pc.M; q.K = pc.K; q.N = pc.N;
    q.A = A.data;
    q.lda = pc.strideA;
    q.W = W.data;
    q.W_bytes = W.size();
    if (!blocks) {
      const DeviceBuffer &S = buf(d, i++);
      q.scales = S.data;
      q.ldb = pc.strideB;
      q.lds = pc.scaleStride;
    }
    // bindings behind the weights: D (binary fusion) or a stand-in, [the RMSNorm weight], C
    const bool binary = k.fusionType == (uint32_t)MatMulFusion::Binary;
    const DeviceBuffer *D = nullptr, *NW = nullptr;
    if (binary) D = &buf(d, i++);
    if (blocks && (k.flags & kBlockFlagRmsNorm)) NW = &buf(d, i++);
    if (!binary) D = &buf(d, i++);
    const DeviceBuffer &C = buf(d, i++);
    q.C = (float *)C.data;
    q.ldc = pc.strideC;
    q.D = (const float *)D->data;
    q.ldd = (pc.N + 3) & ~3u;
    if (NW) {
      q.a_norm_weight = (const float *)NW->data;
      q.a_norm_eps = normEps;
    }
    q.fusion_type = (int32_t)k.fusionType;
    q.fusion_op = (int32_t)k.fusionOp;
    // plane-layout variant indices (the reference's Tiled / GemvKPar8 / CoopMat ... tables) all map onto the library's
    // own choice for that layout: the coalesced mat-vec up to four rows, the any-shape kernel beyond; block
    // variants are the C ABI's own
    q.variant = blocks ? (int32_t)k.variant : CUTB_VARIANT_AUTO;
    q.workspace = wsPtr();
    q.workspace_bytes = wsBytes();
    q.status = status_;
    q.flags = blocks ? k.flags : 0;  // kBlockFlag* are the C ABI's CUTB_FLAG_* bit for bit
    return q;
  }

  void launchAll(CommandBufferObj &cb, std::vector<cutb_qmatmul_desc> &descs) {
    for (size_t i = 0; i < cb.dispatches.size(); ++i) {
      const ComputeDispatch &d = cb.dispatches[i];
      if (d.isBarrier) continue;  // one in-order stream: dispatches are already ordered
      const KernelDesc &k = descOf(d);
      if (isMatmul(d)) {
        descs[i].workspace = wsPtr();
        descs[i].workspace_bytes = wsBytes();
        cutbCheck(cutb_qmatmul(&descs[i], stream_), d.label.c_str());
      } else if (k.op == Dequantize) {
        struct PC {
          uint32_t rows, cols, outputStride;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &raw = buf(d, 0), &out = buf(d, 1);
        cutbCheck(cutb_dequant(cutbFormat(k.format), raw.data, raw.size(), (float *)out.data, pc.rows, pc.cols,
                               pc.outputStride, stream_), "Dequantize");
      } else if (k.op == RequantQ8Blocks) {
        struct PC {
          uint32_t rows, cols;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &raw = buf(d, 0), &out = buf(d, 1);
        cutbCheck(cutb_requant_q8_0_blocks(cutbFormat(k.format), raw.data, raw.size(), out.data, pc.rows, pc.cols, stream_),
                  "RequantQ8Blocks");
      } else if (k.op == GluPairs) {
        struct PC {
          uint32_t rows, colsOut, strideIn, strideOut;
        } pc = pushConstants<PC>(d);
        cutbCheck(cutb_glu_pairs((const float *)buf(d, 0).data, (float *)buf(d, 1).data, pc.rows, pc.colsOut, pc.strideIn, pc.strideOut,
                                 (int)k.fusionOp, stream_), "GluPairs");
      } else if (k.op == TransposeQ4) {
        struct PC {
          uint32_t N, K, strideInHalf, strideOutHalf;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &in = buf(d, 0), &out = buf(d, 1);
        cutbCheck(cutb_transpose_q4(in.data, out.data, pc.N, pc.K, pc.strideInHalf, pc.strideOutHalf, stream_), "TransposeQ4");
      } else if (k.op == RMSNorm) {
        struct PC {
          uint32_t dim, alignedDim;
          float eps;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &x = buf(d, 0), &w = buf(d, 1), &y = buf(d, 2);
        cutbCheck(cutb_rmsnorm(k.dtypeA == (uint32_t)DataType::Float16 ? CUTB_F16 : CUTB_F32, x.data, w.data, y.data, d.size.y,
                               pc.dim, pc.alignedDim, pc.eps, stream_), "RMSNorm");
      } else if (k.op == Embedding) {
        struct PC {
          uint32_t numIndices, embDim;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &idx = buf(d, 0), &table = buf(d, 1), &out = buf(d, 2);
        cutbCheck(cutb_embedding((const uint32_t *)idx.data, (const float *)table.data, (float *)out.data, pc.numIndices,
                                 pc.embDim, table.getShape()[0], status_, stream_), "Embedding");
      } else if (k.op == EmbeddingCol) {
        struct PC {
          uint32_t numIndices, embDim, vocabStride, scaleStride, outStride;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &idx = buf(d, 0), &mat = buf(d, 1), &sc = buf(d, 2), &out = buf(d, 3);
        cutbCheck(cutb_embedding_col((int)k.fusionType, (const uint32_t *)idx.data, mat.data, sc.data, (float *)out.data, pc.numIndices,
                                     pc.embDim, mat.getShape()[1], pc.vocabStride, pc.scaleStride, pc.outStride, status_, stream_),
                  "EmbeddingCol");
      } else if (k.op == CacheWrite && k.variant == BatchedKVCacheWriteOpNode::kVariant) {
        struct PC {
          uint32_t batchSize, kvDim, alignedKvDim, headDim, halfDim, kStride, vStride, kOffset, vOffset;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &kc = buf(d, 2);
        cutbCheck(cutb_batched_kv_write(k.dtypeA == (uint32_t)DataType::Float16 ? CUTB_F16 : CUTB_F32,
                                        (const float *)buf(d, 0).data + pc.kOffset, (const float *)buf(d, 1).data + pc.vOffset, pc.kStride,
                                        pc.vStride, (const uint32_t *)buf(d, 4).data, (const float *)buf(d, 5).data,
                                        (const float *)buf(d, 6).data, kc.data, buf(d, 3).data, pc.batchSize, pc.kvDim, pc.headDim,
                                        pc.alignedKvDim, kc.getShape()[0], status_, stream_), "BatchedKVCacheWrite");
      } else if (k.op == Attention && k.variant == BatchedAttentionReadCacheOpNode::kVariant) {
        struct PC {
          uint32_t batchSize, nHeads, nKvHeads, headDim, alignedKvDim, nRep;
          float scale;
          uint32_t halfDim, qStride, qOffset;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &kc = buf(d, 1), &out = buf(d, 6);
        cutbCheck(cutb_batched_attention(k.dtypeA == (uint32_t)DataType::Float16 ? CUTB_F16 : CUTB_F32,
                                         (const float *)buf(d, 0).data + pc.qOffset, pc.qStride, kc.data, buf(d, 2).data,
                                         (const uint32_t *)buf(d, 3).data, (const float *)buf(d, 4).data, (const float *)buf(d, 5).data,
                                         (float *)out.data, out.innerDimPadded(), pc.batchSize, pc.nHeads, pc.nKvHeads, pc.headDim,
                                         pc.alignedKvDim, kc.getShape()[0], pc.scale, status_, stream_), "BatchedAttentionReadCache");
      } else if (k.op == CacheWrite) {  // fused RoPE + KV-cache write
        struct PC {
          uint32_t qDim, kvDim, headDim, halfDim, alignedKvDim;
        } pc = pushConstants<PC>(d);
        const DeviceBuffer &kc = buf(d, 6);
        cutbCheck(cutb_rope_kv_write(k.dtypeA == (uint32_t)DataType::Float16 ? CUTB_F16 : CUTB_F32, (const float *)buf(d, 0).data,
                                     (const float *)buf(d, 1).data, (const float *)buf(d, 2).data, (const uint32_t *)buf(d, 3).data,
                                     (const float *)buf(d, 4).data, (const float *)buf(d, 5).data, kc.data, buf(d, 7).data,
                                     (float *)buf(d, 8).data, pc.qDim, pc.kvDim, pc.headDim, pc.alignedKvDim, kc.getShape()[0],
                                     status_, stream_), "FusedRoPEKVWrite");
      } else if (k.op == Attention) {
        const AttnPC pc = pushConstants<AttnPC>(d);
        const DeviceBuffer &kc = buf(d, 1);
        cutbCheck(cutb_attention_decode(k.dtypeA == (uint32_t)DataType::Float16 ? CUTB_F16 : CUTB_F32, (const float *)buf(d, 0).data,
                                        kc.data, buf(d, 2).data, (const uint32_t *)buf(d, 3).data, (float *)buf(d, 4).data, pc.nHeads,
                                        pc.nKvHeads, pc.headDim, pc.alignedKvDim, kc.getShape()[0], pc.scale, attnPtr(), attnBytes(),
                                        status_, stream_), "Attention");
      } else if (k.op == ReduceArgmax || k.op == ReduceArgmin) {
        const uint32_t n = pushConstants<uint32_t>(d);
        cutbCheck(cutb_argreduce(k.op == ReduceArgmax, (const float *)buf(d, 0).data, (float *)buf(d, 1).data, n, stream_),
                  "ReduceArg");
      } else {
        throw std::runtime_error("B200Compute: no kernel for dispatch " + d.label);
      }
    }
  }

  int device_;
  cudaStream_t stream_ = nullptr;
  static constexpr size_t kStageBytes = 4u << 20;
  uint8_t *stage_ = nullptr;  // pinned
  size_t stageUsed_ = 0;
  struct Pending {
    ComputeHandle keep;
    void *dev;
    size_t off, bytes;
  };
  std::vector<Pending> pendingUploads_;
  uint8_t *devStage_ = nullptr, *devResults_ = nullptr;  // device blocks behind the pinned ones
  static constexpr size_t kTableEntries = 4096;
  cutb_copy_range *tableHost_ = nullptr, *tableDev_ = nullptr;  // host-mapped: ranges of the batched copies
  size_t tableUsed_ = 0;
  static constexpr size_t kShadowBytes = 4u << 20;
  uint8_t *shadowStage_ = nullptr;  // pinned: results of the last replayed command buffer, then the status word
  uint64_t epoch_ = 0;               // bumped by everything that can change a device buffer
  bool statusShadowed_ = false;
  ComputeHandle lastReplayedHandle_;
  CommandBufferObj *lastReplayed_ = nullptr;
  std::shared_ptr<Scratch> workspace_;  // split-K partial sums / cast activations of the matmuls
  std::shared_ptr<Scratch> attnWs_;     // attention scratch; its arrival counters start at zero and every launch leaves them zero
  int *status_ = nullptr;
  size_t nextId_ = 0, activeBytes_ = 0, bufferCount_ = 0, totalMem_ = 0;
  uint32_t smemOptin_ = 0;
};

}  // namespace

std::unique_ptr<ComputeInterface> createB200Compute(int device) { return std::make_unique<B200Compute>(device); }

}  // namespace cut
