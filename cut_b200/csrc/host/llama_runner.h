// The llama runner's per-token step on the operator API, in C++.
//
// The reference's runner loads a GGUF model, builds its per-layer operator graphs once and, per token,
// writes {pos, seqLen} and the token id into small device buffers, resubmits the recorded command buffer
// and reads the arg-max back (interface/runner/llama/llama.cpp: config 1070-1130, runLayer 2045-2084,
// forward 2090-2166; replay core/backends/cuda/CudaCommandBuffer.cpp:261-307).  LlamaRunner is that
// sequence over this host's Operations: weights go to the device as raw GGUF blocks (GGUFUploader: fused
// QKV, paired gate / up rows, Q8_0 re-encode of the formats the matmul does not read), the whole token --
// embedding, per layer [QKV projection (RMSNorm fused into its staging), RoPE + KV-cache write,
// attention, output projection + residual, gate-and-up projection with SiLU(gate) * up in its epilogue
// (RMSNorm fused), down projection + residual], final norm + LM head, arg-max -- is recorded into one
// reusable command buffer (one CUDA graph on the B200 backend) and replayed per token.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "cut_api.h"
#include "gguf_upload.h"

namespace cut {

/// Model geometry read from the GGUF metadata ("<arch>.embedding_length", ".block_count", ...; llama.cpp:1084-1118).
struct LlamaConfig {
  uint32_t dim = 0, nLayers = 0, nHeads = 0, nKvHeads = 0, headDim = 0, ffnDim = 0, vocab = 0, maxSeq = 512;
  float ropeFreqBase = 10000.0f, normEps = 1e-5f;
  uint32_t qDim() const { return nHeads * headDim; }
  uint32_t kvDim() const { return nKvHeads * headDim; }
};

struct LlamaRunnerOptions {
  uint32_t maxSeq = 512;   ///< capped by the model's context_length
  bool fuseNorm = true;    ///< RMSNorms inside the projections that consume them (decode mat-vec only)
  bool gluPairs = true;    ///< gate and up as one weight of row pairs, SiLU(gate) * up in the epilogue
  bool act16 = true;       ///< fp32 activations staged at one 16-bit level per 32-k block
  bool kvHalf = true;      ///< fp16 KV cache (the reference's default); false: fp32
};

class LlamaRunner {
public:
  /// Reads the configuration, uploads every weight and records the per-token step.  Throws
  /// std::runtime_error on a file that is not a llama-style model or whose shapes do not fit.
  LlamaRunner(Runtime &rt, const GGUFFile &file, const LlamaRunnerOptions &opt = {});
  const LlamaConfig &config() const { return cfg_; }
  /// One token at position `pos` (rows [0, pos) of the KV cache must hold the tokens before it): writes the
  /// two small buffers, replays the recorded step, returns the arg-max of the logits.
  uint32_t forward(uint32_t token, uint32_t pos);
  /// The prompt as one batch (llama.cpp prefillBatched): every projection is one matmul over all T tokens, K / V
  /// rows go to the cache through the batched RoPE write, every token attends over the rows up to its own.  Tokens
  /// take positions start .. start + T - 1 (start + T <= maxSeq); returns the arg-max after the last token, whose
  /// logits logits() then returns.  Not recorded: the dispatches run once.
  uint32_t prefill(const std::vector<uint32_t> &tokens, uint32_t start = 0);
  /// The logits of the last forward() or prefill() (vocab floats).
  std::vector<float> logits();
  /// Dispatches recorded per token (barriers not counted).
  size_t dispatchesPerToken() const { return dispatches_; }
  /// Bytes of block weights one token streams.
  uint64_t weightBytesPerToken() const { return weightBytes_; }

private:
  struct Layer {
    Tensor attnNorm, ffnNorm;
    BlockWeight wqkv, wq, wk, wv, wo, wgu, wgate, wup, wdown;
    Tensor kCache, vCache;
  };
  Tensor normWeight(const GGUFFile &file, const std::string &name) const;
  Tensor project(const Tensor &x, const BlockWeight &w, const Tensor &norm, MatMulFusion fusion, OperatorEnum fusionOp,
                 const Tensor &d, bool glu, bool overlap);
  void record();

  Runtime &rt_;
  LlamaConfig cfg_;
  LlamaRunnerOptions opt_;
  bool fusedQkv_ = false;
  std::vector<Layer> layers_;
  Tensor table_, finalNorm_, cosT_, sinT_, params_, token_, logits_, next_;
  Tensor lastLogits_;  ///< what logits() reads: the recorded step's or the last prefill's
  BlockWeight lmHead_;
  ComputeHandle cb_;
  size_t dispatches_ = 0;
  uint64_t weightBytes_ = 0;
};

}  // namespace cut
