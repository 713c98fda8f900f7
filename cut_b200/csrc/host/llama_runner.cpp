// LlamaRunner: the reference runner's per-token step recorded over this host's Operations
// (interface/runner/llama/llama.cpp:1070-1130, 2045-2166).
#include "llama_runner.h"

#include <cmath>
#include <cstring>
#include <stdexcept>

#include "../../../include/cutb.h"

namespace cut {

namespace {

uint32_t cutbFormatOf(DequantFormat f) {
  return f == DequantFormat::Q8_0 ? CUTB_Q8_0 : (f == DequantFormat::Q4_0 ? CUTB_Q4_0 : CUTB_Q4_K);
}

// Does the decode mat-vec split K for this shape (then it has no paired-row epilogue)?  Asked of the library's
// own planner with a descriptor that is never launched.
bool matvecSplitsK(DequantFormat f, uint32_t N, uint32_t K) {
  cutb_qmatmul_desc q{};
  q.format = (int32_t)cutbFormatOf(f);
  q.layout = CUTB_LAYOUT_GGUF_BLOCKS;
  q.a_dtype = CUTB_F32;
  q.M = 1;
  q.K = K;
  q.N = N;
  q.lda = K;
  q.ldc = N;
  q.A = q.W = reinterpret_cast<void *>(uintptr_t(256));
  q.C = reinterpret_cast<float *>(uintptr_t(256));
  q.W_bytes = ~0ull;
  q.variant = CUTB_VARIANT_GEMV_MMA;
  q.flags = CUTB_FLAG_ACT_16BIT | CUTB_FLAG_STAGE_PER_CTA;
  return cutb_qmatmul_workspace_bytes(&q) != 0;
}

uint32_t metaU32(const GGUFFile &f, const std::string &key, uint32_t fallback) {
  const auto v = f.metaNumber(key);
  return v ? (uint32_t)*v : fallback;
}

}  // namespace

Tensor LlamaRunner::normWeight(const GGUFFile &file, const std::string &name) const {
  const GGUFTensorInfo &t = file.info(name);
  if (t.type != (uint32_t)GGMLType::F32 || t.elements() != cfg_.dim)
    throw std::runtime_error("llama: " + name + " must be F32 [" + std::to_string(cfg_.dim) + "]");
  const auto bytes = file.readRaw(name);
  return rt_.createTensor({cfg_.dim}, DataType::Float32, bytes.data());
}

LlamaRunner::LlamaRunner(Runtime &rt, const GGUFFile &file, const LlamaRunnerOptions &opt) : rt_(rt), opt_(opt) {
  const std::string arch = file.metaString("general.architecture").value_or("llama");
  const std::string p = arch + ".";
  cfg_.dim = metaU32(file, p + "embedding_length", 0);
  cfg_.nLayers = metaU32(file, p + "block_count", 0);
  cfg_.nHeads = metaU32(file, p + "attention.head_count", 0);
  cfg_.nKvHeads = metaU32(file, p + "attention.head_count_kv", cfg_.nHeads);
  cfg_.ffnDim = metaU32(file, p + "feed_forward_length", 0);
  cfg_.ropeFreqBase = (float)file.metaNumber(p + "rope.freq_base").value_or(10000.0);
  cfg_.normEps = (float)file.metaNumber(p + "attention.layer_norm_rms_epsilon").value_or(1e-5);
  if (cfg_.dim == 0 || cfg_.nLayers == 0 || cfg_.nHeads == 0) throw std::runtime_error("Failed to read model config from GGUF metadata");
  cfg_.headDim = metaU32(file, p + "attention.key_length", cfg_.dim / cfg_.nHeads);
  const uint32_t modelCtx = metaU32(file, p + "context_length", 2048);
  cfg_.maxSeq = opt.maxSeq < modelCtx ? opt.maxSeq : modelCtx;
  if (cfg_.nKvHeads == 0 || cfg_.nHeads % cfg_.nKvHeads != 0) throw std::runtime_error("llama: head_count must be a multiple of head_count_kv");
  if (cfg_.ffnDim == 0 && file.has("blk.0.ffn_gate.weight")) cfg_.ffnDim = (uint32_t)file.info("blk.0.ffn_gate.weight").dims.at(1);
  if (!file.has("token_embd.weight")) throw std::runtime_error("llama: no token_embd.weight");
  cfg_.vocab = (uint32_t)file.info("token_embd.weight").dims.at(1);

  GGUFUploader up(rt, file);
  table_ = up.uploadF32("token_embd.weight");  // [vocab, dim] fp32 (block formats through the dequant operator)
  finalNorm_ = normWeight(file, "output_norm.weight");
  // an untied head, else the embedding matrix again (llama.cpp ties them when output.weight is missing)
  lmHead_ = up.upload(file.has("output.weight") ? "output.weight" : "token_embd.weight");
  weightBytes_ = rt.getTensor(lmHead_.raw).getShape()[0];

  // a fused QKV output is split into q / k / v by buffer views, which start on 256-byte boundaries
  fusedQkv_ = (cfg_.qDim() * 4) % 256 == 0 && (cfg_.kvDim() * 4) % 256 == 0;
  layers_.resize(cfg_.nLayers);
  for (uint32_t l = 0; l < cfg_.nLayers; ++l) {
    const std::string b = "blk." + std::to_string(l) + ".";
    Layer &L = layers_[l];
    L.attnNorm = normWeight(file, b + "attn_norm.weight");
    L.ffnNorm = normWeight(file, b + "ffn_norm.weight");
    if (fusedQkv_) {
      L.wqkv = up.uploadFused({b + "attn_q.weight", b + "attn_k.weight", b + "attn_v.weight"});
    } else {
      L.wq = up.upload(b + "attn_q.weight");
      L.wk = up.upload(b + "attn_k.weight");
      L.wv = up.upload(b + "attn_v.weight");
    }
    L.wo = up.upload(b + "attn_output.weight");
    const GGUFTensorInfo &g = file.info(b + "ffn_gate.weight"), &u = file.info(b + "ffn_up.weight");
    const auto gf = ggmlDequantFormat(g.type);
    const bool native = gf && (*gf == DequantFormat::Q8_0 || *gf == DequantFormat::Q4_0 || *gf == DequantFormat::Q4_K);
    const bool pair = opt.gluPairs && native && g.type == u.type && cfg_.dim % 256 == 0 && !matvecSplitsK(*gf, 2 * cfg_.ffnDim, cfg_.dim);
    if (pair) {
      L.wgu = up.uploadPaired(b + "ffn_gate.weight", b + "ffn_up.weight");
    } else {
      L.wgate = up.upload(b + "ffn_gate.weight");
      L.wup = up.upload(b + "ffn_up.weight");
    }
    L.wdown = up.upload(b + "ffn_down.weight");
    for (const BlockWeight *w : {&L.wqkv, &L.wq, &L.wk, &L.wv, &L.wo, &L.wgu, &L.wgate, &L.wup, &L.wdown})
      if (w->raw) weightBytes_ += rt.getTensor(w->raw).getShape()[0];
    const DataType kvT = opt.kvHalf ? DataType::Float16 : DataType::Float32;
    L.kCache = rt.createTensor({cfg_.maxSeq, cfg_.kvDim()}, kvT);
    L.vCache = rt.createTensor({cfg_.maxSeq, cfg_.kvDim()}, kvT);
  }

  // RoPE tables in float arithmetic, [maxSeq, headDim / 2] (llama.cpp:1652-1666)
  const uint32_t half = cfg_.headDim / 2;
  std::vector<float> c((size_t)cfg_.maxSeq * half), s(c.size());
  for (uint32_t i = 0; i < half; ++i) {
    const float freq = 1.0f / std::pow(cfg_.ropeFreqBase, (2.0f * (float)i) / (float)cfg_.headDim);
    for (uint32_t pos = 0; pos < cfg_.maxSeq; ++pos) {
      const float ang = (float)pos * freq;
      c[(size_t)pos * half + i] = std::cos(ang);
      s[(size_t)pos * half + i] = std::sin(ang);
    }
  }
  cosT_ = rt.createTensor({cfg_.maxSeq, half}, DataType::Float32, c.data());
  sinT_ = rt.createTensor({cfg_.maxSeq, half}, DataType::Float32, s.data());
  const uint32_t zero2[2] = {0, 1}, zero1 = 0;
  params_ = rt.createTensor({2}, DataType::UInt32, zero2);  // {pos, seqLen} (llama.cpp:2087-2094)
  token_ = rt.createTensor({1}, DataType::UInt32, &zero1);
  rt.flush();  // load-time re-encodes have run; nothing of them is recorded
  record();
}

// One projection of the step.  `norm`: the RMSNorm in front of it -- fused into the mat-vec's staging where that
// kernel runs (K a multiple of 256), an operator of its own otherwise.
Tensor LlamaRunner::project(const Tensor &x, const BlockWeight &w, const Tensor &norm, MatMulFusion fusion, OperatorEnum fusionOp,
                            const Tensor &d, bool glu, bool overlap) {
  Operations &ops = rt_.ops();
  const bool matvec = w.K % 256 == 0;  // one fp32 row: the decode mat-vec takes it
  Tensor in = x;
  MatMulBlockOptions o;
  if (matvec) {
    o.flags = (opt_.act16 ? kBlockFlagAct16 : 0u) | (overlap ? 0u : kBlockFlagNoOverlap) | (glu ? kBlockFlagGluPairs : 0u);
    if (norm && opt_.fuseNorm) {
      o.flags |= kBlockFlagRmsNorm;
      o.normWeight = norm;
      o.normEps = cfg_.normEps;
    }
  }
  if (norm && !(o.flags & kBlockFlagRmsNorm)) in = ops.rmsNorm(x, norm, cfg_.normEps);
  if (!matvec) {
    if (fusion == MatMulFusion::Unary) return ops.matmulBlocksUnary(fusionOp, in, w.raw, w.format, w.N);
    if (fusion == MatMulFusion::Binary) return ops.matmulBlocksBinary(fusionOp, in, w.raw, w.format, w.N, d);
    return ops.matmulBlocks(in, w.raw, w.format, w.N);
  }
  return ops.matmulBlocksFused(in, w.raw, w.format, w.N, o, fusion, fusionOp, d);
}

void LlamaRunner::record() {
  Operations &ops = rt_.ops();
  ComputeInterface &iface = rt_.iface();
  const uint32_t qDim = cfg_.qDim(), kvDim = cfg_.kvDim();
  Tensor x = ops.embedding(token_, table_);  // [1, dim]
  for (uint32_t l = 0; l < cfg_.nLayers; ++l) {
    Layer &L = layers_[l];
    Tensor q, k, v;
    if (fusedQkv_) {
      // (measured on the 32-layer step: the QKV mat-vec gains from starting under the previous layer's down projection)
      Tensor qkv = project(x, L.wqkv, L.attnNorm, MatMulFusion::None, {}, {}, false, l > 0);
      q = iface.createBufferView(qkv, 0, {qDim}, DataType::Float32);
      k = iface.createBufferView(qkv, (size_t)qDim * 4, {kvDim}, DataType::Float32);
      v = iface.createBufferView(qkv, (size_t)(qDim + kvDim) * 4, {kvDim}, DataType::Float32);
    } else {
      Tensor h = ops.rmsNorm(x, L.attnNorm, cfg_.normEps);
      q = project(h, L.wq, {}, MatMulFusion::None, {}, {}, false, false);
      k = project(h, L.wk, {}, MatMulFusion::None, {}, {}, false, false);
      v = project(h, L.wv, {}, MatMulFusion::None, {}, {}, false, false);
    }
    Tensor qRoped = ops.fusedRoPEKVWrite(q, k, v, params_, cosT_, sinT_, L.kCache, L.vCache, cfg_.headDim);
    ops.barrier();
    Tensor att = ops.attention(qRoped, L.kCache, L.vCache, params_, cfg_.nHeads, cfg_.nKvHeads, cfg_.headDim);
    Tensor x1 = project(att, L.wo, {}, MatMulFusion::Binary, BinaryAdd, x, false, false);
    Tensor act;
    if (L.wgu.raw) {
      act = project(x1, L.wgu, L.ffnNorm, MatMulFusion::Unary, UnarySilu, {}, true, true);
    } else {
      Tensor h = opt_.fuseNorm && cfg_.dim % 256 == 0 ? Tensor{} : ops.rmsNorm(x1, L.ffnNorm, cfg_.normEps);
      const Tensor &in = h ? h : x1;
      const Tensor nrm = h ? Tensor{} : L.ffnNorm;
      Tensor gate = project(in, L.wgate, nrm, MatMulFusion::Unary, UnarySilu, {}, false, true);
      act = project(in, L.wup, nrm, MatMulFusion::Binary, BinaryMul, gate, false, true);
    }
    x = project(act, L.wdown, {}, MatMulFusion::Binary, BinaryAdd, x1, false, false);
  }
  logits_ = project(x, lmHead_, finalNorm_, MatMulFusion::None, {}, {}, false, false);
  lastLogits_ = logits_;
  next_ = ops.reduce(ReduceArgmax, logits_);
  dispatches_ = iface.pendingDispatches();
  cb_ = iface.submitReusable();
  iface.wait(cb_);
}

uint32_t LlamaRunner::forward(uint32_t token, uint32_t pos) {
  if (pos >= cfg_.maxSeq) throw std::runtime_error("llama: position " + std::to_string(pos) + " is past the KV cache");
  if (token >= cfg_.vocab) throw std::runtime_error("llama: token id past the vocabulary");
  const uint32_t params[2] = {pos, pos + 1};
  rt_.copyToTensor(params_, params, sizeof(params));
  rt_.copyToTensor(token_, &token, sizeof(token));
  rt_.iface().resubmit(cb_);
  rt_.iface().wait(cb_);
  float best = 0.f;
  rt_.copyFromTensor(next_, &best, sizeof(best));
  lastLogits_ = logits_;
  return (uint32_t)best;
}

uint32_t LlamaRunner::prefill(const std::vector<uint32_t> &tokens, uint32_t start) {
  const uint32_t T = (uint32_t)tokens.size();
  if (T == 0 || (uint64_t)start + T > cfg_.maxSeq) throw std::runtime_error("llama: prefill takes 1 .. maxSeq - start tokens");
  for (uint32_t t : tokens)
    if (t >= cfg_.vocab) throw std::runtime_error("llama: token id past the vocabulary");
  Operations &ops = rt_.ops();
  ComputeInterface &iface = rt_.iface();
  const uint32_t qDim = cfg_.qDim(), kvDim = cfg_.kvDim();
  std::vector<uint32_t> pos(T);
  for (uint32_t i = 0; i < T; ++i) pos[i] = start + i;
  Tensor tok = rt_.createTensor({T}, DataType::UInt32, tokens.data());
  Tensor positions = rt_.createTensor({T}, DataType::UInt32, pos.data());
  // batch projections: the tensor-core GEMM from 17 tokens up, the mat-vec below (no fusion flags: RMSNorm and the
  // gated activation are operators of their own here)
  auto mm = [&](const Tensor &a, const BlockWeight &w, MatMulFusion fusion, OperatorEnum op, const Tensor &d) {
    if (fusion == MatMulFusion::Unary) return ops.matmulBlocksUnary(op, a, w.raw, w.format, w.N);
    if (fusion == MatMulFusion::Binary) return ops.matmulBlocksBinary(op, a, w.raw, w.format, w.N, d);
    return ops.matmulBlocks(a, w.raw, w.format, w.N);
  };
  Tensor x = ops.embedding(tok, table_);  // [T, dim]
  for (uint32_t l = 0; l < cfg_.nLayers; ++l) {
    Layer &L = layers_[l];
    Tensor h = ops.rmsNorm(x, L.attnNorm, cfg_.normEps);
    Tensor att;
    if (fusedQkv_) {
      Tensor qkv = mm(h, L.wqkv, MatMulFusion::None, {}, {});  // [T, qDim + 2 kvDim]: q, k, v are its columns
      const uint32_t width = qDim + 2 * kvDim;
      ops.batchedKVCacheWrite(qkv, qkv, L.kCache, L.vCache, positions, cosT_, sinT_, T, cfg_.nKvHeads, cfg_.headDim, width, width, qDim,
                              qDim + kvDim);
      ops.barrier();
      att = ops.batchedAttentionReadCache(qkv, L.kCache, L.vCache, positions, cosT_, sinT_, T, cfg_.nHeads, cfg_.nKvHeads, cfg_.headDim,
                                          width, 0);
    } else {
      Tensor q = mm(h, L.wq, MatMulFusion::None, {}, {}), k = mm(h, L.wk, MatMulFusion::None, {}, {}),
             v = mm(h, L.wv, MatMulFusion::None, {}, {});
      ops.batchedKVCacheWrite(k, v, L.kCache, L.vCache, positions, cosT_, sinT_, T, cfg_.nKvHeads, cfg_.headDim, kvDim, kvDim, 0, 0);
      ops.barrier();
      att = ops.batchedAttentionReadCache(q, L.kCache, L.vCache, positions, cosT_, sinT_, T, cfg_.nHeads, cfg_.nKvHeads, cfg_.headDim,
                                          qDim, 0);
    }
    Tensor x1 = mm(att, L.wo, MatMulFusion::Binary, BinaryAdd, x);
    Tensor h2 = ops.rmsNorm(x1, L.ffnNorm, cfg_.normEps);
    Tensor act;
    if (L.wgu.raw) {
      // (the GEMM's own paired epilogue, kBlockFlagGluPairs, is slower at prefill sizes than this bandwidth-bound pass)
      act = ops.gluPairs(mm(h2, L.wgu, MatMulFusion::None, {}, {}), UnarySilu);
    } else {
      Tensor gate = mm(h2, L.wgate, MatMulFusion::Unary, UnarySilu, {});
      act = mm(h2, L.wup, MatMulFusion::Binary, BinaryMul, gate);
    }
    x = mm(act, L.wdown, MatMulFusion::Binary, BinaryAdd, x1);
  }
  // the last token's row through the final norm and the head
  const size_t rowBytes = (size_t)rt_.getTensor(x).innerDimPadded() * sizeof(float);
  Tensor last;
  if (((size_t)(T - 1) * rowBytes) % iface.bufferOffsetAlignment() == 0) {
    last = iface.createBufferView(x, (size_t)(T - 1) * rowBytes, {cfg_.dim}, DataType::Float32);
  } else {  // (a row that does not start on a view boundary: through the host, dim floats)
    std::vector<float> all((size_t)T * cfg_.dim);
    rt_.copyFromTensor(x, all.data(), all.size() * sizeof(float));
    last = rt_.createTensor({cfg_.dim}, DataType::Float32, all.data() + (size_t)(T - 1) * cfg_.dim);
  }
  Tensor logits = ops.matmulBlocks(ops.rmsNorm(last, finalNorm_, cfg_.normEps), lmHead_.raw, lmHead_.format, lmHead_.N);
  Tensor next = ops.reduce(ReduceArgmax, logits);
  float best = 0.f;
  rt_.copyFromTensor(next, &best, sizeof(best));  // flushes
  lastLogits_ = logits;
  return (uint32_t)best;
}

std::vector<float> LlamaRunner::logits() {
  std::vector<float> out(cfg_.vocab);
  rt_.copyFromTensor(lastLogits_, out.data(), out.size() * sizeof(float));
  return out;
}

}  // namespace cut
