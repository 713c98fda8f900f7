// C entry points over the C++ operator API, for callers that cannot link C++ (the benchmark's
// end-to-end leg drives the boundary the reference's runner would call through this).
#include <chrono>
#include <cstdio>
#include <cstring>
#include <exception>
#include <vector>

#include <stdexcept>

#include "cut_api.h"
#include "gguf_upload.h"
#include "llama_runner.h"

using namespace cut;

// One decode step per `replicas` weight tensors, as the reference's runner drives its backend
// (interface/runner/llama/llama.cpp:2045-2166, core/backends/cuda/CudaCommandBuffer.cpp:261-307): the mat-vecs are
// recorded once through Operations::matmulBlocks and kept as a reusable command buffer; every step uploads its
// activations from host memory (ComputeInterface::copyDataToBuffer), resubmits the command buffer, waits, and
// reads every result back (copyDataFromBuffer).  The weights are model state: uploaded once, before the clock starts.
//
//   format        DequantFormat code of the blocks (16 = Q8_0, 17 = Q4_0, 1 = Q4_K)
//   w_host        one weight tensor of N rows of blocks along K; replica r is its bytes rotated by r * roll_bytes
//   a_host        [replicas][batch][K] activations, fp16 when a_is_half else fp32
//   c_host        [replicas][batch][N] fp32 results of the last step
//   seconds       wall time of the `steps` timed steps
// Returns 0, or -1 with a message in err.
extern "C" __attribute__((visibility("default"))) int cut_host_e2e_matvec_blocks(
    int device, uint32_t format, uint32_t N, uint32_t K, uint32_t batch, uint32_t replicas, const uint8_t *w_host, uint64_t w_bytes,
    uint64_t roll_bytes, const void *a_host, int a_is_half, float *c_host, uint32_t warmup, uint32_t steps, double *seconds,
    uint64_t *h2d_bytes_per_step, uint64_t *d2h_bytes_per_step, char *err, size_t err_cap) {
  try {
    Runtime rt(device);
    const DataType adt = a_is_half ? DataType::Float16 : DataType::Float32;
    const size_t a_bytes = (size_t)batch * K * (a_is_half ? 2 : 4), c_bytes = (size_t)batch * N * sizeof(float);
    std::vector<Tensor> tA(replicas), tW(replicas), tC(replicas);
    std::vector<uint8_t> rolled(w_bytes);
    for (uint32_t r = 0; r < replicas; ++r) {
      const uint64_t sh = w_bytes ? (roll_bytes * r) % w_bytes : 0;
      std::memcpy(rolled.data() + sh, w_host, w_bytes - sh);
      std::memcpy(rolled.data(), w_host + (w_bytes - sh), sh);
      tW[r] = rt.createTensor({(uint32_t)w_bytes}, DataType::Int8, rolled.data());
      tA[r] = batch == 1 ? rt.createTensor({K}, adt, (const uint8_t *)a_host + r * a_bytes)
                         : rt.createTensor({batch, K}, adt, (const uint8_t *)a_host + r * a_bytes);
    }
    for (uint32_t r = 0; r < replicas; ++r) tC[r] = rt.ops().matmulBlocks(tA[r], tW[r], static_cast<DequantFormat>(format), N);
    ComputeHandle cb = rt.iface().submitReusable();
    rt.iface().wait(cb);
    auto step = [&]() {
      for (uint32_t r = 0; r < replicas; ++r) rt.copyToTensor(tA[r], (const uint8_t *)a_host + r * a_bytes, a_bytes);
      rt.iface().resubmit(cb);
      rt.iface().wait(cb);
      for (uint32_t r = 0; r < replicas; ++r) rt.copyFromTensor(tC[r], (uint8_t *)c_host + r * c_bytes, c_bytes);
    };
    for (uint32_t i = 0; i < warmup; ++i) step();
    const auto t0 = std::chrono::steady_clock::now();
    for (uint32_t i = 0; i < steps; ++i) step();
    const auto t1 = std::chrono::steady_clock::now();
    if (seconds) *seconds = std::chrono::duration<double>(t1 - t0).count();
    if (h2d_bytes_per_step) *h2d_bytes_per_step = (uint64_t)replicas * a_bytes;
    if (d2h_bytes_per_step) *d2h_bytes_per_step = (uint64_t)replicas * c_bytes;
    return 0;
  } catch (const std::exception &e) {
    if (err && err_cap) snprintf(err, err_cap, "%s", e.what());
    return -1;
  }
}

// Greedy decoding of a llama-style GGUF model through LlamaRunner (llama_runner.h): the prompt is fed one token
// per step (positions 0, 1, ...), then `n_generate` tokens are generated from the arg-max of each step.
//
//   option_bits   1 fused RMSNorms, 2 paired gate / up rows, 4 activations staged at 16 bits, 8 fp16 KV cache,
//                 16 the prompt as ONE batch (LlamaRunner::prefill) instead of token by token: then only the last
//                 prompt step's arg-max and logits exist (tokens_out / logits_out entries before it stay zero)
//   tokens_out    [n_prompt + n_generate] the arg-max after every step (tokens_out[i] is what follows step i)
//   logits_out    null, or [n_prompt + n_generate][vocab] the logits of every step
//   seconds       wall time of the generation steps only (the prompt steps are warm-up)
// Returns 0, or -1 with a message in err.
extern "C" __attribute__((visibility("default"))) int cut_host_llama_generate(
    int device, const char *gguf_path, uint32_t max_seq, uint32_t option_bits, const uint32_t *prompt, uint32_t n_prompt,
    uint32_t n_generate, uint32_t *tokens_out, float *logits_out, uint32_t *vocab_out, double *seconds, uint64_t *weight_bytes_per_token,
    uint32_t *dispatches_per_token, char *err, size_t err_cap) {
  try {
    if (!gguf_path || !prompt || n_prompt == 0 || !tokens_out) throw std::runtime_error("llama_generate: null argument or empty prompt");
    Runtime rt(device);
    GGUFFile file(gguf_path);
    LlamaRunnerOptions opt;
    opt.maxSeq = max_seq;
    opt.fuseNorm = (option_bits & 1u) != 0;
    opt.gluPairs = (option_bits & 2u) != 0;
    opt.act16 = (option_bits & 4u) != 0;
    opt.kvHalf = (option_bits & 8u) != 0;
    LlamaRunner runner(rt, file, opt);
    const uint32_t vocab = runner.config().vocab;
    if (vocab_out) *vocab_out = vocab;
    if (weight_bytes_per_token) *weight_bytes_per_token = runner.weightBytesPerToken();
    if (dispatches_per_token) *dispatches_per_token = (uint32_t)runner.dispatchesPerToken();
    uint32_t pos = 0, next = 0;
    auto keep = [&](uint32_t step) {
      tokens_out[step] = next;
      if (logits_out) {
        const std::vector<float> l = runner.logits();
        std::memcpy(logits_out + (size_t)step * vocab, l.data(), (size_t)vocab * sizeof(float));
      }
    };
    if (option_bits & 16u) {
      next = runner.prefill(std::vector<uint32_t>(prompt, prompt + n_prompt), 0);
      pos = n_prompt;
      keep(n_prompt - 1);
    } else {
      for (uint32_t i = 0; i < n_prompt; ++i, ++pos) {
        next = runner.forward(prompt[i], pos);
        keep(i);
      }
    }
    const auto t0 = std::chrono::steady_clock::now();
    for (uint32_t i = 0; i < n_generate; ++i, ++pos) {
      next = runner.forward(next, pos);
      keep(n_prompt + i);
    }
    const auto t1 = std::chrono::steady_clock::now();
    if (seconds) *seconds = std::chrono::duration<double>(t1 - t0).count();
    return 0;
  } catch (const std::exception &e) {
    if (err && err_cap) snprintf(err, err_cap, "%s", e.what());
    return -1;
  }
}
