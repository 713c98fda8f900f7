"""One-token decode step of a Llama-style decoder over raw GGUF-block weights, on the C ABI.

The per-token dispatch sequence of the reference's runner (interface/runner/llama/llama.cpp:
runLayer 2045-2084, forward 2090-2166): embedding gather, then per layer RMSNorm -> fused QKV
mat-vec -> fused RoPE + KV-cache write -> grouped-query attention -> output projection with the
residual add fused -> RMSNorm -> gate mat-vec with SiLU fused -> up mat-vec with the multiply
fused -> down projection with the residual add fused; final RMSNorm, LM head, arg-max.  Position
and token live in device buffers ({pos, seqLen} as in the reference's runtimeParams), the whole
step is recorded once into a CUDA graph and replayed per token; the arg-max feeds the next
token on the device, so a decode loop makes no host round trip.

torch supplies device memory, the stream and the graph capture; every kernel of the step is this
package's.  Weights are raw GGUF blocks ([N rows][K / block] of Q8_0, Q4_0 or Q4_K), Q/K/V
concatenated along N, exactly as a GGUF file stores them.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib as L
from . import ops, synth

UNARY_SILU, BINARY_ADD, BINARY_MUL = 133, 0, 2  # OperatorEnum codes (operators/runtime/ComputeOpsShared.h)


@dataclass
class LlamaConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 32000
    eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq: int = 2048
    fmt: int = L.Q4_K
    kv_dtype: torch.dtype = torch.float16

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim


def rope_tables(cfg: LlamaConfig):
    """cos / sin [max_seq, head_dim / 2] in float32 arithmetic (llama.cpp:1652-1666)."""
    half = cfg.head_dim // 2
    freq = (np.float32(1.0) / np.power(np.float32(cfg.rope_theta), (2 * np.arange(half, dtype=np.float32)) / np.float32(cfg.head_dim)))
    ang = np.arange(cfg.max_seq, dtype=np.float32)[:, None] * freq.astype(np.float32)[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def soften_scales(raw: np.ndarray, fmt: int, shift: int = 4) -> np.ndarray:
    """Divides the fp16 super-block scales (d, dmin) of Q4_K blocks by 2^shift (exponent arithmetic on normal halves; smaller
    ones become zero).  The benchmark's Q4_K distribution gives weights of magnitude ~2, hence activations far beyond what
    a trained model produces (and beyond fp16, which the prefill GEMM rounds its activations to); the 32-weight formats'
    distributions are small already and are returned unchanged."""
    if fmt != L.Q4_K or shift == 0:
        return raw
    blocks = raw.reshape(-1, 144).copy()
    for off in (0, 2):
        h = blocks[:, off:off + 2].copy().view(np.uint16).reshape(-1)
        e = (h >> 10) & 0x1F
        h = np.where(e > shift, h - (shift << 10), 0).astype(np.uint16)
        blocks[:, off:off + 2] = h.view(np.uint8).reshape(-1, 2)
    return blocks.reshape(-1)


def synthetic_weights(cfg: LlamaConfig, seed: int = 0, distinct_layers: bool = True, scale_shift: int = 0) -> dict:
    """Random-init weights as host arrays: block tensors from the synthetic generators of the
    benchmark configurations, norms near 1, an fp32 embedding table ~N(0, 0.02).  With
    distinct_layers False, layer 0 is generated and the others are row rotations of it (different
    matrices at different addresses for a fraction of the generation time)."""
    rng = np.random.default_rng(seed)
    shapes = {"wqkv": (cfg.q_dim + 2 * cfg.kv_dim, cfg.hidden), "wo": (cfg.hidden, cfg.q_dim), "wgate": (cfg.ffn, cfg.hidden),
              "wup": (cfg.ffn, cfg.hidden), "wdown": (cfg.hidden, cfg.ffn)}
    layers = []
    for l in range(cfg.n_layers):
        if l == 0 or distinct_layers:
            lw = {k: soften_scales(synth.make_weights(cfg.fmt, n, kk, seed=seed * 1000 + l * 10 + i), cfg.fmt, scale_shift)
                  for i, (k, (n, kk)) in enumerate(shapes.items())}
        else:
            lw = {}
            for k, (n, kk) in shapes.items():
                rb = synth.row_bytes(cfg.fmt, kk)
                lw[k] = np.roll(layers[0][k].reshape(n, rb), 16 * l, axis=0).reshape(-1)
        lw["attn_norm"] = (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32)
        lw["ffn_norm"] = (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32)
        layers.append(lw)
    return {"layers": layers, "final_norm": (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32),
            "lm_head": soften_scales(synth.make_weights(cfg.fmt, cfg.vocab, cfg.hidden, seed=seed * 1000 + 999), cfg.fmt, scale_shift),
            "embedding": (0.02 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(np.float32)}


class LlamaDecoder:
    """Device state of one model and the recorded decode step.

    `step(token, pos)` runs one token eagerly; `capture()` records the step once and `replay(n)`
    runs n further tokens from the device-resident {token, pos}, greedy (arg-max feeds back)."""

    def __init__(self, cfg: LlamaConfig, weights: dict, device: torch.device | str = "cuda", act_16bit: bool = True,
                 overlap=("qkv", "gate", "up"), fuse_norm: bool = True, glu_pairs: bool = True,
                 fuse_rope: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("LlamaDecoder needs a CUDA device: there is no CPU path")
        if cfg.hidden % 4 or cfg.n_heads % cfg.n_kv_heads:
            raise ValueError("hidden must be a multiple of 4 and n_heads a multiple of n_kv_heads")
        self.cfg, self.dev = cfg, torch.device(device)
        up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.dev)
        self.glu = glu_pairs
        self.layers = []
        for lw in weights["layers"]:
            dl = {k: up(v) for k, v in lw.items() if not (glu_pairs and k in ("wgate", "wup"))}
            if glu_pairs:  # gate row i and up row i side by side: one launch computes silu(gate) * up
                rb = synth.row_bytes(cfg.fmt, cfg.hidden)
                dl["wgu"] = up(np.stack([lw["wgate"].reshape(cfg.ffn, rb), lw["wup"].reshape(cfg.ffn, rb)], axis=1).reshape(-1))
            self.layers.append(dl)
        self.final_norm, self.lm_head, self.table = up(weights["final_norm"]), up(weights["lm_head"]), up(weights["embedding"])
        cos_t, sin_t = rope_tables(cfg)
        self.cos_t, self.sin_t = up(cos_t), up(sin_t)
        ld = (cfg.kv_dim + 3) // 4 * 4
        self.k_cache = [torch.zeros((cfg.max_seq, ld), dtype=cfg.kv_dtype, device=self.dev) for _ in range(cfg.n_layers)]
        self.v_cache = [torch.zeros((cfg.max_seq, ld), dtype=cfg.kv_dtype, device=self.dev) for _ in range(cfg.n_layers)]
        f32 = lambda n: torch.zeros(n, dtype=torch.float32, device=self.dev)
        self.params = torch.zeros(2, dtype=torch.int32, device=self.dev)  # {pos, seqLen}
        self.token = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.x = [f32(cfg.hidden), f32(cfg.hidden)]
        self.h, self.qkv, self.q_roped, self.attn = f32(cfg.hidden), f32(cfg.q_dim + 2 * cfg.kv_dim), f32(cfg.q_dim), f32(cfg.q_dim)
        self.gate, self.act, self.logits, self.next_tok = f32(cfg.ffn), f32(cfg.ffn), f32(cfg.vocab), f32(1)
        self.attn_ws = ops.attention_workspace(cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.max_seq, self.dev)
        # fp32 activations staged at one 16-bit level per 32-k block: fp16-grade error, fp32 range
        self.act_flags = L.FLAG_ACT_16BIT if act_16bit else 0
        # overlap: which mat-vecs that directly follow a mat-vec may prefetch under their predecessor's tail (True: all).
        # Measured on the 32-layer step: qkv (after down), gate and up each gain, together +3.6 %; down loses 9 %, and the
        # output projection started under the attention kernel (which holds 64 SMs) loses 15 %: its 148 persistent
        # CTAs double up on the free SMs.
        self.overlap = overlap
        # fuse_norm: the RMSNorms run inside the projections that consume them (no launch, no round trip of h)
        self.fuse_norm = fuse_norm
        # fuse_rope: RoPE + KV-cache write inside the attention launch
        self.fuse_rope = fuse_rope
        self._keep, self._descs, self.launches_per_step = [], [], 0
        self._plan()
        self.graph = None

    # -- the recorded sequence: a list of closures over prepared descriptors --------------------
    def _matvec(self, A, W, N, out, fusion_type=L.FUSION_NONE, fusion_op=0, D=None, after_matvec=False, norm=None, glu=False):
        d, _, keep = ops.make_desc(A, W, self.cfg.fmt, N, C_out=out.view(1, -1), D=D.view(1, -1) if D is not None else None,
                                   fusion_type=fusion_type, fusion_op=fusion_op, status=self.status,
                                   flags=self.act_flags | (0 if (after_matvec and self._overlaps(after_matvec)) else L.FLAG_NO_OVERLAP))
        if glu:
            d.flags |= L.FLAG_GLU_PAIRS
        if norm is not None:  # the RMSNorm in front of this projection, applied while the mat-vec stages its activations
            d.flags |= L.FLAG_A_RMSNORM
            d.a_norm_weight, d.a_norm_eps = norm.data_ptr(), self.cfg.eps
            keep = keep + (norm,)
        need = ops.workspace_bytes(d)
        if need and glu:
            raise RuntimeError("glu_pairs needs gate/up shapes that do not split K: construct the decoder with glu_pairs=False")
        if need:  # split-K shapes: scratch owned by this descriptor, sized before capture
            ws = torch.empty(need, dtype=torch.uint8, device=self.dev)
            d.workspace, d.workspace_bytes = ws.data_ptr(), need
            keep = keep + (ws,)
        self._keep.append(keep)
        self._descs.append(d)
        return lambda d=d: L.check(L.lib().cutb_qmatmul(C.byref(d), ops._stream_ptr()))

    def _overlaps(self, name) -> bool:
        return bool(self.overlap) if isinstance(self.overlap, bool) else name in self.overlap

    def _plan(self):
        cfg, lib = self.cfg, L.lib()
        seq = []
        fuse = self.fuse_norm
        st = self.status.data_ptr()
        kvd = L.F16 if cfg.kv_dtype == torch.float16 else L.F32

        def rms(x, w, y):
            return lambda: L.check(lib.cutb_rmsnorm(L.F32, x.data_ptr(), w.data_ptr(), y.data_ptr(), 1, cfg.hidden, cfg.hidden, cfg.eps,
                                                    ops._stream_ptr()))

        seq.append(lambda: L.check(lib.cutb_embedding(self.token.data_ptr(), self.table.data_ptr(), self.x[0].data_ptr(), 1, cfg.hidden,
                                                      cfg.vocab, st, ops._stream_ptr())))
        q, k, v = self.qkv[: cfg.q_dim], self.qkv[cfg.q_dim: cfg.q_dim + cfg.kv_dim], self.qkv[cfg.q_dim + cfg.kv_dim:]
        scale = 1.0 / float(np.sqrt(np.float32(cfg.head_dim)))
        for l, lw in enumerate(self.layers):
            kc, vc = self.k_cache[l], self.v_cache[l]
            if fuse:
                seq.append(self._matvec(self.x[0], lw["wqkv"], cfg.q_dim + 2 * cfg.kv_dim, self.qkv, norm=lw["attn_norm"], after_matvec="qkv" if l else False))
            else:
                seq.append(rms(self.x[0], lw["attn_norm"], self.h))
                seq.append(self._matvec(self.h, lw["wqkv"], cfg.q_dim + 2 * cfg.kv_dim, self.qkv))
            if self.fuse_rope:
                seq.append(lambda kc=kc, vc=vc: L.check(lib.cutb_rope_attention_decode(
                    kvd, q.data_ptr(), k.data_ptr(), v.data_ptr(), self.params.data_ptr(), self.cos_t.data_ptr(), self.sin_t.data_ptr(),
                    kc.data_ptr(), vc.data_ptr(), self.attn.data_ptr(), cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, kc.stride(0),
                    cfg.max_seq, scale, self.attn_ws.data_ptr(), self.attn_ws.numel(), st, ops._stream_ptr())))
            else:
                seq.append(lambda kc=kc, vc=vc: L.check(lib.cutb_rope_kv_write(
                    kvd, q.data_ptr(), k.data_ptr(), v.data_ptr(), self.params.data_ptr(), self.cos_t.data_ptr(), self.sin_t.data_ptr(),
                    kc.data_ptr(), vc.data_ptr(), self.q_roped.data_ptr(), cfg.q_dim, cfg.kv_dim, cfg.head_dim, kc.stride(0), cfg.max_seq, st,
                    ops._stream_ptr())))
                seq.append(lambda kc=kc, vc=vc: L.check(lib.cutb_attention_decode(
                    kvd, self.q_roped.data_ptr(), kc.data_ptr(), vc.data_ptr(), self.params.data_ptr(), self.attn.data_ptr(), cfg.n_heads,
                    cfg.n_kv_heads, cfg.head_dim, kc.stride(0), cfg.max_seq, scale, self.attn_ws.data_ptr(), self.attn_ws.numel(), st,
                    ops._stream_ptr())))
            seq.append(self._matvec(self.attn, lw["wo"], cfg.hidden, self.x[1], L.FUSION_BINARY, BINARY_ADD, self.x[0]))
            ffn_in, ffn_norm = (self.x[1], lw["ffn_norm"]) if fuse else (self.h, None)
            if not fuse:
                seq.append(rms(self.x[1], lw["ffn_norm"], self.h))
            if self.glu:
                seq.append(self._matvec(ffn_in, lw["wgu"], 2 * cfg.ffn, self.act, L.FUSION_UNARY, UNARY_SILU, norm=ffn_norm,
                                        after_matvec="gate" if fuse else False, glu=True))
            else:
                seq.append(self._matvec(ffn_in, lw["wgate"], cfg.ffn, self.gate, L.FUSION_UNARY, UNARY_SILU, norm=ffn_norm,
                                        after_matvec="gate" if fuse else False))
                seq.append(self._matvec(ffn_in, lw["wup"], cfg.ffn, self.act, L.FUSION_BINARY, BINARY_MUL, self.gate, after_matvec="up",
                                        norm=ffn_norm))
            seq.append(self._matvec(self.act, lw["wdown"], cfg.hidden, self.x[0], L.FUSION_BINARY, BINARY_ADD, self.x[1], after_matvec="down"))
        if fuse:
            seq.append(self._matvec(self.x[0], self.lm_head, cfg.vocab, self.logits, norm=self.final_norm))
        else:
            seq.append(rms(self.x[0], self.final_norm, self.h))
            seq.append(self._matvec(self.h, self.lm_head, cfg.vocab, self.logits))
        seq.append(lambda: L.check(lib.cutb_argreduce(1, self.logits.data_ptr(), self.next_tok.data_ptr(), cfg.vocab, ops._stream_ptr())))
        self._seq = seq
        # split-K mat-vecs launch a second (reduction) kernel
        self.launches_per_step = len(seq) + sum(1 for d in self._descs if d.workspace_bytes)

    def weight_bytes_per_token(self) -> int:
        """Bytes of block weights one token streams (every projection once, plus the LM head)."""
        return sum(t.numel() for lw in self.layers for k, t in lw.items() if k.startswith("w")) + self.lm_head.numel()

    def set_position(self, token: int, pos: int) -> None:
        self.token.fill_(token)
        self.params.copy_(torch.tensor([pos, pos + 1], dtype=torch.int32))

    def _run(self) -> None:
        for f in self._seq:
            f()

    def _advance(self) -> None:
        # plumbing between tokens: the greedy pick becomes the next token, the position moves on
        self.token.copy_(self.next_tok.to(torch.int32))
        self.params.add_(1)

    def step(self, token: int, pos: int) -> torch.Tensor:
        """One token eagerly; returns the logits (device tensor, overwritten by the next step)."""
        self.set_position(token, pos)
        self._run()
        return self.logits

    def prompt(self, tokens, start: int = 0) -> torch.Tensor:
        """Feeds a prompt through the decode step, one token per step (positions start, start + 1, ...), so the
        KV cache holds what the model computes for it; returns the last step's logits.  (There is no batched
        prefill attention yet: this is the sequential way to the same cache contents.)"""
        logits = self.logits
        for i, t in enumerate(tokens):
            logits = self.step(int(t), start + i)
        return logits

    def prefill(self, tokens, start: int = 0) -> torch.Tensor:
        """The prompt as one batch (interface/runner/llama/llama.cpp prefillBatched): every projection is one matmul over
        all T tokens (the tensor-core GEMM from 17 tokens up), K / V rows go to the cache through the batched RoPE
        write and every token attends over the rows up to its own (in chunks of 512 rows: start + T <= max_seq).  Leaves the cache as T decode steps would (up to rounding) and returns the last
        token's logits; the greedy pick is in next_tok."""
        cfg, dev = self.cfg, self.dev
        T = len(tokens)
        if T == 0 or start + T > cfg.max_seq:
            raise ValueError("prefill: 1 .. max_seq - start tokens per call")
        tok = torch.as_tensor(np.asarray(tokens, dtype=np.int32)).to(dev)
        pos = torch.arange(start, start + T, dtype=torch.int32, device=dev)
        q_dim, kv_dim = cfg.q_dim, cfg.kv_dim
        mm = lambda A, W, N, **kw: ops.qmatmul(A, W, cfg.fmt, N, status=self.status, flags=self.act_flags | L.FLAG_NO_OVERLAP, **kw)
        x = ops.embedding(tok, self.table, status=self.status)
        for l, lw in enumerate(self.layers):
            h = ops.rmsnorm(x, lw["attn_norm"], cfg.eps)
            qkv = mm(h, lw["wqkv"], q_dim + 2 * kv_dim)
            ops.batched_kv_write(qkv[:, q_dim: q_dim + kv_dim], qkv[:, q_dim + kv_dim:], pos, self.cos_t, self.sin_t, self.k_cache[l],
                                 self.v_cache[l], cfg.head_dim, status=self.status)
            att = ops.batched_attention(qkv[:, :q_dim], self.k_cache[l], self.v_cache[l], pos, self.cos_t, self.sin_t, cfg.n_heads,
                                        cfg.n_kv_heads, cfg.head_dim, status=self.status)
            x = mm(att, lw["wo"], cfg.hidden, D=x, fusion_type=L.FUSION_BINARY, fusion_op=BINARY_ADD)
            h = ops.rmsnorm(x, lw["ffn_norm"], cfg.eps)
            if self.glu:
                # (the GEMM has the paired epilogue too, CUTB_FLAG_GLU_PAIRS, but at prefill sizes its serial epilogue
                # costs more than this bandwidth-bound pass: 512 tokens 16.3 against 15.0 ms for the whole prefill)
                act = ops.glu_pairs(mm(h, lw["wgu"], 2 * cfg.ffn), UNARY_SILU)
            else:
                gate = mm(h, lw["wgate"], cfg.ffn, fusion_type=L.FUSION_UNARY, fusion_op=UNARY_SILU)
                act = mm(h, lw["wup"], cfg.ffn, D=gate, fusion_type=L.FUSION_BINARY, fusion_op=BINARY_MUL)
            x = mm(act, lw["wdown"], cfg.hidden, D=x, fusion_type=L.FUSION_BINARY, fusion_op=BINARY_ADD)
        self.x[0].copy_(x[T - 1])
        for f in self._seq[-2 if self.fuse_norm else -3:]:  # final norm, LM head, arg-max of the decode step
            f()
        self.token.copy_(self.next_tok.to(torch.int32))  # decoding continues at position start + T with the greedy pick
        self.params.copy_(torch.tensor([start + T, start + T + 1], dtype=torch.int32))
        return self.logits

    def capture(self) -> None:
        """Records step + advance into one CUDA graph (call after at least one eager step)."""
        torch.cuda.synchronize(self.dev)
        saved = (self.token.clone(), self.params.clone())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._run()
            self._advance()
        self.token.copy_(saved[0])
        self.params.copy_(saved[1])
        self.graph = g

    def replay(self, n: int) -> None:
        if self.graph is None:
            raise RuntimeError("capture() first")
        for _ in range(n):
            self.graph.replay()

    def check_status(self) -> None:
        st = int(self.status.item())
        if st:
            raise L.CutbError(st, "a kernel of the decode step reported an error (position past the cache, token past the "
                                  "vocabulary, or an expired bounded wait)")


# ---- the same model as a GGUF file, and the C++ runner over it ------------------------------------------------------
_GGML_NAME = {L.Q8_0: "Q8_0", L.Q4_0: "Q4_0", L.Q4_K: "Q4_K"}


def write_model_gguf(path: str, cfg: LlamaConfig, weights: dict) -> None:
    """Writes `weights` (the dict of synthetic_weights) as a llama-architecture GGUF v3 file with the tensor names and
    metadata keys the reference's runner reads (interface/runner/llama/llama.cpp:1084-1118, 831-866): Q / K / V as
    three tensors (rows of the fused matrix), norms and the embedding table F32, block weights as raw blocks."""
    from .gguf_write import write_gguf

    t = _GGML_NAME[cfg.fmt]
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32).view(np.uint8).reshape(-1)
    tensors = [("token_embd.weight", "F32", (cfg.vocab, cfg.hidden), f32(weights["embedding"])),
               ("output_norm.weight", "F32", (cfg.hidden,), f32(weights["final_norm"])),
               ("output.weight", t, (cfg.vocab, cfg.hidden), weights["lm_head"])]
    rb = synth.row_bytes(cfg.fmt, cfg.hidden)
    for l, lw in enumerate(weights["layers"]):
        b = f"blk.{l}."
        qkv = lw["wqkv"].reshape(cfg.q_dim + 2 * cfg.kv_dim, rb)
        tensors += [(b + "attn_norm.weight", "F32", (cfg.hidden,), f32(lw["attn_norm"])),
                    (b + "attn_q.weight", t, (cfg.q_dim, cfg.hidden), qkv[: cfg.q_dim].reshape(-1)),
                    (b + "attn_k.weight", t, (cfg.kv_dim, cfg.hidden), qkv[cfg.q_dim: cfg.q_dim + cfg.kv_dim].reshape(-1)),
                    (b + "attn_v.weight", t, (cfg.kv_dim, cfg.hidden), qkv[cfg.q_dim + cfg.kv_dim:].reshape(-1)),
                    (b + "attn_output.weight", t, (cfg.hidden, cfg.q_dim), lw["wo"]),
                    (b + "ffn_norm.weight", "F32", (cfg.hidden,), f32(lw["ffn_norm"])),
                    (b + "ffn_gate.weight", t, (cfg.ffn, cfg.hidden), lw["wgate"]),
                    (b + "ffn_up.weight", t, (cfg.ffn, cfg.hidden), lw["wup"]),
                    (b + "ffn_down.weight", t, (cfg.hidden, cfg.ffn), lw["wdown"])]
    meta = {"general.architecture": "llama", "llama.embedding_length": cfg.hidden, "llama.block_count": cfg.n_layers,
            "llama.attention.head_count": cfg.n_heads, "llama.attention.head_count_kv": cfg.n_kv_heads,
            "llama.attention.key_length": cfg.head_dim, "llama.feed_forward_length": cfg.ffn, "llama.context_length": cfg.max_seq,
            "llama.rope.freq_base": float(cfg.rope_theta), "llama.attention.layer_norm_rms_epsilon": float(cfg.eps)}
    write_gguf(path, meta, tensors)


def run_cpp_runner(path: str, prompt, n_generate: int, *, device: int = 0, max_seq: int = 512, fuse_norm: bool = True,
                   glu_pairs: bool = True, act_16bit: bool = True, kv_half: bool = True, want_logits: bool = False,
                   batch_prompt: bool = False) -> dict:
    """Greedy decoding through the C++ LlamaRunner of libcut_host.so (Runtime -> GGUFFile -> GGUFUploader -> the recorded
    per-token command buffer): the prompt token by token, then n_generate tokens.  Returns the arg-max after every step,
    optionally every step's logits, the seconds spent on the generation steps and the runner's own counts.  With
    batch_prompt the prompt runs as one batch (LlamaRunner::prefill); only its last step's entries are filled then."""
    from . import build

    lib = C.CDLL(build.build_host())
    fn = lib.cut_host_llama_generate
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.c_char_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p, C.c_size_t]
    prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
    steps = len(prompt) + n_generate
    toks = np.zeros(steps, dtype=np.uint32)
    vocab, disp = C.c_uint32(0), C.c_uint32(0)
    secs, wbytes = C.c_double(0.0), C.c_uint64(0)
    err = C.create_string_buffer(512)
    bits = (1 if fuse_norm else 0) | (2 if glu_pairs else 0) | (4 if act_16bit else 0) | (8 if kv_half else 0) | (16 if batch_prompt else 0)
    logits = None
    if want_logits:
        # the vocabulary is in the file: token_embd's outer dimension; a first call without logits reports it
        if fn(device, path.encode(), max_seq, bits, prompt.ctypes.data, 1, 0, toks.ctypes.data, None, C.byref(vocab), None, None, None,
              err, len(err)) != 0:
            raise RuntimeError(f"cut_host_llama_generate: {err.value.decode()}")
        logits = np.zeros((steps, vocab.value), dtype=np.float32)
    rc = fn(device, path.encode(), max_seq, bits, prompt.ctypes.data, len(prompt), n_generate, toks.ctypes.data,
            logits.ctypes.data if logits is not None else None, C.byref(vocab), C.byref(secs), C.byref(wbytes), C.byref(disp), err, len(err))
    if rc != 0:
        raise RuntimeError(f"cut_host_llama_generate: {err.value.decode()}")
    return {"tokens": toks, "logits": logits, "seconds": secs.value, "weight_bytes_per_token": wbytes.value,
            "dispatches_per_token": disp.value, "vocab": vocab.value}
