"""The recorded decode step of a Llama-style decoder against a float64 composition of the CPU
checker's pieces (dequantised weights, RMSNorm, RoPE + fp16 cache write, attention), on small
geometries: logits within rel-L2 1e-3 per step with forced tokens, then greedy decoding through the
captured graph equal to the eager path token for token."""
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu

BLOCK = {0: (34, 32), 1: (18, 32), 2: (144, 256)}  # format -> (block bytes, weights per block)


def _soften(raw: np.ndarray, fmt: int) -> np.ndarray:
    """Divides the fp16 super-block scales of Q4_K by 16 (exponent arithmetic on normal halves): the
    benchmark's Q4_K distribution gives weights of magnitude ~2, which makes the softmax one-hot
    and a tolerance comparison ill-conditioned; the 32-weight formats are small already."""
    shift = 4 if fmt == 2 else 0
    if shift == 0:
        return raw
    bb, _ = BLOCK[fmt]
    blocks = raw.reshape(-1, bb).copy()
    for off in ((0, 2) if fmt == 2 else (0,)):
        h = blocks[:, off:off + 2].copy().view(np.uint16).reshape(-1)
        e = (h >> 10) & 0x1F
        h = np.where(e > shift, h - (shift << 10), 0).astype(np.uint16)
        blocks[:, off:off + 2] = h.view(np.uint8).reshape(-1, 2)
    return blocks.reshape(-1)


class Reference:
    def __init__(self, cfg, w):
        self.cfg = cfg
        deq = lambda raw, n, k: O.dequant_rows(cfg.fmt, raw, n, k).astype(np.float64)
        qkv_n = cfg.q_dim + 2 * cfg.kv_dim
        self.layers = [dict(wqkv=deq(l["wqkv"], qkv_n, cfg.hidden), wo=deq(l["wo"], cfg.hidden, cfg.q_dim),
                            wgate=deq(l["wgate"], cfg.ffn, cfg.hidden), wup=deq(l["wup"], cfg.ffn, cfg.hidden),
                            wdown=deq(l["wdown"], cfg.hidden, cfg.ffn), attn_norm=l["attn_norm"], ffn_norm=l["ffn_norm"])
                       for l in w["layers"]]
        self.final_norm, self.lm = w["final_norm"], deq(w["lm_head"], cfg.vocab, cfg.hidden)
        self.table = w["embedding"]
        from cut_b200.llama_decode import rope_tables

        self.cos_t, self.sin_t = rope_tables(cfg)
        self.kc = [np.zeros((cfg.max_seq, cfg.kv_dim), np.float16) for _ in range(cfg.n_layers)]
        self.vc = [np.zeros((cfg.max_seq, cfg.kv_dim), np.float16) for _ in range(cfg.n_layers)]

    def step(self, token, pos):
        cfg = self.cfg
        x = self.table[token].astype(np.float64)
        norm = lambda v, wt: O.rmsnorm(v.astype(np.float32), wt, cfg.eps).astype(np.float64)
        for l, lw in enumerate(self.layers):
            qkv = (lw["wqkv"] @ norm(x, lw["attn_norm"])).astype(np.float32)
            q, k, v = qkv[:cfg.q_dim], qkv[cfg.q_dim:cfg.q_dim + cfg.kv_dim], qkv[cfg.q_dim + cfg.kv_dim:]
            qr = O.rope_kv_write(q, k, v, pos, self.cos_t, self.sin_t, self.kc[l], self.vc[l], cfg.head_dim)
            a = O.attention(qr, self.kc[l], self.vc[l], pos + 1, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim).astype(np.float64)
            x = x + lw["wo"] @ a
            h = norm(x, lw["ffn_norm"])
            g = lw["wgate"] @ h
            x = x + lw["wdown"] @ ((g / (1.0 + np.exp(-g))) * (lw["wup"] @ h))
        return self.lm @ norm(x, self.final_norm)


@pytest.mark.parametrize("fuse_norm,glu,fuse_rope", [(True, True, True), (True, False, True), (False, False, False), (False, True, False)])
@pytest.mark.parametrize("fmt", [2, 0, 1])
def test_decode_steps_match_composed_checker(fmt, fuse_norm, glu, fuse_rope):
    import torch

    from cut_b200.llama_decode import LlamaConfig, LlamaDecoder, synthetic_weights

    cfg = LlamaConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=512, max_seq=32, fmt=fmt)
    w = synthetic_weights(cfg, seed=fmt + 1)
    for lw in w["layers"]:
        for k in ("wqkv", "wo", "wgate", "wup", "wdown"):
            lw[k] = _soften(lw[k], fmt)
    w["lm_head"] = _soften(w["lm_head"], fmt)
    w["embedding"] = (w["embedding"] * 50).astype(np.float32)
    dec, ref = LlamaDecoder(cfg, w, fuse_norm=fuse_norm, glu_pairs=glu, fuse_rope=fuse_rope), Reference(cfg, w)
    tokens = [3, 500, 17, 17, 0, 301, 42]
    for pos, tok in enumerate(tokens):
        got = dec.step(tok, pos).cpu().numpy().astype(np.float64)
        want = ref.step(tok, pos)
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert np.isfinite(got).all() and rel <= 1e-3, (pos, rel)
    dec.check_status()
    # the caches hold what the checker's hold (fp16, one rounding of nearly equal fp32 values)
    for l in range(cfg.n_layers):
        kc = dec.k_cache[l][: len(tokens), : cfg.kv_dim].float().cpu().numpy()
        assert np.allclose(kc, ref.kc[l][: len(tokens)].astype(np.float32), rtol=2e-3, atol=2e-3)

    # greedy continuation: eager steps against the captured graph, token for token
    pos0 = len(tokens)
    eager, tok = [], 7
    for i in range(6):
        logits = dec.step(tok, pos0 + i)
        tok = int(torch.argmax(logits).item())
        assert tok == int(dec.next_tok.item())
        eager.append(tok)
    dec.set_position(7, pos0)
    dec.capture()
    got = []
    for i in range(6):
        dec.replay(1)
        got.append(int(dec.token.item()))
    assert got == eager
    assert int(dec.params[0].item()) == pos0 + 6
    dec.check_status()
    assert dec.launches_per_step >= 3 + (0 if fuse_norm else 1) + ((7 if fuse_norm else 9) - (1 if glu else 0) - (1 if fuse_rope else 0)) * cfg.n_layers


@pytest.mark.parametrize("fmt,T", [(2, 6), (2, 40), (0, 40), (1, 23), (1, 600)])
@pytest.mark.parametrize("glu", [True, False])
def test_batched_prefill_matches_the_token_by_token_checker(fmt, T, glu):
    """The prompt as one batch (GEMM projections from 17 tokens up, batched RoPE cache write, one attention block per
    KV head and token) against the float64 composition run token by token: caches, last token's logits and the
    next decode step within 3e-3 rel-L2 (the prefill GEMM rounds activations to fp16)."""
    from cut_b200.llama_decode import LlamaConfig, LlamaDecoder, synthetic_weights

    if T > 64 and not glu:
        pytest.skip("the long prompt (attention walking more than one 512-row chunk) once is enough")
    cfg = LlamaConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=512, max_seq=max(64, T + 8), fmt=fmt)
    w = synthetic_weights(cfg, seed=fmt + 11, scale_shift=4)
    w["embedding"] = (w["embedding"] * 50).astype(np.float32)
    dec, ref = LlamaDecoder(cfg, w, glu_pairs=glu), Reference(cfg, w)
    tokens = np.random.default_rng(T).integers(0, cfg.vocab, T)
    for pos, tok in enumerate(tokens):
        want = ref.step(int(tok), pos)
    got = dec.prefill(tokens).cpu().numpy().astype(np.float64)
    dec.check_status()
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert np.isfinite(got).all() and rel <= 3e-3, rel
    for l in range(cfg.n_layers):
        kc = dec.k_cache[l][:T, : cfg.kv_dim].float().cpu().numpy()
        vc = dec.v_cache[l][:T, : cfg.kv_dim].float().cpu().numpy()
        for got_c, want_c in ((kc, ref.kc[l][:T].astype(np.float32)), (vc, ref.vc[l][:T].astype(np.float32))):
            assert np.linalg.norm(got_c - want_c) / np.linalg.norm(want_c) <= 3e-3
        assert not dec.k_cache[l][T:].any()
    assert int(dec.params[0].item()) == T and int(dec.token.item()) == int(np.argmax(got))
    nxt = int(dec.token.item())
    got2 = dec.step(nxt, T).cpu().numpy().astype(np.float64)
    want2 = ref.step(nxt, T)
    assert np.linalg.norm(got2 - want2) / np.linalg.norm(want2) <= 3e-3
    dec.check_status()


def test_position_past_the_cache_is_reported():
    from cut_b200 import _lib as L
    from cut_b200.llama_decode import LlamaConfig, LlamaDecoder, synthetic_weights

    cfg = LlamaConfig(n_layers=1, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=64, max_seq=4, fmt=0)
    dec = LlamaDecoder(cfg, synthetic_weights(cfg))
    dec.step(1, 3)
    dec.check_status()
    dec.step(1, 4)
    with pytest.raises(L.CutbError):
        dec.check_status()


@pytest.mark.parametrize("fuse_norm,glu", [(True, True), (False, False), (True, False)])
@pytest.mark.parametrize("fmt", [2, 0, 1])
def test_cpp_runner_over_a_gguf_file_matches_composed_checker(tmp_path, fmt, fuse_norm, glu):
    """The per-token step as the C++ host records it (LlamaRunner: GGUF header -> device upload with fused QKV and
    paired gate / up rows -> one reusable command buffer over the operator API, replayed per token): every step's
    logits against the float64 composition of the checker's pieces, its arg-max against the logits it returns,
    and greedy generation consistent with them."""
    from cut_b200.llama_decode import LlamaConfig, run_cpp_runner, synthetic_weights, write_model_gguf

    cfg = LlamaConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=512, max_seq=32, fmt=fmt)
    w = synthetic_weights(cfg, seed=fmt + 11)
    for lw in w["layers"]:
        for k in ("wqkv", "wo", "wgate", "wup", "wdown"):
            lw[k] = _soften(lw[k], fmt)
    w["lm_head"] = _soften(w["lm_head"], fmt)
    w["embedding"] = (w["embedding"] * 50).astype(np.float32)
    path = str(tmp_path / "model.gguf")
    write_model_gguf(path, cfg, w)
    prompt, n_gen = [3, 500, 17, 17, 0, 301, 42], 5
    out = run_cpp_runner(path, prompt, n_gen, max_seq=cfg.max_seq, fuse_norm=fuse_norm, glu_pairs=glu, want_logits=True)
    assert out["vocab"] == cfg.vocab and out["logits"].shape == (len(prompt) + n_gen, cfg.vocab)
    # separate RMSNorm launches when not fused; gate and up as two launches when not paired; RoPE and attention are two
    per_layer = 6 + (0 if fuse_norm else 2) + (0 if glu else 1)
    assert out["dispatches_per_token"] >= 3 + (0 if fuse_norm else 1) + per_layer * cfg.n_layers
    ref = Reference(cfg, w)
    feed = list(prompt)
    for step in range(len(prompt) + n_gen):
        want = ref.step(feed[step], step)
        got = out["logits"][step].astype(np.float64)
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert np.isfinite(got).all() and rel <= 1e-3, (step, rel)
        assert int(out["tokens"][step]) == int(np.argmax(out["logits"][step]))
        if step + 1 >= len(prompt):
            feed.append(int(out["tokens"][step]))  # generation continues with the runner's own greedy pick


@pytest.mark.parametrize("fmt,T", [(2, 7), (0, 40), (1, 23)])
def test_cpp_runner_batched_prefill_matches_composed_checker(tmp_path, fmt, T):
    """LlamaRunner::prefill: the prompt as one batch through the operator API (GEMM projections from 17 tokens up, the
    GluPairs operator over the paired gate / up rows, batched RoPE cache write and attention), then recorded decode
    steps that read the cache the prefill wrote: the last prompt step's logits and every generated step's against the
    float64 composition run token by token (3e-3 rel-L2: the prefill GEMM rounds its activations to fp16)."""
    from cut_b200.llama_decode import LlamaConfig, run_cpp_runner, synthetic_weights, write_model_gguf

    cfg = LlamaConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=512, max_seq=64, fmt=fmt)
    w = synthetic_weights(cfg, seed=fmt + 11, scale_shift=4)
    w["embedding"] = (w["embedding"] * 50).astype(np.float32)
    path = str(tmp_path / "model.gguf")
    write_model_gguf(path, cfg, w)
    prompt = np.random.default_rng(T).integers(0, cfg.vocab, T)
    n_gen = 4
    out = run_cpp_runner(path, prompt, n_gen, max_seq=cfg.max_seq, want_logits=True, batch_prompt=True)
    ref = Reference(cfg, w)
    for pos, tok in enumerate(prompt):
        want = ref.step(int(tok), pos)
    feed = int(out["tokens"][T - 1])
    for step in range(T - 1, T + n_gen):
        if step >= T:
            want = ref.step(feed, step)
            feed = int(out["tokens"][step])
        got = out["logits"][step].astype(np.float64)
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert np.isfinite(got).all() and rel <= 3e-3, (step, rel)
        assert int(out["tokens"][step]) == int(np.argmax(out["logits"][step]))
