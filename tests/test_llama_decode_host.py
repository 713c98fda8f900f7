"""CPU checks of the decoder's host side: synthetic weight layout, the scale softening, the RoPE tables and
the refusal to run without a device (there is no CPU path)."""
import numpy as np
import pytest

from cut_b200 import synth
from cut_b200.llama_decode import LlamaConfig, LlamaDecoder, rope_tables, soften_scales, synthetic_weights
from oracle import oracle as O


def test_soften_scales_divides_q4k_values_exactly():
    raw = synth.make_weights(synth.Q4_K, 8, 512, seed=3)
    soft = soften_scales(raw, synth.Q4_K, 4)
    a, b = O.dequant_rows(synth.Q4_K, raw, 8, 512), O.dequant_rows(synth.Q4_K, soft, 8, 512)
    blocks = raw.reshape(-1, 144)
    d = blocks[:, 0:2].copy().view(np.uint16).reshape(-1)
    dm = blocks[:, 2:4].copy().view(np.uint16).reshape(-1)
    keep = (((d >> 10) & 0x1F) > 4) & (((dm >> 10) & 0x1F) > 4)  # both scales stay normal halves: an exact division by 16
    rows = np.repeat(keep.reshape(8, 2), 256, axis=1)
    assert keep.any() and np.array_equal(b[rows], (a[rows] / 16).astype(np.float32))
    assert soften_scales(raw, synth.Q4_K, 0) is raw
    q8 = synth.make_weights(synth.Q8_0, 4, 64, seed=1)
    assert soften_scales(q8, synth.Q8_0, 4) is q8


def test_synthetic_weights_shapes_and_row_rotation():
    cfg = LlamaConfig(n_layers=3, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=128, max_seq=16, fmt=synth.Q4_0)
    w = synthetic_weights(cfg, seed=5, distinct_layers=False)
    rb = synth.row_bytes(cfg.fmt, cfg.hidden)
    assert w["layers"][0]["wqkv"].size == (cfg.q_dim + 2 * cfg.kv_dim) * rb and w["lm_head"].size == cfg.vocab * rb
    l0, l2 = w["layers"][0]["wgate"].reshape(cfg.ffn, rb), w["layers"][2]["wgate"].reshape(cfg.ffn, rb)
    assert np.array_equal(np.roll(l0, 32, axis=0), l2) and not np.array_equal(l0, l2)
    assert w["embedding"].shape == (cfg.vocab, cfg.hidden) and w["final_norm"].shape == (cfg.hidden,)


def test_rope_tables_follow_the_runner():
    cfg = LlamaConfig(head_dim=8, max_seq=5, rope_theta=10000.0)
    cos_t, sin_t = rope_tables(cfg)
    assert cos_t.shape == (5, 4) and cos_t.dtype == np.float32
    for pos in range(5):
        for i in range(4):
            freq = np.float32(1.0) / np.float32(np.power(np.float32(10000.0), np.float32(2 * i) / np.float32(8)))
            ang = np.float32(pos) * freq
            assert abs(cos_t[pos, i] - np.cos(ang)) <= 1e-6 and abs(sin_t[pos, i] - np.sin(ang)) <= 1e-6


def test_decoder_needs_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    cfg = LlamaConfig(n_layers=1, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=64, max_seq=4, fmt=synth.Q8_0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        LlamaDecoder(cfg, synthetic_weights(cfg))
