"""CPU checks of the attention checker itself: the RoPE + cache-write restatement against the
formula in numpy, the attention restatement against a float64 softmax, and its half conversion
against numpy's round-to-nearest-even."""
import numpy as np

from oracle import oracle as O


def test_f16_rne_matches_numpy():
    rng = np.random.default_rng(0)
    halves = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32).view(np.uint32)
    bits = np.concatenate([rng.integers(0, 2**32, 20000, dtype=np.uint64).astype(np.uint32), halves[::17], halves[::17] + 0x1000,
                           halves[::17] + 0x0FFF, halves[::17] + 0x1001])
    vals = bits.view(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    for x, w in zip(vals, want):
        if not np.isnan(x):
            assert O.f32_to_f16_rne(float(x)) == int(w)


def test_rope_kv_write_restatement():
    rng = np.random.default_rng(1)
    n_heads, n_kv, hd, max_seq, pos = 4, 2, 8, 16, 5
    half = hd // 2
    q = rng.uniform(-1, 1, n_heads * hd).astype(np.float32)
    k = rng.uniform(-1, 1, n_kv * hd).astype(np.float32)
    v = rng.uniform(-1, 1, n_kv * hd).astype(np.float32)
    ang = (np.arange(max_seq, dtype=np.float32)[:, None] / np.power(np.float32(10000.0), 2 * np.arange(half, dtype=np.float32) / hd))
    cos_t, sin_t = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)

    def rope(x):
        x = x.reshape(-1, hd)
        a, b = x[:, :half], x[:, half:]
        c, s = cos_t[pos], sin_t[pos]
        return np.concatenate([a * c - b * s, a * s + b * c], axis=1).reshape(-1).astype(np.float32)

    for dt in (np.float32, np.float16):
        kc = np.zeros((max_seq, n_kv * hd), dt)
        vc = np.zeros((max_seq, n_kv * hd), dt)
        q_out = O.rope_kv_write(q, k, v, pos, cos_t, sin_t, kc, vc, hd)
        assert np.array_equal(q_out, rope(q))
        assert np.array_equal(kc[pos], rope(k).astype(dt)) and np.array_equal(vc[pos], v.astype(dt))
        assert not kc[:pos].any() and not kc[pos + 1:].any()


def test_attention_restatement_and_reference_geometries():
    rng = np.random.default_rng(2)
    for n_heads, n_kv, hd, seq, max_seq in [(1, 1, 4, 3, 8), (4, 2, 8, 4, 16), (8, 2, 32, 50, 64)]:
        q = rng.uniform(0.1, 10.0, n_heads * hd).astype(np.float32)
        kc = rng.uniform(0.1, 10.0, (max_seq, n_kv * hd)).astype(np.float32)
        vc = rng.uniform(0.1, 10.0, (max_seq, n_kv * hd)).astype(np.float32)
        got = O.attention(q, kc, vc, seq, n_heads, n_kv, hd)
        rep = n_heads // n_kv
        for h in range(n_heads):
            ks = kc[:seq, (h // rep) * hd:(h // rep + 1) * hd].astype(np.float64)
            vs = vc[:seq, (h // rep) * hd:(h // rep + 1) * hd].astype(np.float64)
            s = ks @ q[h * hd:(h + 1) * hd].astype(np.float64) * float(np.float32(1.0 / np.sqrt(np.float32(hd))))
            p = np.exp(s - s.max())
            want = (p / p.sum()) @ vs
            assert np.allclose(got[h * hd:(h + 1) * hd], want, rtol=1e-6, atol=1e-6)
    assert not O.attention(q, kc, vc, 0, n_heads, n_kv, hd).any()
