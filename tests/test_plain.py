"""The plain implementation against the reference's own small vectors (read from
its unit tests as text) and against independent restatements of its parts."""
import math

import numpy as np

import plain_llama as plain


def test_gemv_layout_vector():
    # model/gemv_helpers_test.go:23-42: x=[2,3], W=[[1,2],[10,20]] ([out,in]) -> [8,80]
    out = plain.linear(np.array([[2.0, 3.0]], dtype=np.float32), np.array([[1, 2], [10, 20]], dtype=np.float32))
    assert out.tolist() == [[8.0, 80.0]]


def test_finish_decode_step_vector():
    # model/cpu_decode_step_test.go:9-26: hidden [3,4], eps 0, unit norm, LM rows
    # [1,0],[0,1],[1,1] -> argmax 2
    cfg = {"rms_norm_eps": 0.0}
    w = {"model.norm.weight": np.ones(2, dtype=np.float32),
         "lm_head.weight": np.array([[1, 0], [0, 1], [1, 1]], dtype=np.float32)}
    cfg = dict(cfg)
    logits = plain.linear(plain.rms_norm(np.array([[3.0, 4.0]], dtype=np.float32), w["model.norm.weight"], 0.0),
                          w["lm_head.weight"])[0]
    assert plain.argmax_first(logits) == 2
    s = 1.0 / math.sqrt((9 + 16) / 2)
    np.testing.assert_allclose(logits, [3 * s, 4 * s, 7 * s], rtol=1e-6)


def test_argmax_tie_goes_to_the_lowest_index():
    # model/inference_helpers.go:153-166 (strict '>')
    assert plain.argmax_first(np.array([1.0, 5.0, 5.0, 2.0], dtype=np.float32)) == 1


def reference_attention_vector():
    """The case of model/attention_test.go:48-68: one query over seqLen = 17 keys, 6
    heads on 2 key/value heads of 32 channels, q, k and v all benchSeq (x_i =
    float32(sin(0.013 i)), model/cpu_hotpath_bench_test.go:12-18, each starting at
    i = 0), scale 0.37; and what that file's own oracle, the triple loop
    gqaAttentionScaleReference (:8-46), gives for it, restated with its float32
    running sums."""
    T, nh, nkv, hd, scale = 17, 6, 2, 32, np.float32(0.37)
    seq = lambda n: np.sin(np.arange(n, dtype=np.float64) * 0.013).astype(np.float32)
    q, k, v = seq(nh * hd), seq(T * nkv * hd), seq(T * nkv * hd)
    kv_dim = nkv * hd
    want = np.zeros(nh * hd, dtype=np.float32)
    for head in range(nh):
        kvh = head // (nh // nkv)
        scores = np.zeros(T, dtype=np.float32)
        for t in range(T):
            total = np.float32(0)
            for d in range(hd):
                total = np.float32(total + q[head * hd + d] * k[t * kv_dim + kvh * hd + d])
            scores[t] = total * scale
        mx = scores.max()
        exp_sum = np.float32(0)
        for t in range(T):
            scores[t] = np.float32(math.exp(float(scores[t] - mx)))
            exp_sum = np.float32(exp_sum + scores[t])
        scores = scores / exp_sum
        for d in range(hd):
            total = np.float32(0)
            for t in range(T):
                total = np.float32(total + scores[t] * v[t * kv_dim + kvh * hd + d])
            want[head * hd + d] = total
    return q, k.reshape(T, kv_dim), v.reshape(T, kv_dim), want, (T, nh, nkv, hd, float(scale))


def test_attention_on_the_reference_vector():
    # model/attention_test.go:48-68, tolerance 2e-5 as there
    q, k, v, want, (T, nh, nkv, hd, scale) = reference_attention_vector()
    queries = np.zeros((T, nh * hd), dtype=np.float32)
    queries[T - 1] = q                                   # the query of the newest token sees all 17 keys
    got = plain.causal_gqa_attention(queries, k, v, nh, nkv, hd, scale=scale)[T - 1]
    assert np.abs(got - want).max() < 2e-5
    assert np.abs(want).max() > 0.05                     # the vector is not trivially zero


def test_attention_window_keeps_the_last_keys_only():
    T, hd = 9, 4
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((T, hd)).astype(np.float32) for _ in range(3))
    full = plain.causal_gqa_attention(q, k, v, 1, 1, hd)
    win = plain.causal_gqa_attention(q, k, v, 1, 1, hd, window=3)
    np.testing.assert_allclose(win[:3], full[:3], rtol=1e-6)
    alone = plain.causal_gqa_attention(q[6:9], k[6:9], v[6:9], 1, 1, hd)
    np.testing.assert_allclose(win[8], alone[2], rtol=1e-5)


def test_rope_is_half_split_and_a_rotation():
    hd = 8
    inv = plain.rope_inv_freq({"head_dim": hd, "rope_theta": 10000.0, "rope_scaling": None})
    np.testing.assert_allclose(inv, [10000.0 ** (-2 * i / hd) for i in range(hd // 2)])
    x = np.arange(1, hd + 1, dtype=np.float32)[None, :]
    y = plain.rope(x, [3], inv, 1, hd)[0]
    for i in range(hd // 2):
        c, s = math.cos(3 * inv[i]), math.sin(3 * inv[i])
        assert abs(y[i] - (x[0, i] * c - x[0, i + hd // 2] * s)) < 1e-5
        assert abs(y[i + hd // 2] - (x[0, i] * s + x[0, i + hd // 2] * c)) < 1e-5
    np.testing.assert_allclose(plain.rope(x, [0], inv, 1, hd), x)
    assert abs(np.linalg.norm(y) - np.linalg.norm(x)) < 1e-4


def test_llama3_scaling_of_the_frequencies():
    cfg = {"head_dim": 64, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                            "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}}
    base = plain.rope_inv_freq({**cfg, "rope_scaling": None})
    scaled = plain.rope_inv_freq(cfg)
    wavelen = 2 * math.pi / base
    assert np.all(scaled[wavelen < 8192 / 4] == base[wavelen < 8192 / 4])
    np.testing.assert_allclose(scaled[wavelen > 8192], base[wavelen > 8192] / 8.0)
    mid = (wavelen >= 8192 / 4) & (wavelen <= 8192)
    assert mid.any() and np.all(scaled[mid] < base[mid]) and np.all(scaled[mid] > base[mid] / 8.0)


def test_rms_norm_and_silu():
    x = np.array([[1.0, -2.0, 3.0, 0.5]], dtype=np.float32)
    w = np.array([1.0, 0.5, 2.0, 1.0], dtype=np.float32)
    want = w * x / math.sqrt(float((x ** 2).mean()) + 1e-5)
    np.testing.assert_allclose(plain.rms_norm(x, w, 1e-5), want, rtol=1e-6)
    g = np.array([-3.0, 0.0, 2.0], dtype=np.float32)
    np.testing.assert_allclose(plain.silu_mul(g, np.ones(3, dtype=np.float32)),
                               g / (1 + np.exp(-g)), rtol=1e-6)


def test_uniform_and_inverse_cdf():
    us = [plain.uniform(7, s, t) for s in range(4) for t in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) == len(us)
    assert 0.35 < float(np.mean(us)) < 0.65
    assert plain.uniform(7, 2, 5) == plain.uniform(7, 2, 5) != plain.uniform(8, 2, 5)
    logits = np.log(np.array([0.1, 0.2, 0.7], dtype=np.float32))
    assert plain.sample_temperature(logits, 1.0, 0.05) == 0
    assert plain.sample_temperature(logits, 1.0, 0.25) == 1
    assert plain.sample_temperature(logits, 1.0, 0.95) == 2


def test_forward_does_not_look_ahead(plain_models):
    cfg, w = plain_models["A"]
    tokens = [3, 200, 17, 45, 99, 7]
    full = plain.forward(cfg, w, tokens)
    np.testing.assert_allclose(plain.forward(cfg, w, tokens[:4]), full[:4], rtol=2e-5, atol=2e-6)
    changed = plain.forward(cfg, w, tokens[:5] + [8])
    np.testing.assert_allclose(changed[:5], full[:5], rtol=2e-5, atol=2e-6)
    assert np.abs(changed[5] - full[5]).max() > 1e-3


def test_generate_stops_at_a_stop_token(plain_models):
    cfg, w = plain_models["A"]
    free = plain.generate(cfg, w, [5, 6, 7], 6)
    assert len(free) == 6
    stopped = plain.generate(cfg, w, [5, 6, 7], 6, stop=(free[2],))
    assert stopped == free[:free.index(free[2]) + 1]
