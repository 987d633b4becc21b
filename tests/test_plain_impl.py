"""The plain implementation checked against hand-derived values and the reference's known answers."""
import math

import torch

import plain_impl as P


def test_bf16_rounding_is_nearest_even():
    x = torch.tensor([1.0, 1.00390625, 1.005859375, 1.001953125, 3.0e38, -2.5], dtype=torch.float64)
    # 1 + 2^-8 is a tie between 1.0 and 1+2^-7: even mantissa wins (1.0); 1 + 3*2^-9 rounds up
    assert P.bf16_round(x).tolist() == x.to(torch.float32).to(torch.bfloat16).double().tolist()
    assert float(P.bf16_round(torch.tensor([1.00390625]))) == 1.0


def test_rms_norm_known_values():
    # tests/cpp/model/qwen3_cpu_oracle_test.cpp:28-38: rows (3, 4) and (0, 0), weights (1, 2), eps 1:
    # bf16(3 / sqrt(13.5)), bf16(8 / sqrt(13.5)), 0, 0
    out = P.rms_norm(torch.tensor([[3.0, 4.0], [0.0, 0.0]]), torch.tensor([1.0, 2.0]), 1.0, rounding="bf16")
    assert out.tolist() == [[0.81640625, 2.171875], [0.0, 0.0]]


def test_rope_pairs_and_positions():
    D = 8
    cos, sin = P.rope_angles([0, 3], D, 10000.0)
    x = torch.arange(2 * 1 * D, dtype=torch.float64).reshape(2, 1, D)
    out = P.rope_apply(x, cos, sin)
    assert torch.equal(out[0], x[0])                               # position 0 rotates nothing
    inv = [10000.0 ** (-2 * i / D) for i in range(D // 2)]
    for i in range(D // 2):
        a = 3 * inv[i]
        assert abs(float(out[1, 0, i]) - (x[1, 0, i] * math.cos(a) - x[1, 0, i + 4] * math.sin(a))) < 1e-5
        assert abs(float(out[1, 0, i + 4]) - (x[1, 0, i + 4] * math.cos(a) + x[1, 0, i] * math.sin(a))) < 1e-5


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(0)
    T, heads, kv, D = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, D, generator=g, dtype=torch.float64) for n in (heads, kv, kv))
    out = P.attention(q, k, v, 0.3)
    assert torch.allclose(out[0, :2], v[0, 0].expand(2, D)) and torch.allclose(out[0, 2:], v[0, 1].expand(2, D))
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 9.0, -9.0                                       # the future must not matter
    assert torch.equal(P.attention(q, k2, v2, 0.3)[:5], out[:5])
    # online-softmax form of the reference for one row (qwen_bf16_primitives.cu:674-733)
    t, h = 6, 3
    m, l, acc = -math.inf, 0.0, torch.zeros(D, dtype=torch.float64)
    for j in range(t + 1):
        s = float(q[t, h] @ k[j, 1]) * 0.3
        m2 = max(m, s)
        a, b = (0.0 if l == 0.0 else math.exp(m - m2)), math.exp(s - m2)
        l, acc, m = l * a + b, acc * a + b * v[j, 1], m2
    assert torch.allclose(out[t, h], acc / l)
    w = P.attention(q, k, v, 0.3, window=3)
    assert torch.allclose(w[:3], out[:3]) and not torch.allclose(w[5], out[5])
    assert torch.allclose(w[8], P.attention(q[6:], k[6:], v[6:], 0.3)[2])


def test_silu_mul_and_residual_round_once():
    g, u = torch.tensor([1.0, -2.0]), torch.tensor([3.0, 0.5])
    exact = torch.tensor([1.0 / (1 + math.exp(-1.0)) * 3.0, -2.0 / (1 + math.exp(2.0)) * 0.5], dtype=torch.float64)
    assert torch.allclose(P.silu_mul(g, u), exact)
    assert torch.equal(P.silu_mul(g, u, "bf16"), P.bf16_round(exact))
    assert float(P.residual_add(torch.tensor([1.0]), torch.tensor([0.001953125]), "bf16")) == 1.0


def test_philox_known_answers():
    # tests/cpp/model/qwen3_sampler_test.cpp:11-15
    assert P.philox_word(0, 0) == 0x6627E8D5
    assert P.philox_word(0, 3) == 0x9B00DBD8
    assert P.philox_word(0, 4) == 0xF8E4CCA4


def test_sampler_definition():
    logits = [0.0, 2.0, 2.0, -1.0, 1.0]
    assert P.sample(logits)[0] == 1                                  # greedy tie -> lower id
    assert P.sample(logits, suppressed=[1])[0] == 2
    assert P.sample(logits, temperature=1.0, top_k=1, seed=3, ordinal=9)[0] == 1
    assert P.sample(logits, temperature=1.0, top_p=0.3, seed=3, ordinal=9)[0] == 1   # the first already reaches 0.3
    # replayable, keyed by (seed, ordinal)
    a = [P.sample(logits, temperature=1.5, seed=11, ordinal=o)[0] for o in range(50)]
    assert a == [P.sample(logits, temperature=1.5, seed=11, ordinal=o)[0] for o in range(50)]
    assert a != [P.sample(logits, temperature=1.5, seed=12, ordinal=o)[0] for o in range(50)]
    # inverse CDF by hand
    tok, logprob, word = P.sample(logits, temperature=1.0, seed=5, ordinal=2)
    u = (word + 0.5) / 2 ** 32
    order = [1, 2, 4, 0, 3]
    w = [math.exp(logits[i] - 2.0) for i in order]
    c, pick = 0.0, order[-1]
    for i, x in zip(order, w):
        c += x / sum(w)
        if c > u:
            pick = i
            break
    assert tok == pick and abs(logprob - (logits[tok] - math.log(sum(math.exp(x) for x in logits)))) < 1e-5


def test_forward_positions_do_not_depend_on_what_follows(model_dirs):
    from conftest import load_plain_weights
    for name in ("A", "B"):
        cfg, w = load_plain_weights(model_dirs[name])
        toks = torch.randint(0, cfg["vocab_size"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
        full = P.forward(cfg, w, toks)
        assert full.shape == (40, cfg["vocab_size"])
        assert torch.allclose(P.forward(cfg, w, toks[:17]), full[:17], atol=1e-12)
        assert float((P.forward(cfg, w, toks, "bf16") - full).abs().max()) < 0.05 * float(full.std())
    # the window of configuration B matters beyond its length and not before
    cfg_now = dict(cfg, use_sliding_window=False)
    nowin = P.forward(cfg_now, w, toks)
    assert torch.allclose(nowin[:24], full[:24], atol=1e-12) and not torch.allclose(nowin[30], full[30], atol=1e-6)
