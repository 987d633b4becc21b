"""The plain implementation against the reference project's own CPU oracles (tests/golden/).

``tests/golden/make_golden.py`` compiled the reference's per-op oracles and ran a tiny Qwen3-shaped model
through them; its outputs are committed as ``qwen3_oracle_outputs.json``.  Both sides round to bf16 at the
same places; the oracle accumulates in float32 in index order, the plain implementation in float64, so a
value near a rounding boundary may fall to the other side: the comparison allows a few bf16 ulps of the
logits' scale, and the samplers must pick the same tokens."""
import json
import os

import torch

import plain_impl
from golden_model import CONFIG, SAMPLE_CASES, TOKENS, make_weights

HERE = os.path.dirname(os.path.abspath(__file__))


def _golden():
    with open(os.path.join(HERE, "golden", "qwen3_oracle_outputs.json")) as f:
        return json.load(f)


def test_plain_forward_matches_the_reference_oracles():
    gold = _golden()
    w = {k: v.to(torch.float64) for k, v in make_weights().items()}
    T, V = len(TOKENS), CONFIG["vocab_size"]
    want = torch.tensor(gold["logits"], dtype=torch.float64).reshape(T, V)
    got = plain_impl.forward(CONFIG, w, TOKENS, "bf16")
    truth = plain_impl.forward(CONFIG, w, TOKENS, "none")
    spread = float(want.std())
    # the two bf16 pipelines differ by accumulation order only; both sit the same distance from the truth
    assert float((got - want).abs().max()) < 0.02 * spread, float((got - want).abs().max()) / spread
    assert float((got - want).abs().mean()) < 0.004 * spread
    assert abs(float((got - truth).abs().mean()) - float((want - truth).abs().mean())) < 0.002 * spread
    assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_plain_attention_matches_the_reference_oracle():
    gold = _golden()
    w = {k: v.to(torch.float64) for k, v in make_weights().items()}
    T = len(TOKENS)
    eps = CONFIG["rms_norm_eps"]
    h = plain_impl.embedding(w["model.embed_tokens.weight"], TOKENS)
    for layer in range(CONFIG["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        xn = plain_impl.rms_norm(h, w[p + "input_layernorm.weight"], eps, "bf16")
        # attention output before the o projection
        D, heads, kvh = CONFIG["head_dim"], CONFIG["num_attention_heads"], CONFIG["num_key_value_heads"]
        q = plain_impl.linear(xn, w[p + "self_attn.q_proj.weight"], "bf16").reshape(T, heads, D)
        k = plain_impl.linear(xn, w[p + "self_attn.k_proj.weight"], "bf16").reshape(T, kvh, D)
        v = plain_impl.linear(xn, w[p + "self_attn.v_proj.weight"], "bf16").reshape(T, kvh, D)
        cos, sin = plain_impl.rope_angles(range(T), D, CONFIG["rope_theta"])
        q = plain_impl.rope_apply(plain_impl.rms_norm(q, w[p + "self_attn.q_norm.weight"], eps, "bf16"), cos, sin, "bf16")
        k = plain_impl.rope_apply(plain_impl.rms_norm(k, w[p + "self_attn.k_norm.weight"], eps, "bf16"), cos, sin, "bf16")
        a = plain_impl.attention(q, k, v, float(torch.tensor(D ** -0.5, dtype=torch.float32)), None, "bf16")
        want = torch.tensor(gold["attention"][layer], dtype=torch.float64)
        got = a.reshape(-1)[::16]
        assert got.shape == want.shape
        assert float((got - want).abs().max()) < 0.02 * float(want.std()), layer
        out, _ = plain_impl.attention_block(CONFIG, w, layer, xn, list(range(T)), "bf16")
        h = plain_impl.residual_add(h, out, "bf16")
        xn = plain_impl.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps, "bf16")
        h = plain_impl.residual_add(h, plain_impl.mlp_block(w, layer, xn, "bf16"), "bf16")


def test_plain_sampler_matches_the_reference_sampler():
    gold = _golden()
    T, V = len(TOKENS), CONFIG["vocab_size"]
    row = torch.tensor(gold["logits"], dtype=torch.float32).reshape(T, V)[-1]
    best = int(row.argmax())
    for (t, p, k, seed, ordinal, suppress), (tok, logprob, word) in zip(SAMPLE_CASES, gold["samples"]):
        got_tok, got_lp, got_word = plain_impl.sample(row.tolist(), temperature=t, top_p=p, top_k=k, seed=seed,
                                                      ordinal=ordinal, suppressed=[best] if suppress else [])
        assert (got_tok, got_word) == (tok, word), (t, p, k, seed, ordinal, suppress)
        assert abs(got_lp - logprob) < 1e-5
    assert gold["philox"][:3] == [0x6627E8D5, 0x9B00DBD8, 0xF8E4CCA4]
    assert gold["philox"][3] == plain_impl.philox_word(0, 1000003)
