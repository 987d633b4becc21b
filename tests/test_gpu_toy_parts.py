"""Parts that are no model's: a feed-forward with routing and another position encoding, defined here,
registered, built into a model beside the architecture's own parts and stepped through the engine — whole,
in portions and mixed — without a change to the framework's files.  Each has its plain formula here too."""
import math
from dataclasses import dataclass, replace

import pytest
import torch

import plain_impl
import traces

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _reference(cfg, w, token_ids, ffn_at=None, rope=None):
    """plain_impl.forward with one layer's feed-forward or every layer's rotation replaced (float64)."""
    T = len(token_ids)
    eps = cfg["rms_norm_eps"]
    heads, kv_heads, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    h = plain_impl.embedding(w["model.embed_tokens.weight"], token_ids)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        xn = plain_impl.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        if rope is None:
            a, _ = plain_impl.attention_block(cfg, w, layer, xn, list(range(T)))
        else:
            q = plain_impl.linear(xn, w[p + "self_attn.q_proj.weight"]).reshape(T, heads, D)
            k = plain_impl.linear(xn, w[p + "self_attn.k_proj.weight"]).reshape(T, kv_heads, D)
            v = plain_impl.linear(xn, w[p + "self_attn.v_proj.weight"]).reshape(T, kv_heads, D)
            q = rope(plain_impl.rms_norm(q, w[p + "self_attn.q_norm.weight"], eps))
            k = rope(plain_impl.rms_norm(k, w[p + "self_attn.k_norm.weight"], eps))
            scale = float(torch.tensor(1.0 / math.sqrt(D), dtype=torch.float32))
            a = plain_impl.attention(q, k, v, scale, plain_impl.layer_window(cfg, layer))
            a = plain_impl.linear(a.reshape(T, heads * D), w[p + "self_attn.o_proj.weight"])
        h = plain_impl.residual_add(h, a)
        xn = plain_impl.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        y = ffn_at[layer](xn) if ffn_at and layer in ffn_at else plain_impl.mlp_block(w, layer, xn)
        h = plain_impl.residual_add(h, y)
    xn = plain_impl.rms_norm(h, w["model.norm.weight"], eps)
    return plain_impl.linear(xn, w["model.embed_tokens.weight"])


def _run(spec, weights, requests, pages=24):
    from pih_b200.cache import CacheManager
    from pih_b200.engine import ModelRunner
    from pih_b200.kernels import get_ops
    from pih_b200.models import CausalLM
    from pih_b200.parts import Runtime
    rt = Runtime(torch.device(DEV), torch.float32, get_ops(torch.device(DEV)))
    model = CausalLM(spec, weights, rt)
    cache = CacheManager(model.cache_needs(), [e.reads_cache_of for e in spec.schedule], page_size=16, num_pages=pages,
                         max_requests=3, device=rt.device, dtype=rt.dtype)
    runner = ModelRunner(model, cache)
    out = {name: traces.replay(runner, getattr(traces, name)(requests, **kw))
           for name, kw in (("whole", {}), ("portions", {}), ("mixed", dict(seed=2, max_live=3)))}
    rt.ops.check_errors()
    cache.check()
    return out


def _plain_weights(weights):
    return {k: v.to(F64).cpu() for k, v in weights.items()}


def test_a_toy_feed_forward_with_routing(tiny_configs):
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    from pih_b200.parts import TensorInfo, register_ffn, unregister
    from pih_b200.weights import random_tensors

    @dataclass(frozen=True)
    class RoutedSpec:
        hidden: int
        experts: int
        kind: str = "toy_routed"

    @register_ffn("toy_routed")
    class RoutedFeedForward:
        """y = p_e * (x . W_e^T) for the expert e with the largest router logit; p = softmax of the logits
        (32-bit).  Every expert's product runs for every row and the chosen one is picked (a toy)."""

        @classmethod
        def expected_tensors(cls, spec):
            out = {"toy.router.weight": TensorInfo((spec.experts, spec.hidden))}
            for e in range(spec.experts):
                out[f"toy.experts.{e}.weight"] = TensorInfo((spec.hidden, spec.hidden))
            return out

        def __init__(self, spec, weights, rt):
            self.spec, self.rt = spec, rt
            self.router = weights["toy.router.weight"].to(rt.device, rt.dtype)
            self.experts = [weights[f"toy.experts.{e}.weight"].to(rt.device, rt.dtype) for e in range(spec.experts)]

        def forward(self, x):
            ops = self.rt.ops
            logits = ops.linear(x, self.router).float()
            probs = torch.softmax(logits, dim=-1)
            top = probs.argmax(dim=-1)
            ys = torch.stack([ops.linear(x, w) for w in self.experts], dim=1)        # [T, E, H]
            rows = torch.arange(x.shape[0], device=x.device)
            return (ys[rows, top].float() * probs[rows, top][:, None]).to(x.dtype)

    try:
        cfg = tiny_configs["A"]
        base = config_from_dict(cfg).model_spec()
        blocks = list(base.blocks)
        blocks[1] = replace(blocks[1], ffn=RoutedSpec(hidden=base.hidden, experts=3))
        spec = replace(base, blocks=tuple(blocks))
        weights = random_tensors(expected_tensors(spec), seed=8, sigma=0.08, dtype=torch.float32)
        assert "model.layers.1.toy.router.weight" in weights and "model.layers.1.mlp.gate_proj.weight" not in weights
        requests = traces.make_requests(cfg["vocab_size"], [40, 25, 33], seed=3)
        got = _run(spec, weights, requests)
        w = _plain_weights(weights)

        def routed(xn):
            logits = plain_impl.linear(xn, w["model.layers.1.toy.router.weight"])
            probs = torch.softmax(logits, dim=-1)
            top = probs.argmax(dim=-1)
            ys = torch.stack([plain_impl.linear(xn, w[f"model.layers.1.toy.experts.{e}.weight"]) for e in range(3)], dim=1)
            rows = torch.arange(xn.shape[0])
            return ys[rows, top] * probs[rows, top][:, None]

        experts_used = set()
        for rid, toks in requests.items():
            ref = _reference(cfg, w, toks, ffn_at={1: routed})
            for name in ("whole", "portions", "mixed"):
                err = float((got[name][rid].double().cpu() - ref).abs().max())
                assert err < 5e-5, (name, rid, err)
        # the router does route: more than one expert is chosen over these rows
        xn = torch.randn(64, base.hidden, dtype=F64)
        experts_used.update(plain_impl.linear(xn, w["model.layers.1.toy.router.weight"]).argmax(-1).tolist())
        assert len(experts_used) > 1
    finally:
        unregister("ffn", "toy_routed")


def test_a_toy_position_encoding(tiny_configs):
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    from pih_b200.parts import register_position, unregister
    from pih_b200.weights import random_tensors

    @dataclass(frozen=True)
    class SlowRotarySpec:
        head_dim: int
        rotary_dim: int
        period: float
        max_positions: int
        kind: str = "toy_slow_rotary"

    @register_position("toy_slow_rotary")
    class SlowRotary:
        """Rotates only the first ``rotary_dim`` columns of a head, pair i by the angle pos * (i + 1) / period —
        angles that are linear, not geometric, in i."""

        @classmethod
        def expected_tensors(cls, spec):
            return {}

        def __init__(self, spec, weights, rt):
            self.rotary_dim = spec.rotary_dim
            pos = torch.arange(spec.max_positions, dtype=F64)[:, None]
            angle = pos * (torch.arange(spec.rotary_dim // 2, dtype=F64) + 1)[None, :] / spec.period
            self._table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32).to(rt.device)

        def rotation_table(self):
            return self._table

    try:
        cfg = tiny_configs["A"]
        base = config_from_dict(cfg).model_spec()
        D = cfg["head_dim"]
        rot = D // 2
        pos_spec = SlowRotarySpec(head_dim=D, rotary_dim=rot, period=7.0, max_positions=base.max_positions)
        blocks = tuple(replace(b, mixer=replace(b.mixer, position=pos_spec)) for b in base.blocks)
        spec = replace(base, blocks=blocks)
        weights = random_tensors(expected_tensors(spec), seed=9, sigma=0.08, dtype=torch.float32)
        requests = traces.make_requests(cfg["vocab_size"], [40, 25, 33], seed=4)
        got = _run(spec, weights, requests)
        w = _plain_weights(weights)

        def rope(x):                                      # [T, heads, D], rows at positions 0..T-1
            T = x.shape[0]
            angle = torch.arange(T, dtype=F64)[:, None] * (torch.arange(rot // 2, dtype=F64) + 1)[None, :] / 7.0
            cos = torch.cos(angle).to(torch.float32).to(F64)
            sin = torch.sin(angle).to(torch.float32).to(F64)
            return torch.cat([plain_impl.rope_apply(x[..., :rot], cos, sin), x[..., rot:].to(F64)], dim=-1)

        for rid, toks in requests.items():
            ref = _reference(cfg, w, toks, rope=rope)
            usual = plain_impl.forward(cfg, w, toks)
            assert float((ref - usual).abs().max()) > 1e-3          # the encoding matters
            for name in ("whole", "portions", "mixed"):
                err = float((got[name][rid].double().cpu() - ref).abs().max())
                assert err < 5e-5, (name, rid, err)
    finally:
        unregister("position", "toy_slow_rotary")
