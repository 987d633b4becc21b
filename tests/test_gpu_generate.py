"""Generation through the entry point, long decoding, the first tokens of a
sequence, each part alone, and a toy mixer with state of its own."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_impl
import traces
from conftest import ROOT, load_plain_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(model_dirs, tiny_configs, name, dtype):
    """The benchmark definition's workload of tiny A: 3 requests, prompts 5/11/17, 8 greedy tokens, page 16 — and B's."""
    from pih_b200.engine import Engine
    lengths = [5, 11, 17] if name == "A" else [1, 9, 33, 64]
    new = 8 if name == "A" else 12
    prompts = list(traces.make_requests(tiny_configs[name]["vocab_size"], lengths, seed=21).values())
    engine = Engine(model_dirs[name], dtype, page_size=16 if name == "A" else 8, max_cache_tokens=1024,
                    maximum_batch_sequences=4, maximum_batch_tokens=8 if name == "B" else 64)
    results = engine.complete_batch(prompts, max_tokens=new, ignore_eos=True)
    engine.rt.ops.check_errors()
    cfg, w = load_plain_weights(model_dirs[name])
    rounding = "none" if dtype == "float32" else "bf16"
    for prompt, res in zip(prompts, results):
        assert res["schema"] == "pih.token-generation-result.v1"
        assert res["prompt_tokens"] == len(prompt) and res["completion_tokens"] == new
        assert res["finish_reason"] == "length"
        ids = list(prompt)
        for i, tok in enumerate(res["token_ids"]):
            logits = plain_impl.forward(cfg, w, ids, rounding)[-1]
            best = int(torch.argmax(logits))
            if tok != best:
                # a near-tie may fall the other way in bf16: the chosen token must be within rounding of the best
                gap = float(logits[best] - logits[tok])
                assert dtype == "bfloat16" and gap < 0.02 * float(logits.std()), (i, tok, best, gap)
            ids.append(tok)
    engine.cache.check()
    assert all(f == engine.cache.num_pages for f in engine.cache.num_free_pages())


def test_temperature_sampling_is_independent_of_batching(model_dirs, tiny_configs):
    """The benchmark definition's workload of tiny B: chunked prefill (8) mixed with decode, temperature 0.8, seed 7."""
    from pih_b200.engine import Engine
    prompts = list(traces.make_requests(384, [1, 9, 33, 64], seed=22).values())
    kw = dict(max_tokens=12, temperature=0.8, seed=7, ignore_eos=True)
    together = Engine(model_dirs["B"], "float32", page_size=8, max_cache_tokens=1024, maximum_batch_sequences=4,
                      maximum_batch_tokens=8).complete_batch(prompts, **kw)
    alone_engine = Engine(model_dirs["B"], "float32", page_size=8, max_cache_tokens=1024,
                          maximum_batch_sequences=1, maximum_batch_tokens=64)
    for prompt, res in zip(prompts, together):
        assert alone_engine.complete(prompt, **kw)["token_ids"] == res["token_ids"]
    # and it follows the plain sampler on the plain logits
    cfg, w = load_plain_weights(model_dirs["B"])
    ids = list(prompts[1])
    for i, tok in enumerate(together[1]["token_ids"]):
        ref, _, _ = plain_impl.sample(plain_impl.forward(cfg, w, ids)[-1].float().tolist(), temperature=0.8,
                                      seed=7, ordinal=i)
        assert tok == ref
        ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, dtype):
    """300 tokens one by one after a short prompt (pages fill and follow each other, windows move on)."""
    from pih_b200.engine.factory import create_runner
    import test_gpu_replay as tr
    name = "B"
    toks = traces.make_requests(384, [330], seed=23)["r0"]
    steps = traces.tail_decode({"r0": toks}, tail=300)
    _, _, cache, runner = create_runner(model_dirs[name], dtype, page_size=8, max_cache_tokens=384, max_requests=2)
    got = traces.replay(runner, steps)
    cfg, w = load_plain_weights(model_dirs[name])
    tr.compare(got, {"r0": plain_impl.forward(cfg, w, toks)}, dtype, "long decoding",
               {"r0": plain_impl.forward(cfg, w, toks, "bf16")} if dtype == "bfloat16" else None)
    # the windowed group gave pages back on the way
    windowed = [g for g in cache.groups if g.need.window is not None]
    assert windowed and windowed[0].pool.pages_handed_out == -(-330 // 8)
    assert all(f == cache.num_pages for f in cache.num_free_pages())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(model_dirs, tiny_configs, name, dtype):
    """Positions 0, 1, 2 decoded one by one from an empty cache."""
    from pih_b200.engine.factory import create_runner
    import test_gpu_replay as tr
    toks = traces.make_requests(tiny_configs[name]["vocab_size"], [4], seed=24)["r0"]
    steps = traces.tail_decode({"r0": toks}, tail=3)
    _, _, _, runner = create_runner(model_dirs[name], dtype, page_size=8, max_cache_tokens=64, max_requests=2)
    got = traces.replay(runner, steps)
    cfg, w = load_plain_weights(model_dirs[name])
    tr.compare(got, {"r0": plain_impl.forward(cfg, w, toks)}, dtype, "first",
               {"r0": plain_impl.forward(cfg, w, toks, "bf16")} if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_each_part_alone(model_dirs, tiny_configs, dtype):
    """Norm, feed-forward, attention mixer and block of configuration B, each against its plain function."""
    from pih_b200.cache import CacheManager
    from pih_b200.config import config_from_dict
    from pih_b200.engine import BatchBuilder, StepEntry
    from pih_b200.kernels import get_ops
    from pih_b200.parts import Runtime, part_class

    cfg, w = load_plain_weights(model_dirs["B"])
    spec = config_from_dict(tiny_configs["B"]).model_spec()
    rt = Runtime(torch.device(DEV), dtype, get_ops(torch.device(DEV)))
    rounding = "none" if dtype == torch.float32 else "bf16"
    tol = dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=4e-3)
    layer = 1
    block_spec = spec.blocks[layer]
    p = block_spec.prefix
    T = 45
    g = torch.Generator().manual_seed(30)
    x = (torch.randn(T, spec.hidden, generator=g)).to(dtype)

    norm = part_class("norm", "rmsnorm")(block_spec.norm_in, {"weight": w[p + "input_layernorm.weight"].to(dtype)}, rt)
    ref = plain_impl.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"], rounding)
    torch.testing.assert_close(norm.forward(x.to(DEV)).cpu().double(), ref, **tol)

    ffn_cls = part_class("ffn", "swiglu")
    ffn = ffn_cls(block_spec.ffn, {n: w[p + n].to(dtype) for n in ffn_cls.expected_tensors(block_spec.ffn)}, rt)
    torch.testing.assert_close(ffn.forward(x.to(DEV)).cpu().double(), plain_impl.mlp_block(w, layer, x, rounding), **tol)

    mixer_cls = part_class("mixer", "attention")
    mixer = mixer_cls(block_spec.mixer, {n: w[p + n].to(dtype) for n in mixer_cls.expected_tensors(block_spec.mixer)}, rt)
    cache = CacheManager([mixer.cache_need()], [None], page_size=8, num_pages=8, max_requests=2,
                         device=rt.device, dtype=dtype)
    cache.add_request("x")
    builder = BatchBuilder(rt.device)
    outs = []
    for lo, hi in [(0, 30), (30, 45)]:                      # two portions: the second reads the first's keys
        cache.append("x", hi - lo)
        step = builder.build([StepEntry("x", [0] * (hi - lo))], cache)
        view = cache.view(0, step.block_tables, step.slot_mappings)
        outs.append(mixer.forward(x[lo:hi].to(DEV), step, view))
        cache.commit("x")
    ref, _ = plain_impl.attention_block(cfg, w, layer, x, list(range(T)), rounding)
    torch.testing.assert_close(torch.cat(outs).cpu().double(), ref, **tol)
    rt.ops.check_errors()


def test_a_toy_mixer_with_state_of_its_own(model_dirs, tiny_configs):
    """A mixer defined here, with per-request state in a state slot, is registered, built into a
    model next to attention layers, and stepped in portions and mixed batches — no framework file changes."""
    from dataclasses import dataclass, replace
    from pih_b200.cache import CacheManager
    from pih_b200.config import config_from_dict
    from pih_b200.engine import ModelRunner, StepEntry
    from pih_b200.kernels import get_ops
    from pih_b200.models import CausalLM, expected_tensors
    from pih_b200.parts import Runtime, StateNeed, TensorInfo, register_mixer, unregister
    from pih_b200.weights import random_tensors

    @dataclass(frozen=True)
    class DecaySpec:
        hidden: int
        decay: float
        kind: str = "toy_decay"

    @register_mixer("toy_decay")
    class DecayMixer:
        """y_t = x_t * gain + s_t, s_t = decay * s_{t-1} + x_t; s lives in the request's state slot."""

        @classmethod
        def expected_tensors(cls, spec):
            return {"toy.gain": TensorInfo((spec.hidden,), "one_plus_normal")}

        def __init__(self, spec, weights, rt):
            self.spec, self.rt = spec, rt
            self.gain = weights["toy.gain"].to(rt.device, torch.float32)

        def cache_need(self):
            return StateNeed((self.spec.hidden,), torch.float32)

        fail_after_writing = False

        def forward(self, x, step, cache):
            # no value leaves the device here (a captured step could not wait for one): the requests' slots are
            # gathered and scattered by index tensors, the row ranges come from the host's copy of cu_q
            out = torch.empty_like(x)
            slots = step.state_slots.long()
            s = cache.state.index_select(0, slots)
            for r in range(step.num_requests):
                sr = s[r]
                for t in range(step.host_cu_q[r], step.host_cu_q[r + 1]):
                    sr = self.spec.decay * sr + x[t].float()
                    out[t] = (x[t].float() * self.gain + sr).to(x.dtype)
                s[r] = sr
            cache.state.index_copy_(0, slots, s)
            if DecayMixer.fail_after_writing:
                raise RuntimeError("the toy mixer fails after it has advanced its state")
            return out

    try:
        base = config_from_dict(tiny_configs["A"]).model_spec()
        blocks = list(base.blocks)
        blocks[1] = replace(blocks[1], mixer=DecaySpec(hidden=base.hidden, decay=0.5))
        spec = replace(base, blocks=tuple(blocks))
        rt = Runtime(torch.device(DEV), torch.float32, get_ops(torch.device(DEV)))
        weights = random_tensors(expected_tensors(spec), seed=4, sigma=0.05, dtype=torch.float32)
        assert "model.layers.1.toy.gain" in weights and "model.layers.1.self_attn.q_proj.weight" not in weights
        model = CausalLM(spec, weights, rt)
        cache = CacheManager(model.cache_needs(), [None, None], page_size=16, num_pages=16, max_requests=3,
                             device=rt.device, dtype=rt.dtype)
        assert len(cache.groups) == 1 and list(cache.state_tensors) == [1]
        runner = ModelRunner(model, cache)
        reqs = traces.make_requests(256, [40, 25, 33], seed=6)
        whole = traces.replay(runner, traces.whole(reqs))
        mixed = traces.replay(runner, traces.mixed(reqs, seed=1, max_live=3))
        for rid in reqs:
            assert float((whole[rid] - mixed[rid]).abs().max()) < 1e-5
        # the same under CUDA graphs: decode steps are captured and replayed, and the state advances once a step
        cache_g = CacheManager(model.cache_needs(), [None, None], page_size=16, num_pages=16, max_requests=3,
                               device=rt.device, dtype=rt.dtype)
        graphed = ModelRunner(model, cache_g, cuda_graphs=True)
        tail = traces.replay(graphed, traces.tail_decode(reqs, tail=12))
        mixed_g = traces.replay(graphed, traces.mixed(reqs, seed=2, max_live=3))
        assert any(k[0] == "decode" for k in graphed._graphs)
        for rid in reqs:
            assert float((whole[rid] - tail[rid]).abs().max()) < 1e-5
            assert float((whole[rid] - mixed_g[rid]).abs().max()) < 1e-5
        # a step that fails after the mixer wrote its state leaves the old state behind, and runs again as new
        toks = reqs["r0"]
        runner.step([StepEntry("x", toks[:10], [9])])
        slot = cache.requests["x"].slot
        state_before = cache.state_tensors[1][slot].clone()
        DecayMixer.fail_after_writing = True
        with pytest.raises(RuntimeError, match="toy mixer fails"):
            runner.step([StepEntry("x", toks[10:14], [3])])
        DecayMixer.fail_after_writing = False
        assert cache.requests["x"].num_tokens == 10 and cache.requests["x"].pending == 0
        assert torch.equal(cache.state_tensors[1][slot], state_before)
        again = runner.step([StepEntry("x", toks[10:14], [3])])
        assert float((again[0].cpu() - whole["r0"][13]).abs().max()) < 1e-5
        runner.finish("x")
        cache.check()
        # state matters: another decay gives other logits after the first token
        blocks[1] = replace(blocks[1], mixer=DecaySpec(hidden=base.hidden, decay=0.0))
        model0 = CausalLM(replace(base, blocks=tuple(blocks)), weights, rt)
        cache0 = CacheManager(model0.cache_needs(), [None, None], page_size=16, num_pages=16, max_requests=3,
                              device=rt.device, dtype=rt.dtype)
        other = traces.replay(ModelRunner(model0, cache0), traces.whole(reqs))
        assert float((other["r0"][0] - whole["r0"][0]).abs().max()) < 1e-6
        assert float((other["r0"][5] - whole["r0"][5]).abs().max()) > 1e-4
    finally:
        unregister("mixer", "toy_decay")


def test_worker_command_line(model_dirs):
    """bin/pih-worker in the reference's manner: --generate-tokens ID,ID,... --max-tokens COUNT."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "pih-worker"), "--model", model_dirs["A"],
           "--generate-tokens", "5,17,3,200", "--max-tokens", "6", "--dtype", "float32"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(proc.stdout.strip().splitlines()[-1])
    assert res["schema"] == "pih.token-generation-result.v1" and res["prompt_tokens"] == 4
    assert res["finish_reason"] in ("stop", "length") and res["completion_tokens"] == len(res["token_ids"]) <= 6
    cfg, w = load_plain_weights(model_dirs["A"])
    ref = plain_impl.generate_greedy(cfg, w, [5, 17, 3, 200], len(res["token_ids"]))
    assert res["token_ids"] == ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_log_probabilities_through_the_entry_point(model_dirs, tiny_configs, dtype):
    """``logprobs=True`` on the GPU, graphs and run-ahead on: one log-probability per token, equal to the plain
    implementation's log-softmax at the tokens that the engine chose (greedy and sampled requests in one batch)."""
    from pih_b200.engine import Engine
    vocab = tiny_configs["A"]["vocab_size"]
    prompts = list(traces.make_requests(vocab, [23, 9, 40], seed=15).values())
    e = Engine(model_dirs["A"], dtype, page_size=16, max_cache_tokens=1024, maximum_batch_sequences=4)
    per = [dict(logprobs=True, top_logprobs=4), dict(logprobs=True, temperature=0.8, seed=3), dict()]
    got = e.complete_batch(prompts, max_tokens=9, ignore_eos=True, parameters_per_prompt=per)
    e.drain()
    e.rt.ops.check_errors()
    assert "logprobs" not in got[2] and "top_logprobs" not in got[1]
    # the greedy request's list of the most probable ids opens with its token and that token's log-probability
    assert len(got[0]["top_logprobs"]) == 9
    for tok, lp, row in zip(got[0]["token_ids"], got[0]["logprobs"], got[0]["top_logprobs"]):
        assert len(row) == 4 and row[0]["token_id"] == tok and abs(row[0]["logprob"] - lp) < 1e-5
        assert all(a["logprob"] >= b["logprob"] for a, b in zip(row, row[1:]))
    cfg, w = load_plain_weights(model_dirs["A"])
    for r, prompt, temperature in ((got[0], prompts[0], 1.0), (got[1], prompts[1], 0.8)):
        assert len(r["logprobs"]) == 9 and all(lp <= 0.0 for lp in r["logprobs"])
        logits = plain_impl.forward(cfg, w, prompt + r["token_ids"])[len(prompt) - 1:-1].double()
        want = torch.log_softmax(logits / temperature, dim=-1)[torch.arange(9), torch.tensor(r["token_ids"])]
        tol = 1e-3 if dtype == "float32" else 0.25           # bf16: the logits themselves carry rounding
        torch.testing.assert_close(torch.tensor(r["logprobs"], dtype=torch.float64), want, rtol=tol, atol=tol)
