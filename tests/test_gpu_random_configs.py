"""Seeded random configurations of the architecture — head sizes in steps of 16 up to 256, any number of heads and
groups, widths and vocabularies that are no power of two, windows, page sizes from 4 to 128 — through the
replay families against the plain implementation, in 32-bit and in bfloat16.  Every kernel has to take the size
or leave it to one that does; none may give a wrong result."""
import random

import pytest

import plain_impl
import traces
from conftest import load_plain_weights
from test_gpu_replay import compare

pytestmark = pytest.mark.gpu


def _random_config(rng):
    kv = rng.choice([1, 2, 3, 4])
    group = rng.choice([1, 2, 3, 4, 7])
    layers = rng.choice([1, 2, 3])
    window = rng.choice([None, None, 20, 70])
    raw = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "torch_dtype": "bfloat16", "hidden_act": "silu",
           "use_cache": True, "tie_word_embeddings": rng.choice([True, False]),
           "hidden_size": rng.choice([34, 50, 66, 40, 64, 72, 100, 136, 160, 200, 250, 256, 1024]),
           "intermediate_size": rng.choice([30, 48, 96, 104, 200, 264, 320, 1000]), "num_hidden_layers": layers,
           "num_attention_heads": kv * group, "num_key_value_heads": kv,
           "head_dim": rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 160, 192, 208, 256, 128, 64]),
           "vocab_size": rng.choice([97, 256, 1001, 5000]), "max_position_embeddings": 1024,
           "rope_theta": rng.choice([10000.0, 1e6]), "rms_norm_eps": rng.choice([1e-6, 1e-5]), "bos_token_id": 0,
           "eos_token_id": 1, "attention_bias": False, "use_sliding_window": window is not None}
    if window is not None:
        raw.update(sliding_window=window, max_window_layers=rng.randrange(0, layers))
    return raw, rng.choice([4, 8, 16, 32, 64, 128])


@pytest.mark.parametrize("seed", range(10))
def test_a_random_configuration(tmp_path, seed):
    from pih_b200.config import config_from_dict
    from pih_b200.engine.factory import create_runner
    from pih_b200.weights import write_random_model
    rng = random.Random(1000 + seed)
    raw, page = _random_config(rng)
    what = (f"head_dim {raw['head_dim']} heads {raw['num_attention_heads']}/{raw['num_key_value_heads']} hidden "
            f"{raw['hidden_size']} intermediate {raw['intermediate_size']} vocab {raw['vocab_size']} layers "
            f"{raw['num_hidden_layers']} window {raw.get('sliding_window')} page {page}")
    d = str(tmp_path)
    write_random_model(d, config_from_dict(raw), seed=seed, sigma=0.06)
    cfg, w = load_plain_weights(d)
    requests = traces.make_requests(raw["vocab_size"], [rng.randrange(20, 200) for _ in range(4)], seed=seed)
    truth = {r: plain_impl.forward(cfg, w, t, "none") for r, t in requests.items()}
    plain = {r: plain_impl.forward(cfg, w, t, "bf16") for r, t in requests.items()}
    for dtype in ("float32", "bfloat16"):
        for family in ("tail_decode", "portions", "mixed"):
            steps = getattr(traces, family)(requests)
            _, model, cache, runner = create_runner(d, dtype, page_size=page, max_requests=4,
                                                    max_cache_tokens=traces.peak_tokens(steps, round_to=max(64, page)))
            got = {r: g.cpu() for r, g in traces.replay(runner, steps).items()}
            model.rt.ops.check_errors()
            compare(got, truth, dtype, f"{what}: {dtype} {family}", plain)
            cache.check()


@pytest.mark.parametrize("seed", range(4))
def test_greedy_generation_on_a_random_configuration(tmp_path, seed):
    """Scheduler, run-ahead, sampler and step function together, in 32-bit: the tokens of the plain implementation."""
    import torch
    from pih_b200.config import config_from_dict
    from pih_b200.engine import Engine
    from pih_b200.weights import write_random_model
    rng = random.Random(2000 + seed)
    raw, page = _random_config(rng)
    d = str(tmp_path)
    write_random_model(d, config_from_dict(raw), seed=seed, sigma=0.08)
    cfg, w = load_plain_weights(d)
    prompts = list(traces.make_requests(raw["vocab_size"], [rng.randrange(1, 70) for _ in range(5)], seed=seed).values())
    engine = Engine(d, "float32", page_size=page, max_cache_tokens=1024, maximum_batch_sequences=3,
                    maximum_batch_tokens=rng.choice([8, 32, 200]))
    results = engine.complete_batch(prompts, max_tokens=7, ignore_eos=True)
    engine.rt.ops.check_errors()
    for prompt, res in zip(prompts, results):
        ids = list(prompt)
        for tok in res["token_ids"]:
            logits = plain_impl.forward(cfg, w, ids)[-1]
            best = int(torch.argmax(logits))
            assert tok == best or float(logits[best] - logits[tok]) < 1e-4, (ids[len(prompt):], tok, best)
            ids.append(tok)
        assert res["completion_tokens"] == 7 and res["finish_reason"] == "length"
    engine.cache.check()
    assert all(f == engine.cache.num_pages for f in engine.cache.num_free_pages())
