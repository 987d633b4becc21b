"""The engine at the layer sizes of Qwen3-0.6B (hidden 1024, 16/8 heads of 128, intermediate 3072, the whole
vocabulary of 151 936; two layers, random weights): the shapes that the benchmark times, which the tiny
configurations never reach — the few-rows products with their fused prologues, the 32-bit-output head, the
decode attention that norms and rotates for itself and merges as a cluster, the tcgen05 prompt attention."""
import pytest

import plain_impl
import traces
from conftest import load_plain_weights
from test_gpu_replay import TOL_F32, compare

pytestmark = pytest.mark.gpu

SIZES = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "torch_dtype": "bfloat16", "hidden_act": "silu",
         "use_cache": True, "tie_word_embeddings": True, "hidden_size": 1024, "intermediate_size": 3072,
         "num_hidden_layers": 2, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128,
         "vocab_size": 151936, "max_position_embeddings": 40960, "rope_theta": 1000000.0, "rms_norm_eps": 1e-06,
         "bos_token_id": 151643, "eos_token_id": 151645, "attention_bias": False, "use_sliding_window": False}


@pytest.fixture(scope="module")
def full_size(tmp_path_factory):
    from pih_b200.config import config_from_dict
    from pih_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("qwen3_0_6b_sizes"))
    write_random_model(d, config_from_dict(SIZES), seed=3, sigma=0.03)
    requests = traces.make_requests(SIZES["vocab_size"], [150, 40, 97], seed=5)
    cfg, w = load_plain_weights(d)
    truth = {rid: plain_impl.forward(cfg, w, toks, "none") for rid, toks in requests.items()}
    plain_bf16 = {rid: plain_impl.forward(cfg, w, toks, "bf16") for rid, toks in requests.items()}
    return d, requests, truth, plain_bf16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["whole", "tail_decode", "portions", "mixed"])
def test_replay_at_full_layer_sizes(full_size, dtype, family):
    from pih_b200.engine.factory import create_runner
    d, requests, truth, plain_bf16 = full_size
    steps = traces.mixed(requests, seed=1, max_live=3) if family == "mixed" else getattr(traces, family)(requests)
    _, model, cache, runner = create_runner(d, dtype, page_size=16, max_requests=4,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=64) + 64)
    got = {rid: g.cpu() for rid, g in traces.replay(runner, steps).items()}
    model.rt.ops.check_errors()
    if dtype == "float32":
        for rid in requests:
            err = float((got[rid].double() - truth[rid]).abs().max())
            assert err < TOL_F32, f"{family} {rid}: max abs error {err:.3e}"
    else:
        compare(got, truth, dtype, f"full size {family}", plain_bf16)
    cache.check()
