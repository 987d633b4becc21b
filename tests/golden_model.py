"""The tiny model behind tests/golden/: sizes that the reference's fixed-size oracles accept
(16 query heads, 8 kv heads, head_dim 128, rope theta 1e6), seeded bf16 weights, and the order in which
tests/golden/oracle_driver.cpp reads the tensors."""
import torch

CONFIG = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "torch_dtype": "bfloat16", "hidden_act": "silu",
    "tie_word_embeddings": True, "hidden_size": 48, "intermediate_size": 80, "num_hidden_layers": 2,
    "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 96,
    "max_position_embeddings": 64, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "use_sliding_window": False,
}
TOKENS = [5, 17, 3, 90, 41, 9, 77, 5, 60]
SAMPLE_CASES = [  # temperature, top_p, top_k, seed, ordinal, suppress the greedy token?
    (0.0, 1.0, None, 0, 0, False), (0.8, 1.0, None, 7, 0, False), (0.8, 1.0, None, 7, 5, False),
    (1.5, 0.9, None, 123, 2, False), (1.0, 1.0, 5, 9, 1, False), (2.0, 0.5, 40, 99, 11, False),
    (0.0, 1.0, None, 0, 0, True), (1.0, 1.0, None, 4, 3, True)]


def tensor_order():
    names = ["model.embed_tokens.weight"]
    for i in range(CONFIG["num_hidden_layers"]):
        p = f"model.layers.{i}."
        names += [p + "input_layernorm.weight", p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                  p + "self_attn.v_proj.weight", p + "self_attn.q_norm.weight", p + "self_attn.k_norm.weight",
                  p + "self_attn.o_proj.weight", p + "post_attention_layernorm.weight", p + "mlp.gate_proj.weight",
                  p + "mlp.up_proj.weight", p + "mlp.down_proj.weight"]
    return names + ["model.norm.weight"]


def make_weights():
    c = CONFIG
    H, I, V, D = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["head_dim"]
    Hq, Hkv = c["num_attention_heads"] * D, c["num_key_value_heads"] * D
    shapes = {"embed_tokens.weight": (V, H), "input_layernorm.weight": (H,), "q_proj.weight": (Hq, H),
              "k_proj.weight": (Hkv, H), "v_proj.weight": (Hkv, H), "q_norm.weight": (D,), "k_norm.weight": (D,),
              "o_proj.weight": (H, Hq), "post_attention_layernorm.weight": (H,), "gate_proj.weight": (I, H),
              "up_proj.weight": (I, H), "down_proj.weight": (H, I), "norm.weight": (H,)}
    g = torch.Generator().manual_seed(2024)
    out = {}
    for name in tensor_order():
        key = ".".join(name.split(".")[-2:])              # e.g. q_proj.weight, embed_tokens.weight, norm.weight
        shape = shapes[key]
        t = torch.randn(shape, generator=g) * 0.08
        if len(shape) == 1:
            t = t + 1.0
        out[name] = t.to(torch.bfloat16)
    return out
