"""Plain, slow implementation of the Qwen3 dense decoder and its sampler.

Whole sequences, no cache, no batching, one function per part, float64
arithmetic on the CPU.  It is written from the formulas of the reference
project (GuiminChen/pih); every function cites the file and lines it was
read from (paths are relative to the reference's root).  It shares no code
with the ``pih_b200`` package: it takes a plain ``dict`` as configuration
and a ``dict`` of tensors by safetensors name.

``rounding`` selects where values are rounded:

* ``"none"``  — nothing is rounded (float64 throughout): the truth that the
  engine's true 32-bit path is compared with;
* ``"bf16"``  — every op rounds its output once to bfloat16, at exactly the
  places where the reference's kernels store bf16
  (kernels/cuda/qwen_bf16_primitives.cu), logits stay unrounded
  (src/backend/cuda/gemm_plan.cpp:111-113 gives the LM head an fp32 output).

The reference has no whole-model forward on the CPU, so the composition of
the parts rests on the order of its execution schedule
(plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:19-64); the per-op
functions are checked once against the reference's own CPU oracles by
``tests/golden/make_golden.py``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# --------------------------------------------------------------------------
# rounding
# --------------------------------------------------------------------------
def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even to bfloat16, returned as float64.

    include/pih/core/bfloat16.h:13-27 (= kernels/cuda/qwen_bf16_primitives.cu:16-24):
    add 0x7fff + lsb of the kept part to the float32 bit pattern, keep the
    upper 16 bits.  The value is first rounded to float32 because the
    kernels hold their results in float32 before the store.
    """
    bits = x.to(torch.float32).contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    rounded = bits + 0x7FFF + ((bits >> 16) & 1)
    out = ((rounded >> 16) << 16) & 0xFFFFFFFF
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)
    return out.view(torch.float32).to(F64)


def _rounder(rounding: str):
    if rounding == "none":
        return lambda x: x
    if rounding == "bf16":
        return bf16_round
    raise ValueError(rounding)


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embedding(table: torch.Tensor, token_ids) -> torch.Tensor:
    """h[t,:] = table[id[t],:], a copy without scale.

    plugins/model-qwen3/qwen3_cpu_oracle.cpp:42-69 (ids outside the table are
    an error); kernels/cuda/qwen_bf16_primitives.cu:247-262.
    """
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]):
        raise ValueError("token id is outside the vocabulary")
    return table.to(F64)[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, rounding="none") -> torch.Tensor:
    """y = (x * 1/sqrt(mean(x^2) + eps)) * w, rounded once.

    plugins/model-qwen3/qwen3_cpu_oracle.cpp:85-97;
    kernels/cuda/qwen_bf16_primitives.cu:285-324.  The weight multiplies
    directly (there is no ``1 + w``).
    """
    r = _rounder(rounding)
    x = x.to(F64)
    scale = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return r(x * scale * weight.to(F64))


def linear(x: torch.Tensor, weight: torch.Tensor, rounding="none") -> torch.Tensor:
    """y = x . W^T with W stored [out, in], no bias.

    src/backend/cuda/gemm_plan.cpp:107-129,192-197 (row-major A[m,k] times
    W[n,k] transposed, 32-bit accumulation, bf16 output);
    plugins/model-qwen3/qwen3_config.cpp:65-70 rejects biases.
    """
    return _rounder(rounding)(x.to(F64) @ weight.to(F64).T)


def rope_angles(positions, head_dim: int, theta: float):
    """cos/sin of pos * theta^(-2i/D), i = 0..D/2-1, cast to float32.

    plugins/model-qwen3/qwen3_cpu_oracle.cpp:146-155 (double arithmetic, then
    a cast to float).
    """
    pos = torch.as_tensor(positions, dtype=F64).reshape(-1, 1)
    pair = torch.arange(head_dim // 2, dtype=F64)
    inv = torch.pow(torch.tensor(float(theta), dtype=F64), -2.0 * pair / head_dim)
    angle = pos * inv
    return (torch.cos(angle).to(torch.float32).to(F64),
            torch.sin(angle).to(torch.float32).to(F64))


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rounding="none") -> torch.Tensor:
    """Rotate-half on [T, heads, D]: pairs (x_i, x_{i+D/2}), one row of angles per token.

    plugins/model-qwen3/qwen3_cpu_oracle.cpp:183-196;
    kernels/cuda/qwen_bf16_primitives.cu:326-347.
    """
    half = x.shape[-1] // 2
    first, second = x[..., :half].to(F64), x[..., half:].to(F64)
    c, s = cos[:, None, :], sin[:, None, :]
    out = torch.cat([first * c - second * s, second * c + first * s], dim=-1)
    return _rounder(rounding)(out)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: int | None = None, rounding="none") -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q [T, heads, D]; k, v [T, kv_heads, D].  Query head h reads kv head
    h // (heads // kv_heads); the score is (q . k) * scale (the scale after
    the dot product); row t sees keys 0..t; softmax in full precision; the
    output is rounded once.  plugins/model-qwen3/qwen3_gqa_oracle.cpp:59-103;
    kernels/cuda/qwen_bf16_primitives.cu:660-733.

    ``window`` (not in the reference, which rejects sliding windows in
    plugins/model-qwen3/qwen3_config.cpp:65-70): row t sees only the last
    ``window`` keys, t-window+1..t.
    """
    T, heads, D = q.shape
    kv_heads = k.shape[1]
    group = heads // kv_heads
    q, k, v = q.to(F64), k.to(F64), v.to(F64)
    out = torch.zeros(T, heads, D, dtype=F64)
    rows = torch.arange(T)
    visible = rows[None, :] <= rows[:, None]
    if window is not None:
        visible &= rows[None, :] > rows[:, None] - window
    for h in range(heads):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].T) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ v[:, g, :]
    return _rounder(rounding)(out)


def attention_rows(q: torch.Tensor, positions, k: torch.Tensor, v: torch.Tensor, scale: float,
                   window: int | None = None) -> torch.Tensor:
    """``attention`` for some rows only: q [n, heads, D] are the queries at ``positions`` (row i sees keys
    0..positions[i], or the last ``window`` of them) of a sequence whose keys and values are k, v [L, kv_heads, D].
    Same formula (plugins/model-qwen3/qwen3_gqa_oracle.cpp:59-103), without the L x L score matrix."""
    n, heads, D = q.shape
    L, kv_heads = k.shape[0], k.shape[1]
    group = heads // kv_heads
    q, k, v = q.to(F64), k.to(F64), v.to(F64)
    pos = torch.as_tensor(positions, dtype=torch.long)[:, None]
    keys = torch.arange(L)[None, :]
    visible = keys <= pos
    if window is not None:
        visible &= keys > pos - window
    out = torch.zeros(n, heads, D, dtype=F64)
    for h in range(heads):
        g = h // group
        scores = ((q[:, h, :] @ k[:, g, :].T) * scale).masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ v[:, g, :]
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor, rounding="none") -> torch.Tensor:
    """(g / (1 + exp(-g))) * u, rounded once.

    plugins/model-qwen3/qwen3_cpu_oracle.cpp:121-124;
    kernels/cuda/qwen_bf16_primitives.cu:274-283.
    """
    g = gate.to(F64)
    return _rounder(rounding)((g / (1.0 + torch.exp(-g))) * up.to(F64))


def residual_add(h: torch.Tensor, y: torch.Tensor, rounding="none") -> torch.Tensor:
    """h + y, rounded once.  plugins/model-qwen3/qwen3_cpu_oracle.cpp:107-110;
    kernels/cuda/qwen_bf16_primitives.cu:264-272."""
    return _rounder(rounding)(h.to(F64) + y.to(F64))


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def layer_window(cfg: dict, layer: int) -> int | None:
    """Layers with index >= max_window_layers use the sliding window when
    ``use_sliding_window`` is set (an option that the reference's parser
    names and refuses: plugins/model-qwen3/qwen3_config.cpp:65-70)."""
    if not cfg.get("use_sliding_window", False):
        return None
    if layer >= int(cfg.get("max_window_layers", 0)):
        return int(cfg["sliding_window"])
    return None


def attention_block(cfg: dict, w: dict, layer: int, xn: torch.Tensor, positions,
                    rounding="none", kv_override=None):
    """q/k/v projections, per-head q/k RMSNorm, RoPE, attention, o projection.

    Order from plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:19-39:
    q, k, v GEMMs; q-norm, k-norm (rows of length head_dim, one weight for
    all heads, the model's eps); RoPE on q then k; KV append; attention;
    o projection.  Returns (output, (k, v)) so that another layer can read
    this layer's keys and values (``kv_override``).
    """
    p = f"model.layers.{layer}.self_attn."
    T = xn.shape[0]
    heads, kv_heads, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = linear(xn, w[p + "q_proj.weight"], rounding).reshape(T, heads, D)
    q = rms_norm(q, w[p + "q_norm.weight"], eps, rounding)
    cos, sin = rope_angles(positions, D, cfg["rope_theta"])
    q = rope_apply(q, cos, sin, rounding)
    if kv_override is None:
        k = linear(xn, w[p + "k_proj.weight"], rounding).reshape(T, kv_heads, D)
        v = linear(xn, w[p + "v_proj.weight"], rounding).reshape(T, kv_heads, D)
        k = rms_norm(k, w[p + "k_norm.weight"], eps, rounding)
        k = rope_apply(k, cos, sin, rounding)
    else:
        k, v = kv_override
    # plugins/model-qwen3/nvidia_qwen3_bf16_engine.cpp:371: scale = 1/sqrt(head_dim) in fp32
    scale = float(torch.tensor(1.0 / math.sqrt(D), dtype=torch.float32))
    a = attention(q, k, v, scale, layer_window(cfg, layer), rounding)
    out = linear(a.reshape(T, heads * D), w[p + "o_proj.weight"], rounding)
    return out, (k, v)


def mlp_block(w: dict, layer: int, xn: torch.Tensor, rounding="none") -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ).  qwen3_bf16_execution_schedule.cpp:33-38."""
    p = f"model.layers.{layer}.mlp."
    g = linear(xn, w[p + "gate_proj.weight"], rounding)
    u = linear(xn, w[p + "up_proj.weight"], rounding)
    return linear(silu_mul(g, u, rounding), w[p + "down_proj.weight"], rounding)


def forward(cfg: dict, w: dict, token_ids, rounding="none", schedule=None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence starting at position 0.

    Pre-norm blocks: h += attn(norm(h)); h += mlp(norm(h)); then the final
    norm and the output head (plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:51-63).
    With tied embeddings the head is the embedding table
    (plugins/model-qwen3/artifact/qwen3_source_artifact.cpp:40-70 requires the
    two tensors to be byte-identical).

    ``schedule``: the order in which layers run, a list of ``(layer,
    reads_cache_of)``; ``reads_cache_of`` is None or the index of an earlier
    entry of the list whose keys and values this entry attends to instead of
    its own.  Default: every layer once, in order.
    """
    T = len(token_ids)
    positions = list(range(T))
    eps = cfg["rms_norm_eps"]
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    h = embedding(w["model.embed_tokens.weight"], token_ids)
    kept = []
    for layer, reads in schedule:
        p = f"model.layers.{layer}."
        xn = rms_norm(h, w[p + "input_layernorm.weight"], eps, rounding)
        a, kv = attention_block(cfg, w, layer, xn, positions, rounding,
                                kv_override=None if reads is None else kept[reads])
        kept.append(kv)
        h = residual_add(h, a, rounding)
        xn = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps, rounding)
        h = residual_add(h, mlp_block(w, layer, xn, rounding), rounding)
    xn = rms_norm(h, w["model.norm.weight"], eps, rounding)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(xn, head, "none")


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------
def philox_word(seed: int, ordinal: int) -> int:
    """Philox4x32-10, key = seed (lo, hi), counter = (ordinal // 4 lo, hi, 0, 0),
    word ordinal % 4.  plugins/model-qwen3/qwen3_sampler.cpp:85-104.
    Known answers (tests/cpp/model/qwen3_sampler_test.cpp:11-15):
    (0,0) -> 0x6627e8d5, (0,3) -> 0x9b00dbd8, (0,4) -> 0xf8e4cca4."""
    M32 = 0xFFFFFFFF
    block = ordinal // 4
    c = [block & M32, (block >> 32) & M32, 0, 0]
    k0, k1 = seed & M32, (seed >> 32) & M32
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & M32, p1 & M32, ((p0 >> 32) ^ c[3] ^ k1) & M32, p0 & M32]
        k0 = (k0 + 0x9E3779B9) & M32
        k1 = (k1 + 0xBB67AE85) & M32
    return c[ordinal % 4]


def sample(logits, temperature: float = 0.0, top_p: float = 1.0, top_k: int | None = None,
           seed: int = 0, ordinal: int = 0, suppressed=()):
    """One token from one row of logits; returns (token, logprob, rng word).

    plugins/model-qwen3/qwen3_sampler.cpp:106-185: scaled = logit / T (T = 1
    when greedy); suppressed ids are left out; logsumexp over the rest in
    float32 index order; stable sort descending, ties to the lower id;
    greedy takes the first; otherwise keep the first top_k, weights
    exp(scaled - scaled[0]), the shortest prefix with prefix/sum >= top_p,
    renormalise, u = (word + 0.5) / 2^32 in double, first index whose
    cumulative sum (double) exceeds u, else the last.
    """
    import numpy as np
    lg = np.asarray(logits, dtype=np.float32)
    if not np.isfinite(lg).all():
        raise ValueError("logits contain a non-finite value")
    greedy = temperature == 0.0
    scaled = (lg / np.float32(1.0 if greedy else temperature)).astype(np.float32)
    allowed = [i for i in range(lg.shape[0]) if i not in set(suppressed)]
    amax = max(scaled[i] for i in allowed)
    full = np.float32(0.0)
    for i in allowed:
        full = np.float32(full + np.exp(np.float32(scaled[i] - amax), dtype=np.float32))
    lse = np.float32(amax + np.log(full, dtype=np.float32))
    order = sorted(allowed, key=lambda i: (-float(scaled[i]), i))
    if greedy:
        return order[0], float(scaled[order[0]] - lse), 0
    if top_k is not None and top_k < len(order):
        order = order[:top_k]
    weights = np.exp((scaled[order] - scaled[order[0]]).astype(np.float32), dtype=np.float32)
    filtered = np.float32(0.0)
    for x in weights:
        filtered = np.float32(filtered + x)
    prefix = np.float32(0.0)
    retained = 0
    while True:
        prefix = np.float32(prefix + weights[retained])
        retained += 1
        if not (retained < len(weights) and np.float32(prefix / filtered) < np.float32(top_p)):
            break
    retained_sum = np.float32(0.0)
    for x in weights[:retained]:
        retained_sum = np.float32(retained_sum + x)
    word = philox_word(seed, ordinal)
    u = (float(word) + 0.5) / 4294967296.0
    cumulative = 0.0
    selected = retained - 1
    for i in range(retained):
        cumulative += float(np.float32(weights[i] / retained_sum))
        if cumulative > u:
            selected = i
            break
    tok = order[selected]
    return tok, float(scaled[tok] - lse), word


def top_logprobs(logits, count: int, temperature: float = 0.0, suppressed=()):
    """The ``count`` most probable ids of one row with their log-probabilities, best first.

    plugins/model-qwen3/qwen3_sampler.cpp:118-143: scaled = logit / T (T = 1 when greedy); suppressed ids are
    left out; order by scaled value descending, ties to the lower id; the first ``count`` with
    scaled - logsumexp (here in float64: the reference's own float32 sum runs one after the other).
    """
    import numpy as np
    lg = np.asarray(logits, dtype=np.float32)
    scaled = (lg / np.float32(1.0 if temperature == 0.0 else temperature)).astype(np.float32)
    sup = set(suppressed)
    allowed = [i for i in range(lg.shape[0]) if i not in sup]
    vals = scaled[allowed].astype(np.float64)
    lse = float(vals.max() + np.log(np.exp(vals - vals.max()).sum()))
    order = sorted(allowed, key=lambda i: (-float(scaled[i]), i))[:count]
    return [(i, float(scaled[i]) - lse) for i in order]


def generate_greedy(cfg: dict, w: dict, prompt, max_new: int, rounding="none"):
    """Greedy generation by re-running the whole sequence for every token."""
    ids = list(prompt)
    out = []
    for _ in range(max_new):
        logits = forward(cfg, w, ids, rounding)
        tok = int(torch.argmax(logits[-1].to(torch.float32)))
        out.append(tok)
        ids.append(tok)
    return out
