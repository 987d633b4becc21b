// Runs a tiny Qwen3-shaped model through the REFERENCE project's own CPU oracles
// (plugins/model-qwen3/qwen3_cpu_oracle.cpp, qwen3_gqa_oracle.cpp, qwen3_sampler.cpp), which are compiled
// from the reference's tree by make_golden.py — none of their code is copied here.  The reference has no
// CPU matrix product (it calls cuBLASLt: src/backend/cuda/gemm_plan.cpp:192-197) and no whole-model
// forward, so this driver supplies the glue: products with 32-bit accumulation rounded once to bf16
// (fp32 for the head), and the order of operations of
// plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:19-64.  The attention oracle is fixed to 16 query
// heads, 8 kv heads and head_dim 128, and the angle oracle to head_dim 128 and theta 1e6, so the tiny
// model has those sizes.
//
// stdin:  text: L H I V T eps, then token ids, then all tensors as floats in the order written by make_golden.py
// stdout: text: logits [T, V], then every 16th element of each layer's attention output, then sampler results
#include <cstdint>
#include <cstdio>
#include <iostream>
#include <vector>

#include "pih/core/bfloat16.h"
#include "pih/model/qwen3_cpu_oracle.h"
#include "pih/model/qwen3_gqa_oracle.h"
#include "pih/model/qwen3_sampler.h"

using pih::BFloat16;
using Vec = std::vector<BFloat16>;

static Vec read_bf16(std::size_t n) {
  Vec v(n);
  for (auto& x : v) {
    float f;
    std::cin >> f;
    x = BFloat16::FromFloat(f);
  }
  return v;
}

// y[m,n] = sum_k x[m,k] w[n,k], float accumulation in k order, one rounding to bf16
static Vec linear_bf16(const Vec& x, const Vec& w, std::size_t M, std::size_t N, std::size_t K) {
  Vec y(M * N);
  for (std::size_t m = 0; m < M; ++m)
    for (std::size_t n = 0; n < N; ++n) {
      float acc = 0.0F;
      for (std::size_t k = 0; k < K; ++k) acc += x[m * K + k].to_float() * w[n * K + k].to_float();
      y[m * N + n] = BFloat16::FromFloat(acc);
    }
  return y;
}

static void check(const pih::Status& s, const char* what) {
  if (!s.ok()) {
    std::fprintf(stderr, "oracle failed: %s\n", what);
    std::exit(1);
  }
}

int main() {
  std::size_t L, H, I, V, T;
  float eps;
  std::cin >> L >> H >> I >> V >> T >> eps;
  constexpr std::size_t heads = 16, kv_heads = 8, D = 128, Hq = heads * D, Hkv = kv_heads * D;
  std::vector<std::int64_t> ids(T), positions(T);
  for (std::size_t t = 0; t < T; ++t) {
    std::cin >> ids[t];
    positions[t] = static_cast<std::int64_t>(t);
  }
  Vec embed = read_bf16(V * H);
  Vec hidden(T * H), normed(T * H);
  check(pih::qwen_embedding_oracle(embed, V, H, ids, hidden), "embedding");
  std::vector<float> cosv(T * D / 2), sinv(T * D / 2);
  check(pih::qwen_rope_angles_oracle(positions, D, 1000000.0, cosv, sinv), "rope angles");
  std::vector<Vec> attention_outputs;
  for (std::size_t layer = 0; layer < L; ++layer) {
    Vec w_in = read_bf16(H), wq = read_bf16(Hq * H), wk = read_bf16(Hkv * H), wv = read_bf16(Hkv * H);
    Vec wqn = read_bf16(D), wkn = read_bf16(D), wo = read_bf16(H * Hq), w_post = read_bf16(H);
    Vec wg = read_bf16(I * H), wu = read_bf16(I * H), wd = read_bf16(H * I);
    check(pih::qwen_rms_norm_oracle(hidden, w_in, T, H, eps, normed), "input norm");
    Vec q = linear_bf16(normed, wq, T, Hq, H), k = linear_bf16(normed, wk, T, Hkv, H),
        v = linear_bf16(normed, wv, T, Hkv, H);
    Vec qn(q.size()), kn(k.size());
    check(pih::qwen_rms_norm_oracle(q, wqn, T * heads, D, eps, qn), "q norm");
    check(pih::qwen_rms_norm_oracle(k, wkn, T * kv_heads, D, eps, kn), "k norm");
    Vec qr(q.size()), kr(k.size());
    check(pih::qwen_rope_oracle(qn, cosv, sinv, T, heads, D, qr), "rope q");
    check(pih::qwen_rope_oracle(kn, cosv, sinv, T, kv_heads, D, kr), "rope k");
    Vec attn(T * Hq);
    check(pih::qwen_gqa_attention_oracle(qr, kr, v, static_cast<std::uint32_t>(T), static_cast<std::uint32_t>(T), 0,
                                         attn), "attention");
    attention_outputs.push_back(attn);
    Vec o = linear_bf16(attn, wo, T, H, Hq);
    Vec summed(T * H);
    check(pih::qwen_residual_add_oracle(hidden, o, summed), "residual 1");
    hidden = summed;
    check(pih::qwen_rms_norm_oracle(hidden, w_post, T, H, eps, normed), "post norm");
    Vec g = linear_bf16(normed, wg, T, I, H), u = linear_bf16(normed, wu, T, I, H), act(T * I);
    check(pih::qwen_silu_mul_oracle(g, u, act), "silu mul");
    Vec down = linear_bf16(act, wd, T, H, I);
    check(pih::qwen_residual_add_oracle(hidden, down, summed), "residual 2");
    hidden = summed;
  }
  Vec w_final = read_bf16(H);
  check(pih::qwen_rms_norm_oracle(hidden, w_final, T, H, eps, normed), "final norm");
  std::vector<float> logits(T * V);
  for (std::size_t t = 0; t < T; ++t)
    for (std::size_t n = 0; n < V; ++n) {
      float acc = 0.0F;
      for (std::size_t k = 0; k < H; ++k) acc += normed[t * H + k].to_float() * embed[n * H + k].to_float();
      logits[t * V + n] = acc;
    }
  std::printf("logits\n");
  for (float x : logits) std::printf("%.9g\n", x);
  for (std::size_t layer = 0; layer < L; ++layer) {
    std::printf("attention %zu\n", layer);
    // every 16th element keeps the file small
    for (std::size_t i = 0; i < attention_outputs[layer].size(); i += 16)
      std::printf("%.9g\n", attention_outputs[layer][i].to_float());
  }
  // the sampler on the last row of logits: greedy, temperature, top-k, top-p, suppression
  std::span<const float> row(logits.data() + (T - 1) * V, V);
  struct Case { float t, p; int k; std::uint64_t seed, ordinal; int suppressed; };
  const Case cases[] = {{0, 1, 0, 0, 0, -1}, {0.8F, 1, 0, 7, 0, -1}, {0.8F, 1, 0, 7, 5, -1}, {1.5F, 0.9F, 0, 123, 2, -1},
                        {1.0F, 1, 5, 9, 1, -1}, {2.0F, 0.5F, 40, 99, 11, -1}, {0, 1, 0, 0, 0, -2}, {1.0F, 1, 0, 4, 3, -2}};
  std::printf("samples\n");
  for (const auto& c : cases) {
    pih::Qwen3SamplingDescriptor d;
    d.mode = c.t == 0 ? pih::Qwen3SamplingMode::kGreedy : pih::Qwen3SamplingMode::kStochastic;
    d.temperature = c.t;
    d.top_p = c.p;
    if (c.k > 0) d.top_k = static_cast<std::uint32_t>(c.k);
    d.seed = c.seed;
    d.sample_ordinal = c.ordinal;
    if (c.suppressed == -2) {                      // suppress the greedy token
      std::uint32_t best = 0;
      for (std::uint32_t i = 1; i < V; ++i)
        if (row[i] > row[best]) best = i;
      d.suppressed_token_ids[0] = best;
      d.suppressed_token_count = 1;
    }
    auto r = pih::qwen3_sample_cpu(row, d);
    if (!r.ok()) {
      std::fprintf(stderr, "sampler failed\n");
      return 1;
    }
    std::printf("%u %.9g %u\n", r->token_id, r->selected_logprob, r->rng_word);
  }
  for (std::uint64_t o : {0ULL, 3ULL, 4ULL, 1000003ULL}) std::printf("philox %u\n", *pih::qwen3_philox_word(0, o));
  return 0;
}
