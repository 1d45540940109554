// Host-side sampling around the decoder step: repetition penalty, temperature / top-k /
// top-p sampling and the 64-token recent window.  Replaces apply_repetition_penalty and
// sample_logits (src/llm/decoder.rs:878-1020) and push_recent_window (:862-874).  The
// reference draws from rand::random::<f32>(); here the uniform number is an argument (or comes
// from the decoder's own xorshift state), so a result can be reproduced.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <unordered_set>
#include <utility>
#include <vector>

#include "../../include/torchburn_b200.h"

namespace tb {
tb_status fail(tb_status code, const char* fmt, ...);
}
using tb::fail;

extern "C" {

tb_status tb_apply_repetition_penalty(float* logits, int64_t vocab, const int64_t* recent, int64_t n_recent,
                                      float penalty) {
  if (!logits || vocab < 0 || (n_recent > 0 && !recent)) return fail(TB_ERR_ARG, "tb_apply_repetition_penalty: bad arguments");
  if (penalty <= 1.0f || n_recent <= 0) return TB_OK;  // decoder.rs:879-881
  std::unordered_set<int64_t> seen;
  for (int64_t i = 0; i < n_recent; ++i) {
    const int64_t t = recent[i];
    if (t < 0 || t >= vocab || !seen.insert(t).second) continue;  // each token once
    const float l = logits[t];
    logits[t] = l > 0.0f ? l / penalty : l * penalty;
  }
  return TB_OK;
}

tb_status tb_sample_logits(const float* logits, int64_t vocab, float temperature, int64_t top_k, float top_p,
                           float uniform01, int64_t* token) {
  if (!token) return fail(TB_ERR_ARG, "tb_sample_logits: null out");
  *token = 0;
  if (vocab == 0) return TB_OK;  // decoder.rs:911-913
  if (!logits || vocab < 0) return fail(TB_ERR_ARG, "tb_sample_logits: bad arguments");
  if (!std::isfinite(temperature) || temperature <= 0.0f || top_k == 1) {
    int64_t best = 0;
    float bv = logits[0];
    for (int64_t i = 1; i < vocab; ++i)
      if (logits[i] > bv) { bv = logits[i]; best = i; }
    *token = best;
    return TB_OK;
  }
  int64_t k = top_k < vocab ? top_k : vocab;
  if (k < 1) k = 1;
  auto clean = [](float v) { return std::isfinite(v) ? v : -INFINITY; };
  std::vector<std::pair<int64_t, float>> top;
  top.reserve((size_t)k);
  if (k >= vocab) {
    for (int64_t i = 0; i < vocab; ++i) top.emplace_back(i, clean(logits[i]));
  } else if (k > 1024) {
    std::vector<std::pair<int64_t, float>> all((size_t)vocab);
    for (int64_t i = 0; i < vocab; ++i) all[(size_t)i] = {i, clean(logits[i])};
    std::nth_element(all.begin(), all.begin() + k, all.end(), [](const auto& a, const auto& b) { return a.second > b.second; });
    top.assign(all.begin(), all.begin() + k);
  } else {
    // running top-k with replacement of the current minimum (decoder.rs:948-975)
    float min_val = -INFINITY;
    size_t min_pos = 0;
    for (int64_t i = 0; i < vocab; ++i) {
      const float val = clean(logits[i]);
      if ((int64_t)top.size() < k) {
        top.emplace_back(i, val);
        if (val < min_val || top.size() == 1) { min_val = val; min_pos = top.size() - 1; }
      } else if (val > min_val) {
        top[min_pos] = {i, val};
        float nm = top[0].second;
        size_t np = 0;
        for (size_t j = 0; j < top.size(); ++j)
          if (top[j].second < nm) { nm = top[j].second; np = j; }
        min_val = nm;
        min_pos = np;
      }
    }
  }
  float max_logit = -INFINITY;
  for (auto& it : top) max_logit = std::max(max_logit, it.second);
  const float inv_temp = 1.0f / temperature;
  for (auto& it : top) it.second = std::exp((it.second - max_logit) * inv_temp);
  float pre_sum = 0.f;
  for (auto& it : top) pre_sum += it.second;
  size_t kept_end = top.size();
  if (top_p > 0.0f && top_p < 1.0f && kept_end > 1 && pre_sum > 0.0f) {
    const float inv_sum = 1.0f / pre_sum;
    std::stable_sort(top.begin(), top.end(), [](const auto& a, const auto& b) { return a.second > b.second; });
    float cum = 0.f;
    for (size_t i = 0; i < top.size(); ++i) {
      if (cum > top_p) { kept_end = i; break; }
      cum += top[i].second * inv_sum;
    }
  }
  float kept_sum = 0.f;
  for (size_t i = 0; i < kept_end; ++i) kept_sum += top[i].second;
  const float r = uniform01 * kept_sum;
  float accum = 0.f;
  for (size_t i = 0; i < kept_end; ++i) {
    accum += top[i].second;
    if (accum >= r) { *token = top[i].first; return TB_OK; }
  }
  *token = top[0].first;
  return TB_OK;
}

int64_t tb_push_recent_window(int64_t* recent, int64_t n_recent, int64_t token) {
  if (!recent || n_recent < 0) return 0;
  constexpr int64_t kWindow = 64;  // RECENT_WINDOW, decoder.rs:859
  if (n_recent >= kWindow) {
    const int64_t drop = n_recent - kWindow + 1;
    memmove(recent, recent + drop, sizeof(int64_t) * (size_t)(n_recent - drop));
    n_recent -= drop;
  }
  recent[n_recent] = token;
  return n_recent + 1;
}


// Leviathan acceptance over the target logits of the K verified positions,
// src/llm/decoder.rs:583-727 (speculative_accept after its verify loop).  The reference seeds a
// splitmix64 generator from the clock; here the caller owns the state, the stream of draws is
// the same function of it.
static double splitmix_u01(uint64_t* st) {
  *st += 0x9E3779B97F4A7C15ull;
  uint64_t z = *st;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (double)(z >> 11) / (double)(1ull << 53);
}

static void softmax_row(const float* logits, int64_t v, float temp, std::vector<float>& out) {
  const float t = (std::isfinite(temp) && temp > 0.0f) ? temp : 1.0f;
  float m = -INFINITY;
  for (int64_t j = 0; j < v; ++j) m = std::max(m, std::isfinite(logits[j]) ? logits[j] : -INFINITY);
  out.resize((size_t)v);
  float s = 0.f;
  for (int64_t j = 0; j < v; ++j) {
    const float x = std::isfinite(logits[j]) ? logits[j] : -INFINITY;
    out[(size_t)j] = std::exp((x - m) / t);
    s += out[(size_t)j];
  }
  const float inv = 1.0f / std::max(s, 1e-30f);
  for (int64_t j = 0; j < v; ++j) out[(size_t)j] *= inv;
}

tb_status tb_speculative_accept_rows(const float* target_logits, int64_t vocab, const int64_t* draft_tokens,
                                     int64_t k, const float* draft_probs, float temperature, float top_p,
                                     uint64_t* rng_state, int64_t* accepted, int64_t* bonus) {
  if (!accepted || !bonus || !rng_state || vocab < 1 || k < 0)
    return fail(TB_ERR_ARG, "tb_speculative_accept_rows: bad arguments");
  *accepted = 0;
  *bonus = vocab - 1;
  if (k == 0) return TB_OK;  // decoder.rs:594-596
  if (!target_logits || !draft_tokens || !draft_probs) return fail(TB_ERR_ARG, "tb_speculative_accept_rows: null operand");
  if (*rng_state == 0) *rng_state = 1;  // decoder.rs:642 (.max(1))
  const int64_t v = vocab;
  std::vector<float> tp;
  for (int64_t i = 0; i < k; ++i) {
    softmax_row(target_logits + i * v, v, temperature, tp);
    const float* dp = draft_probs + i * v;
    const int64_t tok = std::min<int64_t>(std::max<int64_t>(draft_tokens[i], 0), v - 1);
    const float p_target = tp[(size_t)tok];
    const float p_draft = std::max(dp[tok], 0.0f);
    const float accept = std::min(p_target / (p_draft + 1e-12f), 1.0f);
    if (splitmix_u01(rng_state) <= (double)accept) {
      ++*accepted;
      continue;
    }
    // rejected: resample from max(0, p_target - p_draft)
    float s = 0.f;
    for (int64_t j = 0; j < v; ++j) s += std::max(tp[(size_t)j] - dp[j], 0.0f);
    if (s > 1e-12f) {
      const float r = (float)splitmix_u01(rng_state) * s;
      float acc = 0.f;
      int64_t b = v - 1;
      for (int64_t j = 0; j < v; ++j) {
        acc += std::max(tp[(size_t)j] - dp[j], 0.0f);
        if (acc >= r) { b = j; break; }
      }
      *bonus = b;
    } else {
      int64_t b = 0;  // max_by keeps the last maximum
      for (int64_t j = 0; j < v; ++j)
        if (!(tp[(size_t)j] < tp[(size_t)b])) b = j;
      *bonus = b;
    }
    return TB_OK;
  }
  // all accepted: the bonus token comes from the last verified row, with the nucleus cut
  softmax_row(target_logits + (k - 1) * v, v, temperature, tp);
  std::vector<int64_t> idx((size_t)v);
  for (int64_t j = 0; j < v; ++j) idx[(size_t)j] = j;
  std::stable_sort(idx.begin(), idx.end(), [&](int64_t a, int64_t b) { return tp[(size_t)a] > tp[(size_t)b]; });
  int64_t kept = v;
  if (top_p > 0.0f && top_p < 1.0f) {
    float cum = 0.f;
    for (int64_t i = 0; i < v; ++i) {
      if (cum > top_p) { kept = i; break; }
      cum += tp[(size_t)idx[(size_t)i]];
    }
    kept = std::max<int64_t>(kept, 1);
  }
  float mass = 0.f;
  for (int64_t i = 0; i < kept; ++i) mass += tp[(size_t)idx[(size_t)i]];
  const float r = (float)splitmix_u01(rng_state) * std::max(mass, 1e-30f);
  float acc = 0.f;
  int64_t b = idx[(size_t)(kept - 1)];
  for (int64_t i = 0; i < kept; ++i) {
    acc += tp[(size_t)idx[(size_t)i]];
    if (acc >= r) { b = idx[(size_t)i]; break; }
  }
  *bonus = b;
  return TB_OK;
}
}  // extern "C"
