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

}  // extern "C"
