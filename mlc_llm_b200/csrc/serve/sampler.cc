#include "sampler.h"

#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace mlcb {

namespace {
// Candidates with prob >= cutoff, sorted descending. Returns false when their mass cannot reach
// top_p (the caller then retries with a lower cutoff).
bool CollectCandidates(const float* prob, int64_t n, double top_p, float cutoff,
                       std::vector<std::pair<float, int64_t>>* cand) {
  cand->clear();
  double mass = 0;
  for (int64_t i = 0; i < n; ++i)
    if (prob[i] >= cutoff && prob[i] > 0) {
      cand->emplace_back(prob[i], i);
      mass += prob[i];
    }
  if (cand->empty()) return false;
  std::sort(cand->begin(), cand->end(), [](const auto& a, const auto& b) {
    return a.first > b.first || (a.first == b.first && a.second < b.second);
  });
  return cutoff == 0.f || mass >= top_p;
}
}  // namespace

std::pair<int64_t, float> SampleTopPFromProb(const float* prob, int64_t n, double top_p, double uniform) {
  if (top_p <= 0) {
    int64_t arg = 0;
    for (int64_t i = 1; i < n; ++i)
      if (prob[i] > prob[arg]) arg = i;
    return {arg, 1.0f};
  }
  if (top_p >= 1.0 - 1e-5) {
    double cum = 0;
    int64_t last = 0;
    for (int64_t i = 0; i < n; ++i) {
      if (prob[i] > 0) last = i;
      cum += prob[i];
      if (cum >= uniform && prob[i] > 0) return {i, prob[i]};
    }
    return {last, prob[last]};
  }
  std::vector<std::pair<float, int64_t>> cand;
  // elements below top_p / 1024 are rarely needed: at most ~1024 / top_p candidates survive
  if (!CollectCandidates(prob, n, top_p, static_cast<float>(top_p / 1024.0), &cand))
    CollectCandidates(prob, n, top_p, 0.f, &cand);
  if (cand.empty()) throw std::runtime_error("probability row has no positive entry (NaN?)");
  // keep the shortest prefix whose mass reaches top_p
  double kept = 0;
  size_t m = 0;
  while (m < cand.size() && kept < top_p) kept += cand[m++].first;
  double cum = 0;
  for (size_t i = 0; i < m; ++i) {
    cum += cand[i].first;
    if (uniform < cum / kept) return {cand[i].second, cand[i].first};
  }
  return {cand[m - 1].second, cand[m - 1].first};
}

void RenormalizeProbByTopP(float* prob, int64_t n, double top_p) {
  if (top_p >= 1.0 - 1e-5) return;
  std::vector<std::pair<float, int64_t>> cand;
  if (!CollectCandidates(prob, n, top_p, static_cast<float>(top_p / 1024.0), &cand))
    CollectCandidates(prob, n, top_p, 0.f, &cand);
  if (cand.empty()) return;
  double kept = 0;
  size_t m = 0;
  while (m < cand.size() && kept < top_p) kept += cand[m++].first;
  if (top_p <= 0) {
    m = 1;
    kept = cand[0].first;
  }
  const float cutoff = cand[m - 1].first;
  // ties at the cutoff value are all kept, as in the GPU kernel
  double mass = 0;
  for (int64_t i = 0; i < n; ++i)
    if (prob[i] >= cutoff) mass += prob[i];
  for (int64_t i = 0; i < n; ++i) prob[i] = prob[i] >= cutoff ? static_cast<float>(prob[i] / mass) : 0.f;
}

std::pair<int, int64_t> VerifyDraftChain(float* model_probs, const float* draft_probs,
                                         const std::vector<int32_t>& draft_tokens,
                                         const std::vector<double>& uniforms, double final_uniform,
                                         int64_t vocab) {
  const int k = static_cast<int>(draft_tokens.size());
  int accepted = 0;
  for (; accepted < k; ++accepted) {
    float* p = model_probs + static_cast<int64_t>(accepted) * vocab;
    const float* q = draft_probs + static_cast<int64_t>(accepted) * vocab;
    const int32_t tok = draft_tokens[accepted];
    if (p[tok] >= uniforms[accepted] * q[tok]) continue;
    double s = 0;
    for (int64_t i = 0; i < vocab; ++i) {
      p[i] = std::max(p[i] - q[i], 0.f);
      s += p[i];
    }
    if (s > 0)
      for (int64_t i = 0; i < vocab; ++i) p[i] = static_cast<float>(p[i] / s);
    break;
  }
  auto r = SampleTopPFromProb(model_probs + static_cast<int64_t>(accepted) * vocab, vocab, 1.0, final_uniform);
  return {accepted, r.first};
}

}  // namespace mlcb
