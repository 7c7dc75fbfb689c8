// CPU sampling primitives: top-p sampling from a probability row, top-p renormalisation, and the
// chain form of speculative-decoding verification. They define the sampling semantics the GPU
// kernels are tested against and serve the CPU execution path.
//
// Behavioural counterpart: cpp/serve/sampler/cpu_sampler.cc:35-163 (SampleTopPFromProb),
// :172-260 (RenormalizeProbByTopP), :402-503 (draft verification: accept when p >= u*q, otherwise
// resample from normalise(max(p - q, 0))).
#pragma once
#include <cstdint>
#include <utility>
#include <vector>

namespace mlcb {

// Returns (token, probability of that token in `prob`).
std::pair<int64_t, float> SampleTopPFromProb(const float* prob, int64_t n, double top_p, double uniform);
// Keeps the smallest set of largest probabilities whose mass reaches top_p and renormalises.
void RenormalizeProbByTopP(float* prob, int64_t n, double top_p);
// model_probs: [k + 1, vocab] (row i = distribution after i accepted drafts; rows may be modified),
// draft_probs: [k, vocab]. Returns (number of accepted drafts, token sampled after them).
std::pair<int, int64_t> VerifyDraftChain(float* model_probs, const float* draft_probs,
                                         const std::vector<int32_t>& draft_tokens,
                                         const std::vector<double>& uniforms, double final_uniform,
                                         int64_t vocab);

}  // namespace mlcb
