// Logit processing and sampling kernels (one CTA per row of the [n, vocab] fp32 logits / probs).
//
//   mlcb_logit_bias / mlcb_penalty / mlcb_bitmask   in-place logit edits
//   mlcb_softmax_temperature                        probs = softmax(logits / T); T ~ 0 -> uniform over argmax set
//   mlcb_argmax                                     greedy token straight from logits
//   mlcb_sample                                     fused top-k / top-p cutoff + renormalise + inverse-CDF sample
//   mlcb_renorm_top_p                               in-place renormalisation after the top-p cutoff
//   mlcb_take_probs                                 sampled-token prob and top-k (prob, id) lists for logprobs
//   mlcb_verify_tree                                speculative-decoding draft-tree verification
//
// Reference counterparts: compiler_pass/attach_softmax_with_temperature.py:43-274,
// compiler_pass/attach_logit_processor.py:72-285, op/top_p_pivot.py:11-335,
// compiler_pass/attach_sampler.py:69-343, op/batch_spec_verify.py:8-175; CPU semantics in
// cpp/serve/sampler/cpu_sampler.cc:35-163.
#include "common.cuh"

namespace mlcb {

constexpr int ROW_THREADS = 1024;

// ------------------------------------------------------------------ in-place logit edits
// entry i: logits[pos2seq[i], token[i]] += bias[i]
__global__ void logit_bias_kernel(float* logits, const int* pos2seq, const int* token,
                                  const float* bias, int n, int vocab) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int tk = token[i];
  if (tk < 0 || tk >= vocab) return;
  logits[static_cast<size_t>(pos2seq[i]) * vocab + tk] += bias[i];
}
// entry i: token token[i] appeared cnt[i] times in sequence row pos2seq[i];
// penalties[row] = (presence, frequency, repetition)
__global__ void penalty_kernel(float* logits, const int* pos2seq, const int* token, const int* cnt,
                               const float* penalties, int n, int vocab) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int row = pos2seq[i], tk = token[i];
  if (tk < 0 || tk >= vocab) return;
  float* p = logits + static_cast<size_t>(row) * vocab + tk;
  float v = *p;
  v -= penalties[row * 3 + 0] + cnt[i] * penalties[row * 3 + 1];
  const float rep = penalties[row * 3 + 2];
  v = v < 0.f ? v * rep : v / rep;
  *p = v;
}
// rows[r] selects the logits row; bitmask[r, ceil(V/32)]: bit 0 = token banned
__global__ void bitmask_kernel(float* logits, const int* rows, const int* bitmask, int vocab,
                               int words) {
  const int r = blockIdx.y;
  const int row = rows[r];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= vocab) return;
  const int bit = (bitmask[static_cast<size_t>(r) * words + (i >> 5)] >> (i & 31)) & 1;
  if (!bit) logits[static_cast<size_t>(row) * vocab + i] = -3.4028234663852886e38f;
}

// ------------------------------------------------------------------ softmax with temperature
__global__ void __launch_bounds__(ROW_THREADS)
softmax_temp_kernel(const float* __restrict__ logits, float* __restrict__ probs,
                    const float* __restrict__ temperature, int vocab, int active_vocab) {
  __shared__ float scratch[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * vocab;
  const float T = temperature[blockIdx.x];
  const int V = active_vocab > 0 && active_vocab < vocab ? active_vocab : vocab;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += ROW_THREADS) mx = fmaxf(mx, logits[base + i]);
  mx = block_max(mx, scratch);
  if (T < 1e-5f) {
    float c = 0.f;
    for (int i = threadIdx.x; i < V; i += ROW_THREADS) c += logits[base + i] == mx ? 1.f : 0.f;
    c = block_sum(c, scratch);
    for (int i = threadIdx.x; i < vocab; i += ROW_THREADS)
      probs[base + i] = (i < V && logits[base + i] == mx) ? 1.f / c : 0.f;
    return;
  }
  const float invT = 1.f / T;
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += ROW_THREADS) s += __expf((logits[base + i] - mx) * invT);
  s = block_sum(s, scratch);
  const float inv = 1.f / s;
  for (int i = threadIdx.x; i < vocab; i += ROW_THREADS)
    probs[base + i] = i < V ? __expf((logits[base + i] - mx) * invT) * inv : 0.f;
}

// ------------------------------------------------------------------ argmax (first index of the max)
__global__ void __launch_bounds__(ROW_THREADS)
argmax_kernel(const float* __restrict__ x, int* __restrict__ out, float* __restrict__ out_val,
              int vocab) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * vocab;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) {
    float v = x[base + i];
    if (v > best) {
      best = v;
      bi = i;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) {
    sv[w] = best;
    si[w] = bi;
  }
  __syncthreads();
  if (w == 0) {
    best = sv[lane];
    bi = si[lane];
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
      if (out_val) out_val[blockIdx.x] = best;
    }
  }
}

// ------------------------------------------------------------------ cutoff search (top-p / top-k)
// Returns (cutoff value, kept mass): kept = { p_i >= cutoff }, the smallest such set whose mass
// reaches top_p and whose size does not exceed top_k (ties at the cutoff are all kept).
// Search is a bisection over the float bit pattern (positive floats order like their bits).
__device__ float2 find_cutoff(const float* __restrict__ p, int vocab, float top_p, int top_k,
                              float* scratch) {
  float total = 0.f;
  for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) total += p[i];
  total = block_sum(total, scratch);
  if (top_p >= 1.f - 1e-5f && (top_k <= 0 || top_k >= vocab)) return make_float2(0.f, total);
  const float need = top_p >= 1.f - 1e-5f ? -1.f : top_p * total;
  uint32_t lo = 0u, hi = 0x3f800001u;  // invariant: set(lo) satisfies both constraints' "enough" side
  // we look for the largest cutoff c with mass(p >= c) >= need  AND then enforce count <= top_k by
  // raising the cutoff if needed (top-k wins over top-p when both are given). With top_p = 1 there is no mass
  // constraint and the cutoff stays at 0 (a search would climb to 1.0 and leave an empty set for top-k).
  // Other search forms were measured and are not used: evaluating 7 or 15 cutoffs per pass by comparisons in
  // registers, and a 256-bucket radix descent with shared-memory atomics, are both slower than this bisection
  // (a pass is bound by reading the row from L2 and has room for about ten operations per element).
  for (int it = 0; it < 31 && need > 0.f; ++it) {
    const uint32_t mid = lo + (hi - lo) / 2;
    if (mid == lo) break;
    const float c = __uint_as_float(mid);
    float mass = 0.f;
    for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) {
      float v = p[i];
      mass += v >= c ? v : 0.f;
    }
    mass = block_sum(mass, scratch);
    if (mass >= need) lo = mid; else hi = mid;
  }
  float cutoff = __uint_as_float(lo);
  if (top_k > 0 && top_k < vocab) {
    // smallest cutoff >= current with count(p >= cutoff) <= top_k
    uint32_t klo = lo, khi = 0x3f800001u;  // count(klo) may be > k, count(khi) = 0 <= k
    float cnt0 = 0.f;
    for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) cnt0 += p[i] >= cutoff ? 1.f : 0.f;
    cnt0 = block_sum(cnt0, scratch);
    if (cnt0 > top_k) {
      for (int it = 0; it < 31; ++it) {
        const uint32_t mid = klo + (khi - klo) / 2;
        if (mid == klo) break;
        const float c = __uint_as_float(mid);
        float cnt = 0.f;
        for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) cnt += p[i] >= c ? 1.f : 0.f;
        cnt = block_sum(cnt, scratch);
        if (cnt > top_k) klo = mid; else khi = mid;
      }
      cutoff = __uint_as_float(khi);
    }
  }
  float mass = 0.f;
  for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) {
    float v = p[i];
    mass += v >= cutoff ? v : 0.f;
  }
  mass = block_sum(mass, scratch);
  return make_float2(cutoff, mass);
}

// Inverse-CDF sample in index order over { p_i >= cutoff }, target = u * mass.
__device__ int sample_from(const float* __restrict__ p, int vocab, float cutoff, float target,
                           float* scratch, float* thread_sums, int* result) {
  const int chunk = (vocab + ROW_THREADS - 1) / ROW_THREADS;
  const int beg = threadIdx.x * chunk, end = min(vocab, beg + chunk);
  float local = 0.f;
  for (int i = beg; i < end; ++i) {
    float v = p[i];
    local += v >= cutoff ? v : 0.f;
  }
  thread_sums[threadIdx.x] = local;
  if (threadIdx.x == 0) *result = -1;
  __syncthreads();
  // warp 0 scans the 1024 partial sums (32 per lane)
  if (threadIdx.x < 32) {
    float run = 0.f;
    float vals[32];
    for (int k = 0; k < 32; ++k) {
      vals[k] = thread_sums[threadIdx.x * 32 + k];
      run += vals[k];
    }
    float incl = run;
    for (int o = 1; o < 32; o <<= 1) {
      float nb = __shfl_up_sync(0xffffffffu, incl, o);
      if ((threadIdx.x & 31) >= o) incl += nb;
    }
    float excl = incl - run;
    for (int k = 0; k < 32; ++k) {
      thread_sums[threadIdx.x * 32 + k] = excl;  // exclusive prefix of each thread's chunk
      excl += vals[k];
    }
  }
  __syncthreads();
  const float before = thread_sums[threadIdx.x];
  if (local > 0.f && before <= target && target < before + local) {
    float run = before;
    int pick = -1;
    for (int i = beg; i < end; ++i) {
      float v = p[i];
      if (v >= cutoff) {
        run += v;
        pick = i;
        if (run > target) break;
      }
    }
    *result = pick;
  }
  __syncthreads();
  if (*result < 0) {
    // numerical corner (target >= total mass): take the last kept element
    __shared__ int last_kept;
    if (threadIdx.x == 0) last_kept = -1;
    __syncthreads();
    int mine = -1;
    for (int i = beg; i < end; ++i)
      if (p[i] >= cutoff && p[i] > 0.f) mine = i;
    if (mine >= 0) atomicMax(&last_kept, mine);
    __syncthreads();
    if (threadIdx.x == 0) *result = last_kept < 0 ? 0 : last_kept;
    __syncthreads();
  }
  (void)scratch;
  return *result;
}

// probs row = sample_rows[r]; writes token and its renormalised probability.
__global__ void __launch_bounds__(ROW_THREADS)
sample_kernel(const float* __restrict__ probs, const int* __restrict__ sample_rows,
              const float* __restrict__ uniform, const float* __restrict__ top_p,
              const int* __restrict__ top_k, int* __restrict__ out_token,
              float* __restrict__ out_prob, int vocab) {
  __shared__ float scratch[32];
  __shared__ float thread_sums[ROW_THREADS];
  __shared__ int result;
  const int r = blockIdx.x;
  const int row = sample_rows ? sample_rows[r] : r;
  const float* p = probs + static_cast<size_t>(row) * vocab;
  const float tp = top_p ? top_p[r] : 1.f;
  const int tk = top_k ? top_k[r] : 0;
  if (tp <= 0.f) {
    // top_p == 0 means argmax (cpu_sampler.cc:52-70)
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += ROW_THREADS)
      if (p[i] > best) { best = p[i]; bi = i; }
    float bm = block_max(best, scratch);
    __shared__ int arg;
    if (threadIdx.x == 0) arg = 0x7fffffff;
    __syncthreads();
    if (best == bm) atomicMin(&arg, bi);
    __syncthreads();
    if (threadIdx.x == 0) { out_token[r] = arg; if (out_prob) out_prob[r] = 1.f; }
    return;
  }
  const float2 cm = find_cutoff(p, vocab, tp, tk, scratch);
  const int tok = sample_from(p, vocab, cm.x, uniform[r] * cm.y, scratch, thread_sums, &result);
  if (threadIdx.x == 0) {
    out_token[r] = tok;
    if (out_prob) out_prob[r] = cm.y > 0.f ? p[tok] / cm.y : 0.f;
  }
}

__global__ void __launch_bounds__(ROW_THREADS)
renorm_top_p_kernel(float* __restrict__ probs, const int* __restrict__ rows,
                    const float* __restrict__ top_p, int vocab) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* p = probs + static_cast<size_t>(row) * vocab;
  const float2 cm = find_cutoff(p, vocab, top_p[r], 0, scratch);
  const float inv = cm.y > 0.f ? 1.f / cm.y : 0.f;
  for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) {
    float v = p[i];
    p[i] = v >= cm.x ? v * inv : 0.f;
  }
}

// For each r: prob of token[r] in row rows[r], plus the k largest (prob, index) pairs.
__global__ void __launch_bounds__(ROW_THREADS)
take_probs_kernel(const float* __restrict__ probs, const int* __restrict__ rows,
                  const int* __restrict__ token, float* __restrict__ out_prob,
                  float* __restrict__ topk_prob, int* __restrict__ topk_idx, int k, int vocab) {
  __shared__ float scratch[32];
  __shared__ int chosen[32];
  __shared__ int arg;
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  const float* p = probs + static_cast<size_t>(row) * vocab;
  if (threadIdx.x == 0 && out_prob) out_prob[r] = p[token[r]];
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) {
      float v = p[i];
      if (v > best) {
        bool used = false;
        for (int q = 0; q < j; ++q) used |= chosen[q] == i;
        if (!used) { best = v; bi = i; }
      }
    }
    const float bm = block_max(best, scratch);
    if (threadIdx.x == 0) arg = 0x7fffffff;
    __syncthreads();
    if (best == bm) atomicMin(&arg, bi);
    __syncthreads();
    if (threadIdx.x == 0) {
      chosen[j] = arg;
      topk_prob[r * k + j] = bm;
      topk_idx[r * k + j] = arg == 0x7fffffff ? 0 : arg;
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ draft-tree verification
// One CTA per sequence. Node ids index rows of draft_probs / model_probs. parent_ptr[b] holds the
// root on entry and the last accepted node on exit; model_probs rows of nodes where a child was
// rejected are replaced by normalise(max(p - q, 0)) so the caller resamples from them.
__global__ void __launch_bounds__(ROW_THREADS)
verify_tree_kernel(const float* __restrict__ draft_probs, const int* __restrict__ draft_tokens,
                   float* __restrict__ model_probs, const int* __restrict__ first_child,
                   const int* __restrict__ next_sibling, const float* __restrict__ uniform,
                   int* __restrict__ parent_ptr, int vocab, int max_nodes) {
  __shared__ float scratch[32];
  const int b = blockIdx.x;
  int parent = parent_ptr[b];
  int child = first_child[parent];
  int guard = 0;
  while (child >= 0 && guard++ < max_nodes) {
    const int tok = draft_tokens[child];
    const float p = model_probs[static_cast<size_t>(parent) * vocab + tok];
    const float q = draft_probs[static_cast<size_t>(child) * vocab + tok];
    const float u = uniform[child];
    __syncthreads();
    // p > 0: a candidate the draft distribution gives no mass (a lower-ranked child of a draft tree under
    // greedy sampling has q == 0) must not pass on 0 >= 0
    if (p > 0.f && p >= u * q) {
      parent = child;
      child = first_child[child];
    } else {
      float* mp = model_probs + static_cast<size_t>(parent) * vocab;
      const float* dq = draft_probs + static_cast<size_t>(child) * vocab;
      float s = 0.f;
      for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) {
        float v = fmaxf(mp[i] - dq[i], 0.f);
        mp[i] = v;
        s += v;
      }
      s = block_sum(s, scratch);
      const float inv = s > 0.f ? 1.f / s : 0.f;
      for (int i = threadIdx.x; i < vocab; i += ROW_THREADS) mp[i] *= inv;
      __syncthreads();
      child = next_sibling[child];
    }
  }
  if (threadIdx.x == 0) parent_ptr[b] = parent;
}

}  // namespace mlcb

using namespace mlcb;

MLCB_API int mlcb_logit_bias(float* logits, const int* pos2seq, const int* token, const float* bias,
                             int n, int vocab, cudaStream_t stream) {
  if (n <= 0) return 0;
  logit_bias_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, pos2seq, token, bias, n, vocab);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
MLCB_API int mlcb_penalty(float* logits, const int* pos2seq, const int* token, const int* cnt,
                          const float* penalties, int n, int vocab, cudaStream_t stream) {
  if (n <= 0) return 0;
  penalty_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, pos2seq, token, cnt, penalties, n, vocab);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
MLCB_API int mlcb_bitmask(float* logits, const int* rows, const int* bitmask, int nrows, int vocab,
                          cudaStream_t stream) {
  if (nrows <= 0) return 0;
  dim3 grid((vocab + 255) / 256, nrows);
  bitmask_kernel<<<grid, 256, 0, stream>>>(logits, rows, bitmask, vocab, (vocab + 31) / 32);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
MLCB_API int mlcb_softmax_temperature(const float* logits, float* probs, const float* temperature,
                                      int n, int vocab, int active_vocab, cudaStream_t stream) {
  if (n <= 0) return 0;
  softmax_temp_kernel<<<n, ROW_THREADS, 0, stream>>>(logits, probs, temperature, vocab, active_vocab);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
MLCB_API int mlcb_argmax(const float* x, int* out, float* out_val, int n, int vocab,
                         cudaStream_t stream) {
  if (n <= 0) return 0;
  argmax_kernel<<<n, ROW_THREADS, 0, stream>>>(x, out, out_val, vocab);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
MLCB_API int mlcb_sample(const float* probs, const int* sample_rows, const float* uniform,
                         const float* top_p, const int* top_k, int* out_token, float* out_prob, int n,
                         int vocab, cudaStream_t stream) {
  if (n <= 0) return 0;
  sample_kernel<<<n, ROW_THREADS, 0, stream>>>(probs, sample_rows, uniform, top_p, top_k, out_token,
                                               out_prob, vocab);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
MLCB_API int mlcb_renorm_top_p(float* probs, const int* rows, const float* top_p, int n, int vocab,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  renorm_top_p_kernel<<<n, ROW_THREADS, 0, stream>>>(probs, rows, top_p, vocab);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
MLCB_API int mlcb_take_probs(const float* probs, const int* rows, const int* token, float* out_prob,
                             float* topk_prob, int* topk_idx, int n, int k, int vocab,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  if (k > 32) return -1;
  take_probs_kernel<<<n, ROW_THREADS, 0, stream>>>(probs, rows, token, out_prob, topk_prob, topk_idx,
                                                   k, vocab);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
MLCB_API int mlcb_verify_tree(const float* draft_probs, const int* draft_tokens, float* model_probs,
                              const int* first_child, const int* next_sibling, const float* uniform,
                              int* parent_ptr, int nbatch, int vocab, int max_nodes,
                              cudaStream_t stream) {
  if (nbatch <= 0) return 0;
  verify_tree_kernel<<<nbatch, ROW_THREADS, 0, stream>>>(draft_probs, draft_tokens, model_probs,
                                                         first_child, next_sibling, uniform,
                                                         parent_ptr, vocab, max_nodes);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
