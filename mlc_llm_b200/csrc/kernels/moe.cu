// Mixture-of-experts routing kernels: gate top-k (+softmax), expert-major permutation of the
// (token, slot) pairs, and the weighted combine of expert outputs. The expert matmuls themselves are
// the grouped mode of the tcgen05 GEMM (gemm_tcgen05.cu).
//
// Reference counterparts: op/moe_misc.py:63-235 (gating top-k / softmax-top-k), :371-605 (cumsum,
// indices, indptr, scatter_output), :14-32 (moe_sum); call site model/mixtral/mixtral_model.py:64-117.
#include "common.cuh"

namespace mlcb {

// mode 0: softmax over all experts, take top-k, optionally renormalise the k weights to sum 1
//         (equals "top-k of the raw logits then softmax over the k" when renormalised);
// mode 1: top-k over raw scores, weights = raw scores (caller post-processes).
template <typename T>
__global__ void moe_router_kernel(const T* __restrict__ logits, float* __restrict__ weights,
                                  int* __restrict__ experts, int tokens, int E, int k, int mode, int renorm) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const T* row = logits + static_cast<size_t>(t) * E;
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, Cvt<T>::to_f(row[e]));
  float denom = 0.f;
  if (mode == 0)
    for (int e = 0; e < E; ++e) denom += __expf(Cvt<T>::to_f(row[e]) - mx);
  float topv[8];
  int topi[8];
  for (int j = 0; j < k; ++j) {
    topv[j] = -INFINITY;
    topi[j] = -1;
  }
  for (int e = 0; e < E; ++e) {
    const float v = Cvt<T>::to_f(row[e]);
    // insertion into the descending list; ties keep the lower expert index first
    int pos = k;
    while (pos > 0 && v > topv[pos - 1]) --pos;
    if (pos < k) {
      for (int j = k - 1; j > pos; --j) {
        topv[j] = topv[j - 1];
        topi[j] = topi[j - 1];
      }
      topv[pos] = v;
      topi[pos] = e;
    }
  }
  float sum = 0.f;
  for (int j = 0; j < k; ++j) {
    if (mode == 0) topv[j] = __expf(topv[j] - mx) / denom;
    sum += topv[j];
  }
  for (int j = 0; j < k; ++j) {
    weights[static_cast<size_t>(t) * k + j] = (mode == 0 && renorm) ? topv[j] / sum : topv[j];
    experts[static_cast<size_t>(t) * k + j] = topi[j];
  }
}

// Group-limited routing (DeepSeek-V2; reference: python/mlc_llm/op/moe_misc.py:238-368): softmax over all
// experts, keep the `topk_group` expert groups whose best expert scores highest, then the top k experts inside
// the kept groups. One thread per token; ties go to the lower index, as in the plain router.
template <typename T>
__global__ void moe_router_grouped_kernel(const T* __restrict__ logits, float* __restrict__ weights,
                                          int* __restrict__ experts, int tokens, int E, int k, int n_group,
                                          int topk_group, int renorm) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const T* row = logits + static_cast<size_t>(t) * E;
  const int gs = E / n_group;
  float gbest[32];
  float mx = -INFINITY;
  for (int g = 0; g < n_group; ++g) {
    float b = -INFINITY;
    for (int e = g * gs; e < (g + 1) * gs; ++e) b = fmaxf(b, Cvt<T>::to_f(row[e]));
    gbest[g] = b;
    mx = fmaxf(mx, b);
  }
  float denom = 0.f;
  for (int e = 0; e < E; ++e) denom += __expf(Cvt<T>::to_f(row[e]) - mx);
  unsigned keep = 0u;
  for (int j = 0; j < topk_group; ++j) {
    int best = -1;
    float bv = -INFINITY;
    for (int g = 0; g < n_group; ++g)
      if (!((keep >> g) & 1u) && (best < 0 || gbest[g] > bv)) {
        best = g;
        bv = gbest[g];
      }
    keep |= 1u << best;
  }
  float topv[8];
  int topi[8];
  for (int j = 0; j < k; ++j) {
    topv[j] = -INFINITY;
    topi[j] = -1;
  }
  for (int g = 0; g < n_group; ++g) {
    if (!((keep >> g) & 1u)) continue;
    for (int e = g * gs; e < (g + 1) * gs; ++e) {
      const float v = Cvt<T>::to_f(row[e]);
      int pos = k;
      while (pos > 0 && v > topv[pos - 1]) --pos;
      if (pos < k) {
        for (int j = k - 1; j > pos; --j) {
          topv[j] = topv[j - 1];
          topi[j] = topi[j - 1];
        }
        topv[pos] = v;
        topi[pos] = e;
      }
    }
  }
  float sum = 0.f;
  for (int j = 0; j < k; ++j) {
    topv[j] = topi[j] >= 0 ? __expf(topv[j] - mx) / denom : 0.f;
    sum += topv[j];
  }
  for (int j = 0; j < k; ++j) {
    weights[static_cast<size_t>(t) * k + j] = renorm ? topv[j] / sum : topv[j];
    experts[static_cast<size_t>(t) * k + j] = topi[j] >= 0 ? topi[j] : 0;
  }
}

// Single-CTA permutation: counts per expert, exclusive scan, then a slot for every (token, j) pair.
// offsets [E + 1]; sorted_pos [n] = row of pair i in expert-major order; src_token [n] = token of row.
__global__ void __launch_bounds__(1024)
moe_permute_kernel(const int* __restrict__ experts, int n, int k, int E, int* __restrict__ offsets,
                   int* __restrict__ sorted_pos, int* __restrict__ src_token) {
  extern __shared__ int sh[];  // counts[E], cursor[E]
  int* counts = sh;
  int* cursor = sh + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = experts[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      run += counts[e];
    }
    offsets[E] = run;
  }
  __syncthreads();
  // deterministic order inside an expert: pairs are placed in index order by one warp per expert
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    int base = cursor[e];
    for (int i0 = 0; i0 < n; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < n && experts[i] == e;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int pos = base + __popc(m & ((1u << lane) - 1));
        sorted_pos[i] = pos;
        src_token[pos] = i / k;
      }
      base += __popc(m);
    }
  }
}

// The same permutation with the pairs split over the 32 warps of the CTA (the form above walks every pair
// once per expert with one warp, which costs a chain of dependent loads when there are few experts).
// Pass 1 counts per (expert, warp) with match_any, a scan over (expert, warp) gives each warp its first
// row inside every expert, pass 2 places the pairs: pairs of one expert stay in index order.
__global__ void __launch_bounds__(1024)
moe_permute_split_kernel(const int* __restrict__ experts, int n, int k, int E, int* __restrict__ offsets,
                         int* __restrict__ sorted_pos, int* __restrict__ src_token) {
  extern __shared__ int sh[];  // cnt[E][32], total[E]
  int* cnt = sh;
  int* total = sh + E * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < E * 32; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  const int per_warp = ((n + 31) / 32 + 31) / 32 * 32;  // pairs of one warp, a multiple of 32
  const int begin = warp * per_warp, end = min(n, begin + per_warp);
  const unsigned lt = (1u << lane) - 1;
  for (int i0 = begin; i0 < end; i0 += 32) {
    const int i = i0 + lane;
    int e = i < end ? experts[i] : -1;
    if (e < 0 || e >= E) e = -1;
    const unsigned m = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && (m & lt) == 0) cnt[e * 32 + warp] += __popc(m);
    __syncwarp();
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = cnt[e * 32 + w];
      cnt[e * 32 + w] = run;  // first row of warp w inside expert e, relative to the expert
      run += c;
    }
    total[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = total[e];
      offsets[e] = run;
      total[e] = run;
      run += c;
    }
    offsets[E] = run;
  }
  __syncthreads();
  for (int i0 = begin; i0 < end; i0 += 32) {
    const int i = i0 + lane;
    int e = i < end ? experts[i] : -1;
    if (e < 0 || e >= E) e = -1;
    const unsigned m = __match_any_sync(0xffffffffu, e);
    if (e >= 0) {
      const int pos = total[e] + cnt[e * 32 + warp] + __popc(m & lt);
      sorted_pos[i] = pos;
      src_token[pos] = i / k;
    }
    __syncwarp();
    if (e >= 0 && (m & lt) == 0) cnt[e * 32 + warp] += __popc(m);
    __syncwarp();
  }
}

// out[t, :] = sum_j w[t, j] * y[sorted_pos[t * k + j], :]  (+ add[t, :] if given)
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const float* __restrict__ w,
                                   const int* __restrict__ sorted_pos, const T* __restrict__ add,
                                   T* __restrict__ out, int hidden, int k) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = 0; j < k; ++j) {
      const int r = sorted_pos[t * k + j];
      const float wj = w[t * k + j];
      const uint4 v = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(r) * hidden + c);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += wj * Cvt<T>::to_f(e[i]);
    }
    if (add) {
      const uint4 v = *reinterpret_cast<const uint4*>(add + static_cast<size_t>(t) * hidden + c);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += Cvt<T>::to_f(e[i]);
    }
    T o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = Cvt<T>::from_f(acc[i]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden + c) = *reinterpret_cast<uint4*>(o);
  }
}

}  // namespace mlcb

using namespace mlcb;

MLCB_API int mlcb_moe_router(const void* logits, float* weights, int* experts, int tokens, int E, int k,
                             int mode, int renorm, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (k > 8 || k < 1 || E < k) return -1;
  const int blocks = (tokens + 127) / 128;
  if (dtype == 0)
    moe_router_kernel<__half><<<blocks, 128, 0, stream>>>((const __half*)logits, weights, experts, tokens, E, k, mode, renorm);
  else if (dtype == 1)
    moe_router_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>((const __nv_bfloat16*)logits, weights, experts, tokens, E, k, mode, renorm);
  else
    moe_router_kernel<float><<<blocks, 128, 0, stream>>>((const float*)logits, weights, experts, tokens, E, k, mode, renorm);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_moe_router_grouped(const void* logits, float* weights, int* experts, int tokens, int E, int k,
                                     int n_group, int topk_group, int renorm, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (k > 8 || k < 1 || n_group < 1 || n_group > 32 || E % n_group || topk_group < 1 || topk_group > n_group ||
      topk_group * (E / n_group) < k)
    return -1;
  const int blocks = (tokens + 127) / 128;
  if (dtype == 0)
    moe_router_grouped_kernel<__half><<<blocks, 128, 0, stream>>>((const __half*)logits, weights, experts, tokens, E, k, n_group, topk_group, renorm);
  else if (dtype == 1)
    moe_router_grouped_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>((const __nv_bfloat16*)logits, weights, experts, tokens, E, k, n_group, topk_group, renorm);
  else
    moe_router_grouped_kernel<float><<<blocks, 128, 0, stream>>>((const float*)logits, weights, experts, tokens, E, k, n_group, topk_group, renorm);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_moe_permute(const int* experts, int n, int k, int E, int* offsets, int* sorted_pos,
                              int* src_token, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E > 4096) return -1;
  if (E <= 256)
    moe_permute_split_kernel<<<1, 1024, 33 * E * sizeof(int), stream>>>(experts, n, k, E, offsets, sorted_pos, src_token);
  else
    moe_permute_kernel<<<1, 1024, 2 * E * sizeof(int), stream>>>(experts, n, k, E, offsets, sorted_pos, src_token);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_moe_combine(const void* y, const float* w, const int* sorted_pos, const void* add, void* out,
                              int tokens, int hidden, int k, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return -1;
  int threads = hidden / 8;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  if (dtype == 0)
    moe_combine_kernel<__half><<<tokens, threads, 0, stream>>>((const __half*)y, w, sorted_pos, (const __half*)add, (__half*)out, hidden, k);
  else
    moe_combine_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)y, w, sorted_pos, (const __nv_bfloat16*)add, (__nv_bfloat16*)out, hidden, k);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
