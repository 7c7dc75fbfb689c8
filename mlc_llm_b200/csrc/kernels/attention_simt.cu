// Generic paged-KV attention on CUDA cores. It covers every head dimension that is a multiple of 32
// (up to 256), sliding windows with attention sinks, token-tree masks for speculative verification,
// soft-capping, and it can return the log-sum-exp for merging partial results. It is the fallback for
// shapes the tensor-core attention kernel does not take and the on-device oracle for it.
//
// Semantics follow the reference's PagedKVCache attention (nn/kv_cache.py:16-93 and the call site
// model/llama/llama_model.py:157-170): softmax(q.k^T * sm_scale) v over the pages of the sequence,
// causal inside the appended chunk.
#include "common.cuh"

namespace mlcb {

struct AttnArgs {
  const void* q;          // [T, hq, d], row stride q_stride elements
  const void* kv_pages;   // [num_pages, 2, hkv, page, d]
  void* out;              // [T, hq, d] dense
  float* lse;             // [T, hq] or null
  const int* q_seq;       // [T] batch slot of each query token
  const int* q_kvlen;     // [T] number of kv positions visible through the causal rule
  const int* q_kvstart;   // [T] first visible non-sink position (sliding window), may be null
  const unsigned long long* tree_mask;  // [T] or null: bit j = may attend kv position q_kvlen[t]+j
  const int* page_indptr; // [B+1]
  const int* page_indices;
  int q_stride, hq, hkv, d, page, sink;
  float sm_scale, softcap;
};

template <typename T>
__global__ void __launch_bounds__(128) attn_simt_kernel(const AttnArgs a) {
  const int t = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dpl = a.d / 32;  // elements per lane (<= 8)
  const int hk = h / (a.hq / a.hkv);
  const int b = a.q_seq[t];
  const int causal_len = a.q_kvlen[t];
  const int start = a.q_kvstart ? a.q_kvstart[t] : 0;
  const unsigned long long tmask = a.tree_mask ? a.tree_mask[t] : 0ull;
  const int extra = a.tree_mask ? 64 - __clzll(tmask | 1ull) : 0;
  const int total = causal_len + (tmask ? extra : 0);
  const int* pages = a.page_indices + a.page_indptr[b];

  const T* qp = reinterpret_cast<const T*>(a.q) + static_cast<size_t>(t) * a.q_stride + h * a.d;
  float qv[8], acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    qv[i] = i < dpl ? Cvt<T>::to_f(qp[lane + 32 * i]) * a.sm_scale : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const T* kvbase = reinterpret_cast<const T*>(a.kv_pages);
  for (int j = warp; j < total; j += 4) {
    bool visible = j < causal_len ? (j < a.sink || j >= start) : ((tmask >> (j - causal_len)) & 1ull);
    if (!visible) continue;
    const int pg = pages[j / a.page], off = j % a.page;
    const T* kp = kvbase + ((static_cast<size_t>(pg) * 2 * a.hkv + hk) * a.page + off) * a.d;
    const T* vp = kp + static_cast<size_t>(a.hkv) * a.page * a.d;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < dpl) s += qv[i] * Cvt<T>::to_f(kp[lane + 32 * i]);
    s = warp_sum(s);
    if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
    const float mn = fmaxf(m, s);
    const float corr = __expf(m - mn), pexp = __expf(s - mn);
    l = l * corr + pexp;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < dpl) acc[i] = acc[i] * corr + pexp * Cvt<T>::to_f(vp[lane + 32 * i]);
    m = mn;
  }
  __shared__ float sm_m[4], sm_l[4], sm_acc[4][256];
  if (lane == 0) {
    sm_m[warp] = m;
    sm_l[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (i < dpl) sm_acc[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  if (warp == 0) {
    float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    float L = 0.f, w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      w[k] = sm_m[k] == -INFINITY ? 0.f : __expf(sm_m[k] - M);
      L += sm_l[k] * w[k];
    }
    T* op = reinterpret_cast<T*>(a.out) + (static_cast<size_t>(t) * a.hq + h) * a.d;
    const float invL = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < dpl) {
        float o = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) o += sm_acc[k][lane + 32 * i] * w[k];
        op[lane + 32 * i] = Cvt<T>::from_f(o * invL);
      }
    if (a.lse && lane == 0)
      a.lse[static_cast<size_t>(t) * a.hq + h] = L > 0.f ? M + logf(L) : -INFINITY;
  }
}

// Merge two partial attention results (o, lse) in place into the first: used when a sequence's
// attention is computed in pieces (e.g. shared prefix + private suffix).
template <typename T>
__global__ void merge_attn_kernel(T* __restrict__ o1, float* __restrict__ lse1,
                                  const T* __restrict__ o2, const float* __restrict__ lse2, int d) {
  const size_t r = blockIdx.x;
  const float a = lse1[r], b = lse2[r];
  const float mx = fmaxf(a, b);
  const float wa = a == -INFINITY ? 0.f : __expf(a - mx), wb = b == -INFINITY ? 0.f : __expf(b - mx);
  const float inv = (wa + wb) > 0.f ? 1.f / (wa + wb) : 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = (Cvt<T>::to_f(o1[r * d + i]) * wa + Cvt<T>::to_f(o2[r * d + i]) * wb) * inv;
    o1[r * d + i] = Cvt<T>::from_f(v);
  }
  __syncthreads();
  if (threadIdx.x == 0) lse1[r] = (wa + wb) > 0.f ? mx + logf(wa + wb) : -INFINITY;
}

}  // namespace mlcb

using namespace mlcb;

MLCB_API int mlcb_attn_simt(const void* q, const void* kv_pages, void* out, float* lse,
                            const int* q_seq, const int* q_kvlen, const int* q_kvstart,
                            const unsigned long long* tree_mask, const int* page_indptr,
                            const int* page_indices, int tokens, int q_stride, int hq, int hkv, int d,
                            int page, int sink, float sm_scale, float softcap, int dtype,
                            cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d % 32 || d > 256 || hq % hkv) return -1;
  AttnArgs a{q, kv_pages, out, lse, q_seq, q_kvlen, q_kvstart, tree_mask, page_indptr, page_indices,
             q_stride, hq, hkv, d, page, sink, sm_scale, softcap};
  dim3 grid(tokens, hq);
  if (dtype == 0)
    attn_simt_kernel<__half><<<grid, 128, 0, stream>>>(a);
  else
    attn_simt_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_merge_attn(void* o1, float* lse1, const void* o2, const float* lse2, int rows, int d,
                             int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 0)
    merge_attn_kernel<__half><<<rows, 128, 0, stream>>>((__half*)o1, lse1, (const __half*)o2, lse2, d);
  else
    merge_attn_kernel<__nv_bfloat16>
        <<<rows, 128, 0, stream>>>((__nv_bfloat16*)o1, lse1, (const __nv_bfloat16*)o2, lse2, d);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
