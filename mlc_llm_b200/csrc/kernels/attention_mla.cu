// Multi-head latent attention over a compressed cache (DeepSeek-V2 / V3 form).
//
// The cache holds ONE row per token and layer: [rotary key part (rope) | normalised latent (rank)], shared by
// all heads, instead of per-head keys and values. Queries arrive "absorbed": per head [rotated rotary part |
// no-position part multiplied by the key up-projection], so a score is one dot product with the cached row,
// and the context is the softmax-weighted sum of the latent parts of the rows (the value up-projection is
// applied afterwards, outside). Reference semantics: the MLA mode of the paged cache
// (python/mlc_llm/model/deepseek_v2/deepseek_v2_model.py:301-385: append_mla_kv + absorbed attention).
//
// One warp owns one (token, head); the eight warps of a CTA are eight heads of the same token, so the rows
// they walk are the same and come from L1 after the first warp's read. Four rows are in flight per step so
// that the four dot-product reductions overlap.
#include "common.cuh"

namespace mlcb {

struct MlaArgs {
  const void* q;          // [T, hq, D], token stride q_stride elements, D = rope + rank
  const void* cache;      // [num_pages, page, D]
  void* out;              // [T, hq, rank]
  const int* q_seq;       // [T] batch slot of each query token
  const int* q_kvlen;     // [T] rows visible through the causal rule
  const int* q_kvstart;   // [T] first visible non-sink row, or null
  const unsigned long long* tree_mask;  // [T] or null: bit j = may attend row q_kvlen[t] + j
  const int* page_indptr; // [B + 1]
  const int* page_indices;
  int q_stride, hq, rope, rank, page, num_pages, sink;
  float sm_scale;
  int* status;
};

template <typename T>
struct Pair;
template <>
struct Pair<__half> {
  using type = __half2;
  static __device__ __forceinline__ float2 to_f2(__half2 v) { return __half22float2(v); }
  static __device__ __forceinline__ __half2 from_f2(float x, float y) { return __floats2half2_rn(x, y); }
};
template <>
struct Pair<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ __nv_bfloat162 from_f2(float x, float y) { return __floats2bfloat162_rn(x, y); }
};

// ND = D / 64: a lane holds elements [64 i + 2 lane, 64 i + 2 lane + 1] of a row for i < ND.
template <typename T, int ND>
__global__ void __launch_bounds__(256) attn_mla_kernel(const MlaArgs a) {
  using P = Pair<T>;
  using T2 = typename P::type;
  constexpr int D = ND * 64;
  constexpr int U = 4;  // rows in flight
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 8 + warp;
  if (h >= a.hq) return;  // whole warp
  const int nr = a.rope / 64;  // chunks of the rotary part (they take part in the score only)
  const int b = a.q_seq[t];
  const int causal_len = a.q_kvlen[t];
  const int start = a.q_kvstart ? a.q_kvstart[t] : 0;
  const unsigned long long tmask = a.tree_mask ? a.tree_mask[t] : 0ull;
  const int extra = tmask ? 64 - __clzll(tmask) : 0;
  const int total = causal_len + extra;
  const int first_pg = a.page_indptr[b];
  const int n_pg = a.page_indptr[b + 1] - first_pg;
  const int* pages = a.page_indices + first_pg;

  const T2* qp = reinterpret_cast<const T2*>(reinterpret_cast<const T*>(a.q) + static_cast<size_t>(t) * a.q_stride +
                                             static_cast<size_t>(h) * D);
  float2 qv[ND], acc[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const float2 v = P::to_f2(qp[32 * i + lane]);
    qv[i] = make_float2(v.x * a.sm_scale, v.y * a.sm_scale);
    acc[i] = make_float2(0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f;
  bool bad = false;
  const T* base = reinterpret_cast<const T*>(a.cache);
  for (int j0 = 0; j0 < total; j0 += U) {
    float2 row[U][ND];
    float s[U];
    bool vis[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u;
      bool v = j < total && (j < causal_len ? (j < a.sink || j >= start) : ((tmask >> (j - causal_len)) & 1ull) != 0);
      int pg = 0;
      if (v) {
        const int pi = j / a.page;
        pg = pi < n_pg ? pages[pi] : -1;
        if (pg < 0 || pg >= a.num_pages) {  // never dereferenced: reported through the status word
          v = false;
          bad = true;
        }
      }
      float dot = 0.f;
      if (v) {
        const T2* rp = reinterpret_cast<const T2*>(base + (static_cast<size_t>(pg) * a.page + j % a.page) * D);
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          const float2 x = P::to_f2(rp[32 * i + lane]);
          row[u][i] = x;
          dot += qv[i].x * x.x + qv[i].y * x.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < ND; ++i) row[u][i] = make_float2(0.f, 0.f);
      }
      s[u] = dot;
      vis[u] = v;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) s[u] = warp_sum(s[u]);
    float mn = m;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!vis[u]) s[u] = -INFINITY;
      mn = fmaxf(mn, s[u]);
    }
    if (mn == -INFINITY) continue;  // nothing visible so far
    const float corr = __expf(m - mn);
    float p[U], psum = 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      p[u] = __expf(s[u] - mn);
      psum += p[u];
    }
    l = l * corr + psum;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
      float x = acc[i].x * corr, y = acc[i].y * corr;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        x += p[u] * row[u][i].x;
        y += p[u] * row[u][i].y;
      }
      acc[i] = make_float2(x, y);
    }
    m = mn;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T2* op = reinterpret_cast<T2*>(reinterpret_cast<T*>(a.out) + (static_cast<size_t>(t) * a.hq + h) * a.rank);
#pragma unroll
  for (int i = 0; i < ND; ++i)
    if (i >= nr) op[32 * (i - nr) + lane] = P::from_f2(acc[i].x * inv, acc[i].y * inv);
  if (bad && lane == 0 && a.status) atomicCAS(a.status, 0, ERR_BAD_INDEX);
}

// One CTA per token: the row [rotated rotary key | latent] goes to the token's slot of this layer's cache.
template <typename T>
__global__ void __launch_bounds__(128)
mla_append_kernel(const T* __restrict__ rows, T* __restrict__ cache, const int* __restrict__ slots, int d,
                  long long num_slots, int* status) {
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;  // a token that is not cached (stand-in rows of a padded batch)
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, ERR_BAD_INDEX);
    return;
  }
  const uint32_t* in = reinterpret_cast<const uint32_t*>(rows + static_cast<size_t>(t) * d);
  uint32_t* out = reinterpret_cast<uint32_t*>(cache + static_cast<size_t>(slot) * d);
  for (int i = threadIdx.x; i < d / 2; i += blockDim.x) out[i] = in[i];
}

template <typename T>
static int launch_mla(const MlaArgs& a, int tokens, int nd, cudaStream_t stream) {
  dim3 grid(tokens, (a.hq + 7) / 8);
  switch (nd) {
    case 2: attn_mla_kernel<T, 2><<<grid, 256, 0, stream>>>(a); break;
    case 3: attn_mla_kernel<T, 3><<<grid, 256, 0, stream>>>(a); break;
    case 4: attn_mla_kernel<T, 4><<<grid, 256, 0, stream>>>(a); break;
    case 5: attn_mla_kernel<T, 5><<<grid, 256, 0, stream>>>(a); break;
    case 6: attn_mla_kernel<T, 6><<<grid, 256, 0, stream>>>(a); break;
    case 7: attn_mla_kernel<T, 7><<<grid, 256, 0, stream>>>(a); break;
    case 8: attn_mla_kernel<T, 8><<<grid, 256, 0, stream>>>(a); break;
    case 9: attn_mla_kernel<T, 9><<<grid, 256, 0, stream>>>(a); break;
    default: return -1;
  }
  return 0;
}

}  // namespace mlcb

using namespace mlcb;

// q [T, hq, rope + rank] (token stride q_stride elements), cache [num_pages, page, rope + rank] of one layer,
// out [T, hq, rank]. rope and rank are multiples of 64, rope + rank <= 576. Returns -1 for other shapes.
MLCB_API int mlcb_attn_mla(const void* q, const void* cache, void* out, const int* q_seq, const int* q_kvlen,
                           const int* q_kvstart, const unsigned long long* tree_mask, const int* page_indptr,
                           const int* page_indices, int tokens, int q_stride, int hq, int rope, int rank, int page,
                           int num_pages, int sink, float sm_scale, int dtype, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int d = rope + rank;
  if (rope <= 0 || rank <= 0 || rope % 64 || rank % 64 || d > 576 || page <= 0 || (q_stride % 2) || dtype > 1)
    return -1;
  MlaArgs a{q, cache, out, q_seq, q_kvlen, q_kvstart, tree_mask, page_indptr, page_indices,
            q_stride, hq, rope, rank, page, num_pages, sink, sm_scale, status};
  const int rc = dtype == 0 ? launch_mla<__half>(a, tokens, d / 64, stream)
                            : launch_mla<__nv_bfloat16>(a, tokens, d / 64, stream);
  if (rc) return rc;
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// rows [T, d] (contiguous): row t goes to slot slots[t] of cache [num_slots, d]; negative slots are skipped.
MLCB_API int mlcb_mla_append(const void* rows, void* cache, const int* slots, int tokens, int d, long long num_slots,
                             int dtype, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d % 2 || dtype > 1) return -1;
  if (dtype == 0)
    mla_append_kernel<__half><<<tokens, 128, 0, stream>>>(static_cast<const __half*>(rows), static_cast<__half*>(cache),
                                                         slots, d, num_slots, status);
  else
    mla_append_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(rows),
                                                                static_cast<__nv_bfloat16*>(cache), slots, d,
                                                                num_slots, status);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
