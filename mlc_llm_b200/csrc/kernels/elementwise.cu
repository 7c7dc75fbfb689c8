// Memory-bound per-token kernels: RMSNorm, fused residual-add + RMSNorm, SiLU*mul, rotary embedding
// fused with the paged KV append, (dequantising) embedding lookup, row gather/scatter.
//
// Reference counterparts: compiler_pass/fuse_add_norm.py:14-146 (add + RMSNorm, fp32 accumulate),
// model/llama/llama_model.py:122-125 (SwiGLU split), nn/kv_cache.py:29-37 (RoPE applied inside the
// KV-cache append), compiler_pass/fuse_dequantize_take.py:15-91 (dequantising embedding lookup).
#include "common.cuh"

namespace mlcb {

// ------------------------------------------------------------------ (add +) RMSNorm
// One CTA per token. If `residual` is non-null:  residual += x  (written back), out = norm(residual).
// Otherwise out = norm(x). 8 elements (16 bytes) per thread per step.
template <typename T, bool ADD>
__global__ void rmsnorm_kernel(const T* __restrict__ x, T* __restrict__ residual,
                               const T* __restrict__ w, T* __restrict__ out, int hidden, float eps,
                               float w_offset) {
  pdl_launch_dependents();  // a GEMM that follows may set itself up while these rows are normalised
  extern __shared__ float row[];  // hidden floats + 32 scratch
  float* scratch = row + hidden;
  const size_t base = static_cast<size_t>(blockIdx.x) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
    uint4 xv = *reinterpret_cast<const uint4*>(x + base + i);
    const T* xe = reinterpret_cast<const T*>(&xv);
    float v[8];
    if (ADD) {
      uint4 rv = *reinterpret_cast<const uint4*>(residual + base + i);
      const T* re = reinterpret_cast<const T*>(&rv);
      T o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // the sum is rounded to the storage type first, as the unfused add would do
        o[j] = Cvt<T>::from_f(Cvt<T>::to_f(xe[j]) + Cvt<T>::to_f(re[j]));
        v[j] = Cvt<T>::to_f(o[j]);
      }
      *reinterpret_cast<uint4*>(residual + base + i) = *reinterpret_cast<uint4*>(o);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = Cvt<T>::to_f(xe[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      row[i + j] = v[j];
      ss += v[j] * v[j];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / hidden + eps);
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
    uint4 wv = *reinterpret_cast<const uint4*>(w + i);
    const T* we = reinterpret_cast<const T*>(&wv);
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      o[j] = Cvt<T>::from_f(row[i + j] * inv * (Cvt<T>::to_f(we[j]) + w_offset));
    *reinterpret_cast<uint4*>(out + base + i) = *reinterpret_cast<uint4*>(o);
  }
}

// ------------------------------------------------------------------ LayerNorm (+ residual add)
// One CTA per token: out = (v - mean(v)) * rsqrt(var(v) + eps) * w + b, with v = x (+ residual, written
// back). `b` may be null. Statistics in fp32 from the row kept in shared memory (two passes over smem,
// one over global memory).
template <typename T, bool ADD>
__global__ void layernorm_kernel(const T* __restrict__ x, T* __restrict__ residual, const T* __restrict__ w,
                                 const T* __restrict__ b, T* __restrict__ out, int hidden, float eps) {
  extern __shared__ float row[];  // hidden floats + 32 scratch
  float* scratch = row + hidden;
  const size_t base = static_cast<size_t>(blockIdx.x) * hidden;
  float sum = 0.f;
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
    uint4 xv = *reinterpret_cast<const uint4*>(x + base + i);
    const T* xe = reinterpret_cast<const T*>(&xv);
    float v[8];
    if (ADD) {
      uint4 rv = *reinterpret_cast<const uint4*>(residual + base + i);
      const T* re = reinterpret_cast<const T*>(&rv);
      T o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = Cvt<T>::from_f(Cvt<T>::to_f(xe[j]) + Cvt<T>::to_f(re[j]));
        v[j] = Cvt<T>::to_f(o[j]);
      }
      *reinterpret_cast<uint4*>(residual + base + i) = *reinterpret_cast<uint4*>(o);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = Cvt<T>::to_f(xe[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      row[i + j] = v[j];
      sum += v[j];
    }
  }
  const float mean = block_sum(sum, scratch) / hidden;
  float sq = 0.f;
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float dlt = row[i + j] - mean;  // each thread re-reads only what it wrote
      sq += dlt * dlt;
    }
  }
  __syncthreads();  // block_sum's scratch is reused
  const float inv = rsqrtf(block_sum(sq, scratch) / hidden + eps);
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
    uint4 wv = *reinterpret_cast<const uint4*>(w + i);
    const T* we = reinterpret_cast<const T*>(&wv);
    uint4 bv = make_uint4(0, 0, 0, 0);
    if (b) bv = *reinterpret_cast<const uint4*>(b + i);
    const T* be = reinterpret_cast<const T*>(&bv);
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      o[j] = Cvt<T>::from_f((row[i + j] - mean) * inv * Cvt<T>::to_f(we[j]) + (b ? Cvt<T>::to_f(be[j]) : 0.f));
    *reinterpret_cast<uint4*>(out + base + i) = *reinterpret_cast<uint4*>(o);
  }
}

// ------------------------------------------------------------------ plain activations
// out = act(in), elementwise. act: 0 = SiLU, 1 = GELU(tanh), 2 = GELU(erf), 3 = relu(x)^2, 4 = x * sigmoid(1.702 x).
template <typename T>
__global__ void act_kernel(const T* __restrict__ in, T* __restrict__ out, size_t total_vec, int act) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t v = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total_vec; v += stride) {
    uint4 xv = *reinterpret_cast<const uint4*>(in + v * 8);
    const T* xe = reinterpret_cast<const T*>(&xv);
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = Cvt<T>::to_f(xe[j]);
      float r;
      if (act == 0) {
        r = a / (1.f + __expf(-a));
      } else if (act == 1) {
        r = 0.5f * a * (1.f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
      } else if (act == 2) {
        r = 0.5f * a * (1.f + erff(a * 0.7071067811865476f));
      } else if (act == 3) {
        const float p = fmaxf(a, 0.f);
        r = p * p;
      } else {
        r = a / (1.f + __expf(-1.702f * a));
      }
      o[j] = Cvt<T>::from_f(r);
    }
    *reinterpret_cast<uint4*>(out + v * 8) = *reinterpret_cast<uint4*>(o);
  }
}

// ------------------------------------------------------------------ SiLU(gate) * up
// in: [T, 2*I] (gate half then up half), out: [T, I]. act: 0 = SiLU, 1 = GELU(tanh).
template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int inter,
                               size_t total_vec, int act, const int* __restrict__ live_rows) {
  pdl_launch_dependents();
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const int vec_per_row = inter / 8;
  // a device-side row count (expert-parallel buffers: only the rows that arrived are worked on)
  if (live_rows) total_vec = min(total_vec, static_cast<size_t>(max(0, live_rows[0])) * vec_per_row);
  for (size_t v = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total_vec;
       v += stride) {
    const size_t t = v / vec_per_row;
    const int c = static_cast<int>(v % vec_per_row) * 8;
    uint4 g = *reinterpret_cast<const uint4*>(in + t * 2 * inter + c);
    uint4 u = *reinterpret_cast<const uint4*>(in + t * 2 * inter + inter + c);
    const T* ge = reinterpret_cast<const T*>(&g);
    const T* ue = reinterpret_cast<const T*>(&u);
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a = Cvt<T>::to_f(ge[j]);
      float r;
      if (act == 0) {
        r = a / (1.f + __expf(-a));
      } else {
        float k = 0.7978845608028654f * (a + 0.044715f * a * a * a);
        r = 0.5f * a * (1.f + tanhf(k));
      }
      // round the activation to the storage type before the product, as the unfused ops do
      r = Cvt<T>::to_f(Cvt<T>::from_f(r));
      o[j] = Cvt<T>::from_f(r * Cvt<T>::to_f(ue[j]));
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = *reinterpret_cast<uint4*>(o);
  }
}

// ------------------------------------------------------------------ RoPE + paged KV append
// qkv: [T, (hq + 2*hkv) * d], heads ordered q.., k.., v.. . Rotates q and k in place (non-interleaved
// halves over the first `rot_dim` elements) at position pos[t], then copies k and v of token t into
// its page slot. kv_pages layout: [num_pages, 2, hkv, page, d]. slot[t] = page_id * page + offset,
// a negative slot skips the append (used when only q needs rotating).
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, T* __restrict__ kv_pages,
                                   const int* __restrict__ pos, const int* __restrict__ slot,
                                   const float* __restrict__ inv_freq, int hq, int hkv, int d,
                                   int rot_dim, int page, float attn_factor, int* status,
                                   long long num_slots) {
  const int t = blockIdx.x;
  const int heads = hq + 2 * hkv;
  const int half = rot_dim / 2;
  const float p = static_cast<float>(pos[t]);
  T* row = qkv + static_cast<size_t>(t) * heads * d;
  // rotate q and k heads
  const int pairs = (hq + hkv) * half;
  const int jg = half >> 3;  // groups of eight rotary pairs per head
  if (half > 0 && (half & 7) == 0 && (d & 7) == 0 && blockDim.x % jg == 0) {
    // a thread keeps one group of eight frequencies (its sines and cosines are computed once) and walks
    // the heads with 16-byte loads and stores of the two halves
    const int g = threadIdx.x % jg, j0 = g * 8;
    float sn[8], cs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sincosf(p * inv_freq[j0 + j], &sn[j], &cs[j]);
      sn[j] *= attn_factor;
      cs[j] *= attn_factor;
    }
    for (int h = threadIdx.x / jg; h < hq + hkv; h += blockDim.x / jg) {
      T* hp = row + h * d + j0;
      uint4 lo = *reinterpret_cast<const uint4*>(hp), hi = *reinterpret_cast<const uint4*>(hp + half);
      T* le = reinterpret_cast<T*>(&lo);
      T* he = reinterpret_cast<T*>(&hi);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = Cvt<T>::to_f(le[j]), b = Cvt<T>::to_f(he[j]);
        le[j] = Cvt<T>::from_f(a * cs[j] - b * sn[j]);
        he[j] = Cvt<T>::from_f(b * cs[j] + a * sn[j]);
      }
      *reinterpret_cast<uint4*>(hp) = lo;
      *reinterpret_cast<uint4*>(hp + half) = hi;
    }
  } else
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int h = i / half, j = i % half;
    float s, c;
    sincosf(p * inv_freq[j], &s, &c);
    s *= attn_factor;
    c *= attn_factor;
    T* hp = row + h * d;
    const float a = Cvt<T>::to_f(hp[j]), b = Cvt<T>::to_f(hp[j + half]);
    hp[j] = Cvt<T>::from_f(a * c - b * s);
    hp[j + half] = Cvt<T>::from_f(b * c + a * s);
  }
  const long long sl = slot[t];
  if (sl < 0) return;
  if (sl >= num_slots) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, ERR_BAD_INDEX);
    return;
  }
  __syncthreads();
  const long long pg = sl / page;
  const int off = static_cast<int>(sl % page);
  const int vec_per_head = d / 8;
  for (int i = threadIdx.x; i < 2 * hkv * vec_per_head; i += blockDim.x) {
    const int kvsel = i / (hkv * vec_per_head);
    const int rem = i % (hkv * vec_per_head);
    const int h = rem / vec_per_head, v = rem % vec_per_head;
    const uint4 val =
        *reinterpret_cast<const uint4*>(row + (hq + kvsel * hkv + h) * d + v * 8);
    T* dst = kv_pages + (((pg * 2 + kvsel) * hkv + h) * page + off) * static_cast<size_t>(d) + v * 8;
    *reinterpret_cast<uint4*>(dst) = val;
  }
}

// ------------------------------------------------------------------ embedding lookup
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             T* __restrict__ out, int hidden, int vocab, float scale) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * hidden + i);
    if (scale != 1.f) {
      T* e = reinterpret_cast<T*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = Cvt<T>::from_f(Cvt<T>::to_f(e[j]) * scale);
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden + i) = v;
  }
}

// q4f16_1 table in the *artifact* nibble order (element j of a word at bits 4*(j%8)).
__global__ void embed_q4_kernel(const int* __restrict__ ids, const uint32_t* __restrict__ qw,
                                const __half* __restrict__ qs, __half* __restrict__ out, int hidden,
                                int vocab) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const int words = hidden / 8;
  for (int wi = threadIdx.x; wi < words; wi += blockDim.x) {
    const uint32_t x = qw[static_cast<size_t>(id) * words + wi];
    const float s = __half2float(qs[static_cast<size_t>(id) * (hidden / 32) + wi / 4]);
    __half o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      o[j] = __float2half_rn((static_cast<float>((x >> (4 * j)) & 0xf) - 7.f) * s);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden + wi * 8) =
        *reinterpret_cast<uint4*>(o);
  }
}

// ------------------------------------------------------------------ row gather / scatter
// dst[i, :] = src[idx[i], :] (gather) or dst[idx[i], :] = src[i, :] (scatter); rows of `row_bytes`.
__global__ void row_copy_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                const int* __restrict__ idx, int row_bytes, int scatter) {
  const int i = blockIdx.x;
  const size_t s = scatter ? static_cast<size_t>(i) : static_cast<size_t>(idx[i]);
  const size_t d = scatter ? static_cast<size_t>(idx[i]) : static_cast<size_t>(i);
  const uint4* sp = reinterpret_cast<const uint4*>(src + s * row_bytes);
  uint4* dp = reinterpret_cast<uint4*>(dst + d * row_bytes);
  for (int v = threadIdx.x; v < row_bytes / 16; v += blockDim.x) dp[v] = sp[v];
}

// Copies whole KV pages (all layers are handled by the caller looping or by a large row): used for
// tok[i] = last[src[i]] where src[i] >= 0 (deferred-read decode steps: the tokens one step sampled are
// the next step's inputs and stay on the device). A source row outside `last` is reported, not read.
__global__ void token_feed_kernel(int* __restrict__ tok, const int* __restrict__ src, const int* __restrict__ last,
                                  int n, int n_last, int* __restrict__ status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int s = src[i];
  if (s < 0) return;
  if (s >= n_last) {
    if (status) atomicCAS(status, 0, static_cast<int>(ERR_BAD_INDEX));
    return;
  }
  tok[i] = last[s];
}

// copy-on-write of a partially filled last page when a sequence is forked.
__global__ void page_copy_kernel(uint8_t* __restrict__ pages, const int* __restrict__ src_dst,
                                 size_t page_bytes, size_t layer_stride, int pairs) {
  const int pair = blockIdx.x % pairs;
  const int layer = blockIdx.x / pairs;
  const uint4* sp = reinterpret_cast<const uint4*>(pages + layer * layer_stride +
                                                   static_cast<size_t>(src_dst[2 * pair]) * page_bytes);
  uint4* dp = reinterpret_cast<uint4*>(pages + layer * layer_stride +
                                       static_cast<size_t>(src_dst[2 * pair + 1]) * page_bytes);
  for (size_t v = threadIdx.x; v < page_bytes / 16; v += blockDim.x) dp[v] = sp[v];
}

// Copies the KV rows of individual token slots from one paged pool to another (the other pool may
// live on a peer GPU: prefill -> decode hand-off of disaggregated serving). Pools are
// [layers][pages][2][hkv][page][row_bytes]; one warp moves one (token, layer, k|v, head) row.
__global__ void kv_slot_copy_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                    const int* __restrict__ src_slots, const int* __restrict__ dst_slots,
                                    int n, int layers, size_t src_layer_stride, size_t dst_layer_stride, int hkv,
                                    int page, int row_bytes, int src_slot_limit, int dst_slot_limit,
                                    int* __restrict__ status) {
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(n) * layers * 2 * hkv;
  if (warp >= total) return;
  const int h = static_cast<int>(warp % hkv);
  const int kv = static_cast<int>((warp / hkv) % 2);
  const int l = static_cast<int>((warp / (2 * hkv)) % layers);
  const int i = static_cast<int>(warp / (static_cast<long long>(2) * hkv * layers));
  const int ss = src_slots[i], ds = dst_slots[i];
  // a slot outside either pool is never dereferenced: the row is skipped and the host is told
  if (ss < 0 || ss >= src_slot_limit || ds < 0 || ds >= dst_slot_limit) {
    if (lane == 0 && status) atomicCAS(status, 0, static_cast<int>(ERR_BAD_INDEX));
    return;
  }
  const size_t head_bytes = static_cast<size_t>(page) * row_bytes;
  const size_t so = l * src_layer_stride + ((static_cast<size_t>(ss / page) * 2 + kv) * hkv + h) * head_bytes +
                    static_cast<size_t>(ss % page) * row_bytes;
  const size_t dof = l * dst_layer_stride + ((static_cast<size_t>(ds / page) * 2 + kv) * hkv + h) * head_bytes +
                     static_cast<size_t>(ds % page) * row_bytes;
  const uint4* sp = reinterpret_cast<const uint4*>(src + so);
  uint4* dp = reinterpret_cast<uint4*>(dst + dof);
  for (int v = lane; v < row_bytes / 16; v += 32) dp[v] = sp[v];
}

// One decode token of the gated delta rule (Qwen3.5 linear-attention layers; reference:
// python/mlc_llm/model/qwen35/qwen35_model.py:219-365), in place on the slot-indexed state pool:
//   S <- exp(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  out = S^T q
// state: [slots, H, DK, DV] fp32; q, k: [B, H, DK]; v, out: [B, H, DV]; g, beta: [B, H]. One CTA per (head,
// sequence), thread j owns column j of the head's state and keeps it in registers between the two passes, so
// the state is read once and written once.
template <int DK>
__global__ void gdn_step_kernel(float* __restrict__ state, const int* __restrict__ slots, const float* __restrict__ q,
                                const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ g,
                                const float* __restrict__ beta, float* __restrict__ out, int H, int DV) {
  // 2 * DV threads: thread (half, j) keeps rows [half * DK / 2, (half + 1) * DK / 2) of column j in registers
  constexpr int HK = DK / 2;
  extern __shared__ float gdn_sm[];  // ks[DK], qs[DK], red[2][DV]
  float* ks = gdn_sm;
  float* qs = gdn_sm + DK;
  float* red = gdn_sm + 2 * DK;
  const int h = blockIdx.x, b = blockIdx.y;
  const int half = threadIdx.x / DV, j = threadIdx.x - half * DV;
  const size_t bh = static_cast<size_t>(b) * H + h;
  for (int i = threadIdx.x; i < DK; i += blockDim.x) {
    ks[i] = k[bh * DK + i];
    qs[i] = q[bh * DK + i];
  }
  __syncthreads();
  float* S = state + ((static_cast<size_t>(slots[b]) * H + h) * DK + half * HK) * DV + j;
  const float eg = __expf(g[bh]);
  float s[HK];
  float part = 0.f;
#pragma unroll
  for (int i = 0; i < HK; ++i) {
    s[i] = S[static_cast<size_t>(i) * DV] * eg;
    part += s[i] * ks[half * HK + i];
  }
  red[half * DV + j] = part;
  __syncthreads();
  const float u = (v[bh * DV + j] - (red[j] + red[DV + j])) * beta[bh];
  __syncthreads();
  part = 0.f;
#pragma unroll
  for (int i = 0; i < HK; ++i) {
    s[i] += ks[half * HK + i] * u;
    S[static_cast<size_t>(i) * DV] = s[i];
    part += s[i] * qs[half * HK + i];
  }
  red[half * DV + j] = part;
  __syncthreads();
  if (half == 0) out[bh * DV + j] = red[j] + red[DV + j];
}

// RWKV-5 recurrence (reference: python/mlc_llm/model/rwkv5/rwkv5_model.py:64-123). One CTA per
// (head, sequence); thread i owns row i of the head's matrix state (value dimension i, all key dimensions)
// in registers and walks the sequence's tokens in order:
//   out_t[i] = sum_k r_t[k] * (u[k] * k_t[k] * v_t[i] + S[i][k]);   S[i][k] = S[i][k] * w[k] + k_t[k] * v_t[i]
// r, k, v, out: [tokens, heads, H] fp32.  w, u: [heads, H].  The state of sequence s for this layer starts at
// state_base[s] + layer_offset floats and is [heads, H, H].
// PER_TOKEN: the decay `w` is [tokens, heads, H] (RWKV-6, data-dependent) instead of [heads, H].
template <int H, bool PER_TOKEN>
__global__ void __launch_bounds__(H) wkv5_kernel(const float* __restrict__ r, const float* __restrict__ k,
                                                  const float* __restrict__ v, const float* __restrict__ w,
                                                  const float* __restrict__ u, const long long* __restrict__ state_base,
                                                  long long layer_offset, const int* __restrict__ q_indptr,
                                                  float* __restrict__ out, int heads, int total_tokens) {
  __shared__ float sh_r[H], sh_k[H], sh_w[H], sh_u[H];
  const int h = blockIdx.x, seq = blockIdx.y, i = threadIdx.x;
  const int t0 = q_indptr[seq], t1 = q_indptr[seq + 1];
  if (t0 < 0 || t1 > total_tokens || t0 >= t1) return;
  float* state = reinterpret_cast<float*>(state_base[seq]) + layer_offset +
                 (static_cast<size_t>(h) * H + i) * H;
  float s[H];
#pragma unroll
  for (int j = 0; j < H; ++j) s[j] = state[j];
  if (!PER_TOKEN) sh_w[i] = w[h * H + i];
  sh_u[i] = u[h * H + i];
  for (int t = t0; t < t1; ++t) {
    const size_t base = (static_cast<size_t>(t) * heads + h) * H;
    __syncthreads();
    sh_r[i] = r[base + i];
    sh_k[i] = k[base + i];
    if (PER_TOKEN) sh_w[i] = w[base + i];
    __syncthreads();
    const float vi = v[base + i];
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < H; ++j) {
      const float x = sh_k[j] * vi;
      acc += sh_r[j] * (sh_u[j] * x + s[j]);
      s[j] = s[j] * sh_w[j] + x;
    }
    out[base + i] = acc;
  }
#pragma unroll
  for (int j = 0; j < H; ++j) state[j] = s[j];
}

}  // namespace mlcb

using namespace mlcb;

// head_size 32 or 64 (every released RWKV-5 uses 64); other sizes return -1 and the caller falls back.
MLCB_API int mlcb_wkv5(const float* r, const float* k, const float* v, const float* w, const float* u,
                       const long long* state_base, long long layer_offset, const int* q_indptr, float* out,
                       int num_seqs, int heads, int head_size, int total_tokens, int w_per_token,
                       cudaStream_t stream) {
  if (num_seqs <= 0 || total_tokens <= 0) return 0;
  if (heads <= 0 || num_seqs > 65535) return -1;
  dim3 grid(heads, num_seqs);
#define WKV_LAUNCH(HS, PT)                                                                                   \
  wkv5_kernel<HS, PT><<<grid, HS, 0, stream>>>(r, k, v, w, u, state_base, layer_offset, q_indptr, out, heads, \
                                               total_tokens)
  if (head_size == 64) {
    if (w_per_token) WKV_LAUNCH(64, true);
    else WKV_LAUNCH(64, false);
  } else if (head_size == 32) {
    if (w_per_token) WKV_LAUNCH(32, true);
    else WKV_LAUNCH(32, false);
  } else {
    return -1;
  }
#undef WKV_LAUNCH
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// Lets kernels running on `device` dereference memory of `peer` (both in this process's view).
// Returns 0 when access is (already) enabled.
MLCB_API int mlcb_token_feed(int* tok, const int* src, const int* last, int n, int n_last, int* status,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  token_feed_kernel<<<(n + 255) / 256, 256, 0, stream>>>(tok, src, last, n, n_last, status);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_enable_peer_access(int device, int peer) {
  if (device == peer) return 0;
  int can = 0;
  cudaError_t err = cudaDeviceCanAccessPeer(&can, device, peer);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (!can) return -1;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  err = cudaDeviceEnablePeerAccess(peer, 0);
  cudaSetDevice(prev);
  if (err == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return static_cast<int>(err);
}

// Strides in bytes; row_bytes = head_dim * element size (multiple of 16). Slots must lie in
// [0, src_pages * page) and [0, dst_pages * page): the host checks before the launch and the kernel
// skips (and reports ERR_BAD_INDEX for) any row that is not.
MLCB_API int mlcb_kv_slot_copy(const void* src, void* dst, const int* src_slots, const int* dst_slots, int n,
                               int layers, long long src_layer_stride, long long dst_layer_stride, int hkv,
                               int page, int row_bytes, int src_pages, int dst_pages, int* status,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  if (row_bytes % 16 || page <= 0 || src_pages <= 0 || dst_pages <= 0) return -1;
  if (static_cast<long long>(src_pages) * page > 0x7fffffffLL || static_cast<long long>(dst_pages) * page > 0x7fffffffLL)
    return -1;
  const long long warps = static_cast<long long>(n) * layers * 2 * hkv;
  const long long blocks = (warps + 7) / 8;
  kv_slot_copy_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), src_slots, dst_slots, n, layers,
      static_cast<size_t>(src_layer_stride), static_cast<size_t>(dst_layer_stride), hkv, page, row_bytes,
      src_pages * page, dst_pages * page, status);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// dtype: 0 fp16, 1 bf16
MLCB_API int mlcb_rmsnorm(const void* x, void* residual, const void* w, void* out, int tokens,
                          int hidden, float eps, float w_offset, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return -1;
  int threads = hidden / 8;
  threads = threads > 1024 ? 1024 : (threads < 32 ? 32 : (threads + 31) / 32 * 32);
  size_t smem = (hidden + 32) * sizeof(float);
  if (smem > 48 * 1024) return -2;
#define LAUNCH(T)                                                                                  \
  if (residual)                                                                                    \
    rmsnorm_kernel<T, true><<<tokens, threads, smem, stream>>>(                                    \
        (const T*)x, (T*)residual, (const T*)w, (T*)out, hidden, eps, w_offset);                   \
  else                                                                                             \
    rmsnorm_kernel<T, false><<<tokens, threads, smem, stream>>>((const T*)x, nullptr,              \
                                                                (const T*)w, (T*)out, hidden, eps, \
                                                                w_offset);
  if (dtype == 0) {
    LAUNCH(__half)
  } else {
    LAUNCH(__nv_bfloat16)
  }
#undef LAUNCH
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_gdn_step(float* state, const int* slots, const float* q, const float* k, const float* v,
                           const float* g, const float* beta, float* out, int B, int H, int DK, int DV,
                           cudaStream_t stream) {
  if (B <= 0) return 0;
  // the register file bounds the CTA: 2 * DV threads each holding DK / 2 state values
  if (DV < 32 || DV % 32 || DV * DK > 128 * 128) return -1;
  dim3 grid(H, B);
  const int threads = 2 * DV;
  const size_t smem = (2 * static_cast<size_t>(DK) + 2 * DV) * sizeof(float);
  if (DK == 128)
    gdn_step_kernel<128><<<grid, threads, smem, stream>>>(state, slots, q, k, v, g, beta, out, H, DV);
  else if (DK == 64)
    gdn_step_kernel<64><<<grid, threads, smem, stream>>>(state, slots, q, k, v, g, beta, out, H, DV);
  else
    return -1;
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_layernorm(const void* x, void* residual, const void* w, const void* b, void* out, int tokens,
                            int hidden, float eps, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return -1;
  int threads = hidden / 8;
  if (threads > 1024) threads = 1024;
  threads = (threads + 31) / 32 * 32;
  const size_t smem = (static_cast<size_t>(hidden) + 32) * sizeof(float);
  if (smem > 48 * 1024) return -2;
#define LAUNCH(T)                                                                                         \
  if (residual)                                                                                           \
    layernorm_kernel<T, true><<<tokens, threads, smem, stream>>>((const T*)x, (T*)residual, (const T*)w,  \
                                                                 (const T*)b, (T*)out, hidden, eps);      \
  else                                                                                                    \
    layernorm_kernel<T, false><<<tokens, threads, smem, stream>>>((const T*)x, nullptr, (const T*)w,      \
                                                                  (const T*)b, (T*)out, hidden, eps);
  if (dtype == 0) {
    LAUNCH(__half)
  } else {
    LAUNCH(__nv_bfloat16)
  }
#undef LAUNCH
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_act(const void* in, void* out, long long elems, int act, int dtype, cudaStream_t stream) {
  if (elems <= 0) return 0;
  if (elems % 8) return -1;
  const size_t total = static_cast<size_t>(elems / 8);
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  if (dtype == 0)
    act_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)in, (__half*)out, total, act);
  else
    act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, total, act);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_act_mul(const void* in, void* out, int tokens, int inter, int act, int dtype,
                          cudaStream_t stream, const int* live_rows) {
  if (tokens <= 0) return 0;
  if (inter % 8) return -1;
  size_t total = static_cast<size_t>(tokens) * (inter / 8);
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  if (dtype == 0)
    act_mul_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)in, (__half*)out, inter, total, act, live_rows);
  else
    act_mul_kernel<__nv_bfloat16>
        <<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, inter, total, act, live_rows);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_rope_append(void* qkv, void* kv_pages, const int* pos, const int* slot,
                              const float* inv_freq, int tokens, int hq, int hkv, int d, int rot_dim,
                              int page, float attn_factor, long long num_slots, int dtype,
                              int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d % 8 || rot_dim % 2 || rot_dim > d) return -1;
  if (dtype == 0)
    rope_append_kernel<__half><<<tokens, 256, 0, stream>>>((__half*)qkv, (__half*)kv_pages, pos, slot,
                                                          inv_freq, hq, hkv, d, rot_dim, page,
                                                          attn_factor, status, num_slots);
  else
    rope_append_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(
        (__nv_bfloat16*)qkv, (__nv_bfloat16*)kv_pages, pos, slot, inv_freq, hq, hkv, d, rot_dim, page,
        attn_factor, status, num_slots);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_embed(const int* ids, const void* table, void* out, int tokens, int hidden,
                        int vocab, float scale, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return -1;
  if (dtype == 0)
    embed_kernel<__half><<<tokens, 256, 0, stream>>>(ids, (const __half*)table, (__half*)out, hidden,
                                                    vocab, scale);
  else
    embed_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(ids, (const __nv_bfloat16*)table,
                                                           (__nv_bfloat16*)out, hidden, vocab, scale);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_embed_q4(const int* ids, const void* qw, const void* qs, void* out, int tokens,
                           int hidden, int vocab, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden % 32) return -1;
  embed_q4_kernel<<<tokens, 256, 0, stream>>>(ids, (const uint32_t*)qw, (const __half*)qs,
                                              (__half*)out, hidden, vocab);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_row_copy(const void* src, void* dst, const int* idx, int rows, int row_bytes,
                           int scatter, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (row_bytes % 16) return -1;
  row_copy_kernel<<<rows, 256, 0, stream>>>((const uint8_t*)src, (uint8_t*)dst, idx, row_bytes,
                                            scatter);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_page_copy(void* pages, const int* src_dst, int pairs, int layers,
                            long long page_bytes, long long layer_stride, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  page_copy_kernel<<<pairs * layers, 256, 0, stream>>>((uint8_t*)pages, src_dst, (size_t)page_bytes,
                                                      (size_t)layer_stride, pairs);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
