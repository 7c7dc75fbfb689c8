// Attention over whole (unpaged) sequences: vision towers, BERT-style encoders, any place where all
// keys of a sequence are in one tensor. q, k, v are [batch, seq, heads, D] views (any batch / token / head
// strides, D contiguous), out is contiguous [batch, seq, heads, D]. Optional per-batch key length
// (padding) and causal masking. Flash-attention form on the warp-level tensor-core path: a CTA of four
// warps owns 64 query rows of one (batch, head), a warp 16 of them; keys and values arrive in blocks of 64
// through shared memory (row pitch D * 2 + 16 bytes keeps ldmatrix conflict-free), scores and the output
// accumulate in registers with an online softmax. Sequences here are a few hundred tokens, so the kernel is
// sized for occupancy (many small CTAs), not for a deep pipeline.
//
// Reference counterpart: the single-sequence attention the reference's encoders get from
// `op.attention` (python/mlc_llm/op/attention.py:20-186).
#include "common.cuh"

namespace mlcb {

struct EncParams {
  const void *q, *k, *v;
  void* out;
  const int* key_lens;  // [batch] or null
  long long qb, qs, qh, kb, ks, kh, vb, vs, vh;  // element strides: batch, token, head
  int S, H;
  float scale_log2;
  int causal;
};

__device__ __forceinline__ void enc_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void enc_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void enc_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16)
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool BF16>
__device__ __forceinline__ uint32_t enc_pack(float a, float b) {
  if (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, bool BF16>
__global__ void __launch_bounds__(128) enc_attn_kernel(const EncParams p) {
  static_assert(D % 32 == 0 && D <= 128, "head dims 32, 64, 96, 128");
  constexpr int PITCH = D * 2 + 16;
  constexpr int CH = D / 8;  // 16-byte chunks per row
  __shared__ __align__(16) uint8_t sk[64 * PITCH];
  __shared__ __align__(16) uint8_t sv[64 * PITCH];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = blockIdx.x * 64 + warp * 16;
  const int r0 = lane >> 2, cpair = (lane & 3) * 2;
  const int mi = lane >> 3, mr = lane & 7;
  const int klen = p.key_lens ? min(p.S, p.key_lens[b]) : p.S;
  const int kend = p.causal ? min(klen, blockIdx.x * 64 + 64) : klen;

  const uint16_t* qp = reinterpret_cast<const uint16_t*>(p.q) + b * p.qb + h * p.qh;
  const uint16_t* kp = reinterpret_cast<const uint16_t*>(p.k) + b * p.kb + h * p.kh;
  const uint16_t* vp = reinterpret_cast<const uint16_t*>(p.v) + b * p.vb + h * p.vh;

  uint32_t qa[D / 16][4];
  {
    auto load_q = [&](int row, int col) -> uint32_t {
      if (row >= p.S) return 0u;
      return *reinterpret_cast<const uint32_t*>(qp + row * p.qs + col);
    };
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa[ks][0] = load_q(q0 + r0, ks * 16 + cpair);
      qa[ks][1] = load_q(q0 + r0 + 8, ks * 16 + cpair);
      qa[ks][2] = load_q(q0 + r0, ks * 16 + 8 + cpair);
      qa[ks][3] = load_q(q0 + r0 + 8, ks * 16 + 8 + cpair);
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const uint32_t kbase = smem_u32(sk), vbase = smem_u32(sv);

  for (int kb0 = 0; kb0 < kend; kb0 += 64) {
    __syncthreads();  // the previous block's reads are done
    for (int idx = threadIdx.x; idx < 64 * CH; idx += 128) {
      const int key = idx / CH, ch = idx - key * CH;
      const int gk = kb0 + key;
      uint4 kv4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
      if (gk < p.S) {
        kv4 = *reinterpret_cast<const uint4*>(kp + gk * p.ks + ch * 8);
        vv4 = *reinterpret_cast<const uint4*>(vp + gk * p.vs + ch * 8);
      }
      *reinterpret_cast<uint4*>(sk + key * PITCH + ch * 16) = kv4;
      *reinterpret_cast<uint4*>(sv + key * PITCH + ch * 16) = vv4;
    }
    __syncthreads();
    // ---- S = Q K^T : 8 n-tiles of 8 keys
    float sacc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {
        uint32_t b0, b1, b2, b3;
        enc_ldsm_x4(kbase + (nt * 8 + mr) * PITCH + (2 * ks + mi) * 16, b0, b1, b2, b3);
        enc_mma<BF16>(sacc[nt], qa[ks], b0, b1);
        enc_mma<BF16>(sacc[nt], qa[ks + 1], b2, b3);
      }
    }
    // ---- mask + online softmax for rows r0 and r0 + 8 of this warp
    const int row0 = q0 + r0, row1 = q0 + r0 + 8;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int key = kb0 + nt * 8 + cpair + c;
        const bool in = key < klen;
        float v0 = sacc[nt][c] * p.scale_log2, v1 = sacc[nt][2 + c] * p.scale_log2;
        v0 = (in && (!p.causal || key <= row0)) ? v0 : -INFINITY;
        v1 = (in && (!p.causal || key <= row1)) ? v1 : -INFINITY;
        sacc[nt][c] = v0;
        sacc[nt][2 + c] = v1;
        mx0 = fmaxf(mx0, v0);
        mx1 = fmaxf(mx1, v1);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float a0 = mn0 == -INFINITY ? 1.f : exp2f(m0 - mn0);
    const float a1 = mn1 == -INFINITY ? 1.f : exp2f(m1 - mn1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      sacc[nt][0] = exp2f(sacc[nt][0] - ms0);
      sacc[nt][1] = exp2f(sacc[nt][1] - ms0);
      sacc[nt][2] = exp2f(sacc[nt][2] - ms1);
      sacc[nt][3] = exp2f(sacc[nt][3] - ms1);
      s0 += sacc[nt][0] + sacc[nt][1];
      s1 += sacc[nt][2] + sacc[nt][3];
    }
    l0 = l0 * a0 + s0;
    l1 = l1 * a1 + s1;
    m0 = mn0;
    m1 = mn1;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= a0;
      o[j][1] *= a0;
      o[j][2] *= a1;
      o[j][3] *= a1;
    }
    // ---- O += P V : four k-steps of 16 keys
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pa[4];
      pa[0] = enc_pack<BF16>(sacc[2 * kk][0], sacc[2 * kk][1]);
      pa[1] = enc_pack<BF16>(sacc[2 * kk][2], sacc[2 * kk][3]);
      pa[2] = enc_pack<BF16>(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
      pa[3] = enc_pack<BF16>(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < D / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        enc_ldsm_x4_t(vbase + (kk * 16 + (mi & 1) * 8 + mr) * PITCH + (j + (mi >> 1)) * 16, b0, b1, b2, b3);
        enc_mma<BF16>(o[j], pa, b0, b1);
        enc_mma<BF16>(o[j + 1], pa, b2, b3);
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  uint16_t* op = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(b) * p.S * p.H + h) * D;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    if (q0 + r0 < p.S)
      *reinterpret_cast<uint32_t*>(op + static_cast<size_t>(q0 + r0) * p.H * D + j * 8 + cpair) =
          enc_pack<BF16>(o[j][0] * i0, o[j][1] * i0);
    if (q0 + r0 + 8 < p.S)
      *reinterpret_cast<uint32_t*>(op + static_cast<size_t>(q0 + r0 + 8) * p.H * D + j * 8 + cpair) =
          enc_pack<BF16>(o[j][2] * i1, o[j][3] * i1);
  }
}

}  // namespace mlcb

using namespace mlcb;

// Strides are in elements. Returns -1 for an unsupported head dim or misaligned operands (the caller falls
// back to tensor operations).
MLCB_API int mlcb_attn_encoder(const void* q, const void* k, const void* v, void* out, const int* key_lens, int B,
                               int S, int H, int D, long long qb, long long qs, long long qh, long long kb,
                               long long ks, long long kh, long long vb, long long vs, long long vh, float sm_scale,
                               int causal, int dtype, cudaStream_t stream) {
  if (B <= 0 || S <= 0 || H <= 0) return 0;
  if (D != 32 && D != 64 && D != 96 && D != 128) return -1;
  const long long strides[] = {qb, qs, qh, kb, ks, kh, vb, vs, vh};
  for (long long st : strides)
    if (st % 8) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return -1;
  EncParams p{q, k, v, out, key_lens, qb, qs, qh, kb, ks, kh, vb, vs, vh, S, H, sm_scale * 1.4426950408889634f, causal};
  dim3 grid((S + 63) / 64, H, B);
#define LAUNCH(DD)                                                   \
  if (dtype == 1)                                                    \
    enc_attn_kernel<DD, true><<<grid, 128, 0, stream>>>(p);          \
  else                                                               \
    enc_attn_kernel<DD, false><<<grid, 128, 0, stream>>>(p);
  if (D == 32) {
    LAUNCH(32)
  } else if (D == 64) {
    LAUNCH(64)
  } else if (D == 96) {
    LAUNCH(96)
  } else {
    LAUNCH(128)
  }
#undef LAUNCH
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
