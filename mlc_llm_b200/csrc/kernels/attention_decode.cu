// Paged-KV decode attention (head_dim 128, 16-token pages): the KV stream is the whole cost, so the
// kernel is organised around keeping many page loads in flight per SM, without gaps.
//
// A work unit is one (sequence, kv head, KV split) and at most 16 query rows -- the G = hq / hkv heads
// of the kv group times the few tokens appended this step (1 for plain decode, up to 16 / G for short
// verify chunks). CTAs are persistent (two per SM) and walk units blockIdx, blockIdx + grid, ...: a
// producer warp streams the pages of one unit after the other through an 8-deep ring with TMA tile loads
// (128-byte swizzle; 8 KB per page: K and V of the kv head), so the loads of the next unit are already in
// flight while the consumers finish the current one and there is no ramp-up / drain per unit. Four
// consumer warps take the pages round-robin, each running its own online softmax over
// m16n8k16 tensor-core tiles (S = Q.K^T from ldmatrix'd K, then O += P.V from transposed-ldmatrix'd V
// with P taken straight from the S accumulators), so there is no block-wide synchronisation in the page
// loop. The four partial states of a unit are merged through a scratch area of shared memory.
//
// The math uses the warp-level mma path on purpose: with <= 16 query rows the 128-row tcgen05 tile
// would spend its time on barrier round trips per KV block, while this kernel never leaves
// registers between S and O. The prefill / long-chunk path is the tcgen05 kernel in
// attention_tcgen05.cu.
//
// Reference counterpart: the paged decode attention of the reference's PagedKVCache (FlashInfer or
// TIR kernels, compiler_pass/dispatch_kv_cache_creation.py:150-243).
#include "common.cuh"

namespace mlcb {

// Ring depth: a multiple of the four consumer warps. Page number g (counted over all units of the CTA)
// goes to slot g % DEC_STAGES and to warp g % 4, so every slot is always read by the same warp, which
// therefore sees every phase of the slot's barriers in order (a waiter that skipped a phase could take
// an older completion of the same parity for the one it needs).
constexpr int DEC_STAGES = 8;
static_assert(DEC_STAGES % 4 == 0, "a ring slot must belong to one consumer warp");
constexpr int DEC_PAGE_BYTES = 8192;  // K (2 halves x 16 rows x 128 B) + V (same)
constexpr int DEC_THREADS = 160;
constexpr int DEC_MERGE_BYTES = 4 * 16 * 128 * 4 + 4 * 16 * 2 * 4;  // four warps' O rows and (m, l) pairs
constexpr int DEC_SMEM = DEC_STAGES * DEC_PAGE_BYTES + DEC_MERGE_BYTES + 1024 + 256;

struct DecParams {
  const void* q;          // row stride q_stride elements, head h at column h * 128
  void* out;              // [T, hq * 128]
  float* lse;             // [T, hq] natural log, or null
  float* part_o;          // [items, hkv, splits, 16, 128] fp32 (splits > 1)
  float* part_ml;         // [items, hkv, splits, 16, 2]
  const int* item_seq;    // [items] batch slot
  const int* item_qstart; // [items] first token (global index)
  const int* item_ntok;   // [items] tokens of the item (ntok * G <= 16)
  const int* q_kvlen;     // [T]
  const int* page_indptr;
  const int* page_indices;
  int* status;
  long long q_stride;
  int hq, hkv, group, splits;
  int num_units;          // items * hkv * splits
  float scale_log2;
  int is_bf16;
  // masked variant (same visibility rule as the tcgen05 kernel: window start + sinks below q_kvlen, ancestor
  // bits of a token tree at and above it; logit soft-capping). All null / zero for the plain causal form.
  const int* q_kvstart;
  const unsigned long long* tree_mask;
  int sink;
  float cap_pre, cap_log2;
};

__device__ __forceinline__ float dec_tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
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
__device__ __forceinline__ uint32_t pack_pair(float a, float b) {
  if (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One work unit: which pages, which rows.
struct DecUnit {
  int item, hk, split, qstart, ntok, valid_rows, pg_begin, npg;
  int sink_pg, skip;  // pages [sink_pg, sink_pg + skip) lie wholly outside every row's window: never fetched
  const int* pages;
  // i-th page the unit visits -> index into the sequence's page list
  __device__ __forceinline__ int page_index(int i) const {
    const int li = pg_begin + i;
    return li < sink_pg ? li : li + skip;
  }
};
__device__ __forceinline__ DecUnit dec_unit(const DecParams& p, int u) {
  DecUnit d;
  d.split = u % p.splits;
  const int r = u / p.splits;
  d.hk = r % p.hkv;
  d.item = r / p.hkv;
  const int b = p.item_seq[d.item];
  d.qstart = p.item_qstart[d.item];
  d.ntok = p.item_ntok[d.item];
  d.valid_rows = d.ntok * p.group;
  int kv_max = p.q_kvlen[d.qstart + d.ntok - 1];
  d.sink_pg = 0;
  d.skip = 0;
  if (p.tree_mask) {
    int extra = 0;
    for (int i = 0; i < d.ntok; ++i) extra = max(extra, 64 - __clzll(p.tree_mask[d.qstart + i] | 1ull));
    kv_max += extra;
  }
  if (p.q_kvstart) {
    int first = p.q_kvstart[d.qstart];
    for (int i = 1; i < d.ntok; ++i) first = min(first, p.q_kvstart[d.qstart + i]);
    d.sink_pg = (p.sink + 15) / 16;
    d.skip = max(0, first / 16 - d.sink_pg);
  }
  d.pages = p.page_indices + p.page_indptr[b];
  const int total_pages = max(0, (kv_max + 15) / 16 - d.skip);
  const int per_split = (total_pages + p.splits - 1) / p.splits;
  d.pg_begin = d.split * per_split;
  d.npg = max(0, min(total_pages, d.pg_begin + per_split) - d.pg_begin);
  return d;
}

template <bool BF16, bool EXT>
__global__ void __launch_bounds__(DEC_THREADS, 2)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmap_kv, const DecParams p) {
  pdl_launch_dependents();  // the output projection that follows may set itself up meanwhile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  float* sm_o = reinterpret_cast<float*>(smem + DEC_STAGES * DEC_PAGE_BYTES);  // [4 warps][16 rows][128]
  float* sm_ml = sm_o + 4 * 16 * 128;                                          // [4][16][2]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + DEC_STAGES * DEC_PAGE_BYTES + DEC_MERGE_BYTES);
  uint64_t* empty = full + DEC_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + DEC_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;

  if (threadIdx.x < DEC_STAGES) {
    mbar_init(&full[threadIdx.x], 1);
    mbar_init(&empty[threadIdx.x], 1);
    mbar_fence_init();
  }
  if (threadIdx.x == 0) *abort_flag = 0;
  __syncthreads();

  if (warp == 4) {
    // ---------------------------------------------------------------- producer: the pages of this
    // CTA's units back to back; `g` counts pages over all units, so the ring never drains in between
    if (lane == 0) {
      tma_prefetch_desc(&tmap_kv);
      int s = 0;
      uint32_t eph = 1;  // parity of empty[s] to wait for (first pass over the ring: nothing)
      uint32_t g = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
        const DecUnit d = dec_unit(p, u);
        for (int i = 0; i < d.npg; ++i, ++g) {
          if (g >= DEC_STAGES && !mbar_wait(&empty[s], eph, abort_flag, p.status, ERR_WAIT_PRODUCER)) {
            ok = false;
            break;
          }
          int page = d.pages[d.page_index(i)];
          if (page < 0) page = 0;  // released by a sliding window: every position of it is masked
          mbar_expect_tx(&full[s], DEC_PAGE_BYTES);
          uint8_t* dst = smem + s * DEC_PAGE_BYTES;
          const int krow = ((page * 2 + 0) * p.hkv + d.hk) * 16;
          const int vrow = ((page * 2 + 1) * p.hkv + d.hk) * 16;
          tma_load_2d(dst, &tmap_kv, &full[s], 0, krow);
          tma_load_2d(dst + 2048, &tmap_kv, &full[s], 64, krow);
          tma_load_2d(dst + 4096, &tmap_kv, &full[s], 0, vrow);
          tma_load_2d(dst + 6144, &tmap_kv, &full[s], 64, vrow);
          if (++s == DEC_STAGES) {
            s = 0;
            eph ^= 1;
          }
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  const int r0 = lane >> 2;       // fragment rows r0 and r0 + 8
  const int cpair = (lane & 3) * 2;
  const int mi = lane >> 3, mr = lane & 7;  // ldmatrix lane roles
  uint32_t g0 = 0;                // pages of the units before this one (ring position of the unit's page 0)
  bool ok = true;
  for (int u = blockIdx.x; u < p.num_units; u += gridDim.x) {
    const DecUnit d = dec_unit(p, u);
    const int qstart = d.qstart, hk = d.hk, valid_rows = d.valid_rows, npg = d.npg;
    // per-warp softmax state, merged at the end of the unit
    float o[16][4];
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    // Q fragments (A operand), 8 k-steps of 16 along head_dim
    uint32_t qa[8][4];
    {
      const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q);
      auto load_q = [&](int row, int dcol) -> uint32_t {
        if (row >= valid_rows) return 0u;
        const int tok = qstart + row / G, head = hk * G + row % G;
        return *reinterpret_cast<const uint32_t*>(
            qb + (static_cast<size_t>(tok) * p.q_stride + head * 128 + dcol) * 2);
      };
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qa[ks][0] = load_q(r0, ks * 16 + cpair);
        qa[ks][1] = load_q(r0 + 8, ks * 16 + cpair);
        qa[ks][2] = load_q(r0, ks * 16 + 8 + cpair);
        qa[ks][3] = load_q(r0 + 8, ks * 16 + 8 + cpair);
      }
    }
    const int kvlen0 = r0 < valid_rows ? p.q_kvlen[qstart + r0 / G] : 0;
    const int kvlen1 = (r0 + 8) < valid_rows ? p.q_kvlen[qstart + (r0 + 8) / G] : 0;
    int start0 = 0, start1 = 0;
    unsigned long long tm0 = 0ull, tm1 = 0ull;
    if (EXT) {
      if (p.q_kvstart) {
        if (r0 < valid_rows) start0 = p.q_kvstart[qstart + r0 / G];
        if (r0 + 8 < valid_rows) start1 = p.q_kvstart[qstart + (r0 + 8) / G];
      }
      if (p.tree_mask) {
        if (r0 < valid_rows) tm0 = p.tree_mask[qstart + r0 / G];
        if (r0 + 8 < valid_rows) tm1 = p.tree_mask[qstart + (r0 + 8) / G];
      }
    }
    auto visible = [&](int pos, int kvlen, int start, unsigned long long tm) -> bool {
      if (!EXT) return pos < kvlen;
      if (pos < kvlen) return pos >= start || pos < p.sink;
      const int r = pos - kvlen;
      return r < 64 && ((tm >> r) & 1ull);
    };
    // this warp's pages of the unit: those whose number over all units is congruent to the warp index
    for (int i = (warp - static_cast<int>(g0 & 3u)) & 3; i < npg && ok; i += 4) {
      const uint32_t g = g0 + static_cast<uint32_t>(i);
      const int s = g % DEC_STAGES;
      ok = mbar_wait(&full[s], (g / DEC_STAGES) & 1, abort_flag, p.status, ERR_WAIT_TMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t kbase = smem_u32(smem + s * DEC_PAGE_BYTES);
      const uint32_t vbase = kbase + 4096;
      // ---- S = Q K^T for the 16 tokens of the page: two n-tiles of 8 tokens
      float sacc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
        const int token = nt * 8 + mr;
#pragma unroll
        for (int ks = 0; ks < 8; ks += 2) {
          const int chunk = 2 * ks + mi;  // 16-byte chunk along head_dim (0..15)
          const uint32_t addr = kbase + (chunk >> 3) * 2048 + token * 128 + (((chunk & 7) ^ (token & 7)) << 4);
          uint32_t b0, b1, b2, b3;
          ldsm_x4(addr, b0, b1, b2, b3);
          mma16816<BF16>(sacc[nt], qa[ks], b0, b1);
          mma16816<BF16>(sacc[nt], qa[ks + 1], b2, b3);
        }
      }
      // ---- mask + online softmax (rows r0 and r0 + 8)
      const int pos_base = d.page_index(i) * 16;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int pos = pos_base + nt * 8 + cpair + c;
          float v0, v1;
          if (EXT && p.cap_log2 != 0.f) {
            v0 = p.cap_log2 * dec_tanh_approx(sacc[nt][c] * p.cap_pre);
            v1 = p.cap_log2 * dec_tanh_approx(sacc[nt][2 + c] * p.cap_pre);
          } else {
            v0 = sacc[nt][c] * p.scale_log2;
            v1 = sacc[nt][2 + c] * p.scale_log2;
          }
          v0 = visible(pos, kvlen0, start0, tm0) ? v0 : -INFINITY;
          v1 = visible(pos, kvlen1, start1, tm1) ? v1 : -INFINITY;
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
      uint32_t pa[4];
      {
        const float e00 = exp2f(sacc[0][0] - ms0), e01 = exp2f(sacc[0][1] - ms0);
        const float e02 = exp2f(sacc[0][2] - ms1), e03 = exp2f(sacc[0][3] - ms1);
        const float e10 = exp2f(sacc[1][0] - ms0), e11 = exp2f(sacc[1][1] - ms0);
        const float e12 = exp2f(sacc[1][2] - ms1), e13 = exp2f(sacc[1][3] - ms1);
        l0 = l0 * a0 + (e00 + e01 + e10 + e11);
        l1 = l1 * a1 + (e02 + e03 + e12 + e13);
        pa[0] = pack_pair<BF16>(e00, e01);  // row r0,     tokens 0-7
        pa[1] = pack_pair<BF16>(e02, e03);  // row r0 + 8, tokens 0-7
        pa[2] = pack_pair<BF16>(e10, e11);  // row r0,     tokens 8-15
        pa[3] = pack_pair<BF16>(e12, e13);  // row r0 + 8, tokens 8-15
      }
      m0 = mn0;
      m1 = mn1;
      // ---- O = O * alpha + P V : 16 n-tiles of 8 along head_dim, one k-step of 16 tokens
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        o[j][0] *= a0; o[j][1] *= a0; o[j][2] *= a1; o[j][3] *= a1;
        o[j + 1][0] *= a0; o[j + 1][1] *= a0; o[j + 1][2] *= a1; o[j + 1][3] *= a1;
        const int token = (mi & 1) * 8 + mr;
        const int chunk = j + (mi >> 1);
        const uint32_t addr = vbase + (chunk >> 3) * 2048 + token * 128 + (((chunk & 7) ^ (token & 7)) << 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(addr, b0, b1, b2, b3);
        mma16816<BF16>(o[j], pa, b0, b1);
        mma16816<BF16>(o[j + 1], pa, b2, b3);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    g0 += static_cast<uint32_t>(npg);
    // row sums live spread over the 4 lanes of a quad
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---------------------------------------------------------------- merge the four warps of the unit
    // (named barrier over the 128 consumer threads; the producer keeps streaming the next unit's pages)
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float* d0 = sm_o + ((warp * 16 + r0) * 128 + j * 8 + cpair);
      float* d1 = sm_o + ((warp * 16 + r0 + 8) * 128 + j * 8 + cpair);
      if (r0 < valid_rows) {
        d0[0] = o[j][0];
        d0[1] = o[j][1];
      }
      if (r0 + 8 < valid_rows) {
        d1[0] = o[j][2];
        d1[1] = o[j][3];
      }
    }
    if ((lane & 3) == 0) {
      sm_ml[(warp * 16 + r0) * 2] = m0;
      sm_ml[(warp * 16 + r0) * 2 + 1] = l0;
      sm_ml[(warp * 16 + r0 + 8) * 2] = m1;
      sm_ml[(warp * 16 + r0 + 8) * 2 + 1] = l1;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // warp w finalises rows w, w + 4, ...; lane handles 4 consecutive head_dim elements
    for (int row = warp; row < valid_rows; row += 4) {
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_ml[(w * 16 + row) * 2]);
      float L = 0.f, wgt[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = sm_ml[(w * 16 + row) * 2];
        wgt[w] = mw == -INFINITY ? 0.f : exp2f(mw - M);
        L += sm_ml[(w * 16 + row) * 2 + 1] * wgt[w];
      }
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(sm_o + ((w * 16 + row) * 128 + lane * 4));
        acc[0] += v.x * wgt[w]; acc[1] += v.y * wgt[w]; acc[2] += v.z * wgt[w]; acc[3] += v.w * wgt[w];
      }
      const int tok = qstart + row / G, head = hk * G + row % G;
      if (p.splits > 1) {
        const size_t base = ((static_cast<size_t>(d.item) * p.hkv + hk) * p.splits + d.split) * 16 + row;
        *reinterpret_cast<float4*>(p.part_o + base * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if (lane == 0) {
          p.part_ml[base * 2] = M;
          p.part_ml[base * 2 + 1] = L;
        }
      } else {
        const float inv = L > 0.f ? 1.f / L : 0.f;
        uint2 packed;
        packed.x = pack_pair<BF16>(acc[0] * inv, acc[1] * inv);
        packed.y = pack_pair<BF16>(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(p.out) +
                                  ((static_cast<size_t>(tok) * p.hq + head) * 128 + lane * 4) * 2) = packed;
        if (p.lse && lane == 0)
          p.lse[static_cast<size_t>(tok) * p.hq + head] =
              L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
      }
    }
    // the scratch area is rewritten by the next unit; after the barrier all four warps read the same
    // abort flag, so they leave together if any wait of any of them ran out
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*abort_flag) break;
    ok = true;
  }
}

// Combines the per-split partial results: grid (items, hkv), block 128 (lane = 4 head_dim elements
// of one row per warp pass).
template <bool BF16>
__global__ void attn_decode_merge_kernel(const DecParams p) {
  const int item = blockIdx.x, hk = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  const int qstart = p.item_qstart[item];
  const int valid_rows = p.item_ntok[item] * G;
  for (int row = warp; row < valid_rows; row += 4) {
    float M = -INFINITY;
    for (int s = 0; s < p.splits; ++s) {
      const size_t base = ((static_cast<size_t>(item) * p.hkv + hk) * p.splits + s) * 16 + row;
      M = fmaxf(M, p.part_ml[base * 2]);
    }
    float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.splits; ++s) {
      const size_t base = ((static_cast<size_t>(item) * p.hkv + hk) * p.splits + s) * 16 + row;
      const float ms = p.part_ml[base * 2];
      const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
      L += p.part_ml[base * 2 + 1] * w;
      const float4 v = *reinterpret_cast<const float4*>(p.part_o + base * 128 + lane * 4);
      acc[0] += v.x * w; acc[1] += v.y * w; acc[2] += v.z * w; acc[3] += v.w * w;
    }
    const int tok = qstart + row / G, head = hk * G + row % G;
    const float inv = L > 0.f ? 1.f / L : 0.f;
    uint2 packed;
    packed.x = pack_pair<BF16>(acc[0] * inv, acc[1] * inv);
    packed.y = pack_pair<BF16>(acc[2] * inv, acc[3] * inv);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(p.out) +
                              ((static_cast<size_t>(tok) * p.hq + head) * 128 + lane * 4) * 2) = packed;
    if (p.lse && lane == 0)
      p.lse[static_cast<size_t>(tok) * p.hq + head] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
  }
}

}  // namespace mlcb

using namespace mlcb;

// Items are (sequence, query-token range) pairs with ntok * (hq / hkv) <= 16. With splits > 1 the
// caller provides fp32 scratch: part_o [items, hkv, splits, 16, 128] and part_ml [.., 16, 2].
MLCB_API int mlcb_attn_decode(const void* q, const void* kv_pages, void* out, float* lse, const int* item_seq,
                              const int* item_qstart, const int* item_ntok, const int* q_kvlen,
                              const int* page_indptr, const int* page_indices, int num_items,
                              long long q_stride, int hq, int hkv, long long num_pages, float sm_scale,
                              int dtype, int splits, float* part_o, float* part_ml, int* status,
                              cudaStream_t stream, const int* q_kvstart, const unsigned long long* tree_mask,
                              int sink, float softcap) {
  if (num_items <= 0) return 0;
  if (hq % hkv) return -1;
  const int group = hq / hkv;
  if (group > 16) return -2;
  if (splits < 1 || (splits > 1 && (!part_o || !part_ml))) return -5;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(kv_pages)) & 15)
    return -3;
  static bool attr_set[64] = {};
  if (first_use_on_device(attr_set)) {
    cudaFuncSetAttribute(attn_decode_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    cudaFuncSetAttribute(attn_decode_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    cudaFuncSetAttribute(attn_decode_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    cudaFuncSetAttribute(attn_decode_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
  }
  uint64_t dims[2] = {128, static_cast<uint64_t>(num_pages) * 2 * hkv * 16};
  uint64_t strides[1] = {256};
  uint32_t box[2] = {64, 16};
  const CUtensorMap* mkv = get_tensor_map(kv_pages, 2, 2, dims, strides, box, 1);
  if (!mkv) return -4;
  DecParams p;
  p.q = q;
  p.out = out;
  p.lse = lse;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.item_seq = item_seq;
  p.item_qstart = item_qstart;
  p.item_ntok = item_ntok;
  p.q_kvlen = q_kvlen;
  p.page_indptr = page_indptr;
  p.page_indices = page_indices;
  p.status = status;
  p.q_stride = q_stride;
  p.hq = hq;
  p.hkv = hkv;
  p.group = group;
  p.splits = splits;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.is_bf16 = dtype == 1;
  p.num_units = num_items * hkv * splits;
  p.q_kvstart = q_kvstart;
  p.tree_mask = tree_mask;
  p.sink = q_kvstart ? sink : 0;
  p.cap_pre = softcap > 0.f ? sm_scale / softcap : 0.f;
  p.cap_log2 = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  const int max_ctas = 2 * sm_count();
  dim3 grid(p.num_units < max_ctas ? p.num_units : max_ctas);
  const bool ext = q_kvstart || tree_mask || softcap > 0.f;
  if (ext) {
    if (dtype == 1)
      attn_decode_kernel<true, true><<<grid, DEC_THREADS, DEC_SMEM, stream>>>(*mkv, p);
    else
      attn_decode_kernel<false, true><<<grid, DEC_THREADS, DEC_SMEM, stream>>>(*mkv, p);
  } else if (dtype == 1) {
    attn_decode_kernel<true, false><<<grid, DEC_THREADS, DEC_SMEM, stream>>>(*mkv, p);
  } else {
    attn_decode_kernel<false, false><<<grid, DEC_THREADS, DEC_SMEM, stream>>>(*mkv, p);
  }
  count_launch();
  if (splits > 1) {
    dim3 g2(num_items, hkv);
    if (dtype == 1)
      attn_decode_merge_kernel<true><<<g2, 128, 0, stream>>>(p);
    else
      attn_decode_merge_kernel<false><<<g2, 128, 0, stream>>>(p);
    count_launch();
  }
  return static_cast<int>(cudaGetLastError());
}
