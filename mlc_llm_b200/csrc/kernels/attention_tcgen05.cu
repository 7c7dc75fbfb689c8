// Paged-KV attention on the 5th-gen tensor cores (head_dim 128, 16-token pages, fp16 / bf16).
//
// One kernel serves prefill (ragged, causal) and decode. A CTA owns one (query tile, kv head): its
// 128 MMA rows are (token, q-head) pairs of that kv head's group -- G = hq / hkv query heads share a
// kv head, so a tile holds 128 / G tokens and K / V are fetched once for all G heads. Decode fills
// only G rows; the kernel is then bound by the KV stream, which is what the layout optimises for.
//
//   S = Q . K^T   tcgen05.mma, A = Q (smem, K-major), B = K block (smem, K-major), D in TMEM
//   softmax       one thread per row: tcgen05.ld its S row, mask, running max / sum, P -> smem (fp16)
//   O += P . V    tcgen05.mma, A = P (smem), B = V block (smem, MN-major), D accumulates in TMEM
//
// O stays in TMEM for the whole KV loop. The running maximum used for exp2 scaling is only raised
// when the true maximum exceeds it by more than 8 (log2 units), so the TMEM read-modify-write that
// rescales O is rare; the final division by the row sum makes the result exact either way.
//
// KV blocks of 64 tokens (4 pages) stream through a 2-stage ring filled by TMA tile loads (one box
// of 16 rows x 64 elements per page and per half of head_dim, 128-byte swizzle). K and V stages are
// released separately so the next K block loads while P.V still runs. Two CTAs fit per SM (112 KB
// shared memory, 256 TMEM columns each) and overlap each other's dependent phases.
//
// Roles (192 threads): warps 0-3 softmax / epilogue (thread r = row r), warp 4 TMA producer,
// warp 5 MMA issuer and TMEM owner. Every wait is bounded (see common.cuh).
//
// Reference counterpart: the FlashInfer / TIR paged-attention kernels selected by
// compiler_pass/dispatch_kv_cache_creation.py:150-243 and called through
// model/llama/llama_model.py:157-170.
#include "common.cuh"

namespace mlcb {

constexpr int ATT_D = 128;
constexpr int ATT_PAGE = 16;
constexpr int ATT_BLK = 64;                       // kv tokens per block
constexpr int ATT_Q_BYTES = 128 * ATT_D * 2;      // 32 KiB
constexpr int ATT_KV_BYTES = ATT_BLK * ATT_D * 2; // 16 KiB per K (or V) block
constexpr int ATT_P_BYTES = 128 * ATT_BLK * 2;    // 16 KiB
constexpr int ATT_STAGES = 2;
constexpr int ATT_SMEM = ATT_Q_BYTES + 2 * ATT_STAGES * ATT_KV_BYTES + ATT_P_BYTES + 1024 + 256;
constexpr int ATT_THREADS = 192;
constexpr float RESCALE_THRESHOLD = 8.f;

struct AttnTcParams {
  const void* q;            // [T, ...] row stride q_stride elements; head h at column h * 128
  void* out;                // [T, hq * 128]
  float* lse;               // [T, hq] or null (natural log)
  const int* tile_seq;      // [tiles] batch slot
  const int* tile_qstart;   // [tiles] first token (global index) of the tile
  const int* tile_ntok;     // [tiles] tokens in the tile (<= 128 / G)
  const int* q_kvlen;       // [T]
  const int* page_indptr;   // [B + 1]
  const int* page_indices;
  int* status;
  long long q_stride;
  int hq, hkv, group;
  float scale_log2;         // sm_scale * log2(e)
  int is_bf16;
  // masked variant (the EXT instantiation): a position j of the sequence is visible to query token t when
  //   j <  q_kvlen[t]:  j >= q_kvstart[t] (sliding window / chunk start) or j < sink
  //   j >= q_kvlen[t]:  bit (j - q_kvlen[t]) of tree_mask[t] is set (token-tree verification: the tree's
  //                     tokens sit behind the committed prefix, each sees its ancestors and itself)
  const int* q_kvstart;                  // [T] or null
  const unsigned long long* tree_mask;   // [T] or null
  int sink;
  float cap_pre, cap_log2;  // logit soft-capping: cap_log2 * tanh(raw * cap_pre); cap_log2 == 0 means none
};

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <bool EXT>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_kv, const AttnTcParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sq = smem;                                   // 2 halves x [128 x 128 B]
  uint8_t* sk = sq + ATT_Q_BYTES;                       // stages x 2 halves x [64 x 128 B]
  uint8_t* sv = sk + ATT_STAGES * ATT_KV_BYTES;
  uint8_t* sp = sv + ATT_STAGES * ATT_KV_BYTES;         // [128 x 128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sp + ATT_P_BYTES);
  uint64_t* k_full = bars;            // [2]
  uint64_t* v_full = bars + 2;        // [2]
  uint64_t* k_empty = bars + 4;       // [2]
  uint64_t* v_empty = bars + 6;       // [2]
  uint64_t* s_full = bars + 8;        // [2]
  uint64_t* p_full = bars + 10;       // [1]
  uint64_t* pv_done = bars + 11;      // [1]
  uint64_t* q_ready = bars + 12;      // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, hk = blockIdx.y;
  const int G = p.group;
  const int b = p.tile_seq[tile];
  const int qstart = p.tile_qstart[tile];
  const int ntok = p.tile_ntok[tile];
  const int valid_rows = ntok * G;
  int kv_max = p.q_kvlen[qstart + ntok - 1];
  // blocks of 64 positions the tile visits: all of [0, kv_max) unless a window hides a run of whole blocks
  // between the sink blocks and the first position any token of the tile still sees
  int sink_blks = 0, skip = 0;
  if (EXT) {
    if (p.tree_mask) {
      int extra = 0;
      for (int i = 0; i < ntok; ++i) extra = max(extra, 64 - __clzll(p.tree_mask[qstart + i] | 1ull));
      kv_max += extra;
    }
    if (p.q_kvstart) {
      int first = p.q_kvstart[qstart];
      for (int i = 1; i < ntok; ++i) first = min(first, p.q_kvstart[qstart + i]);
      sink_blks = (p.sink + ATT_BLK - 1) / ATT_BLK;
      skip = max(0, first / ATT_BLK - sink_blks);
    }
  }
  const int nblk = max(0, (kv_max + ATT_BLK - 1) / ATT_BLK - skip);
  auto block_of = [&](int j) { return EXT ? (j < sink_blks ? j : j + skip) : j; };
  const int* pages = p.page_indices + p.page_indptr[b];
  const int npages = p.page_indptr[b + 1] - p.page_indptr[b];

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    mbar_init(q_ready, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_kv);
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        // K block
        if (j >= ATT_STAGES) {
          ok = mbar_wait(&k_empty[s], ph ^ 1, abort_flag, p.status, ERR_WAIT_PRODUCER);
          if (!ok) break;
        }
        mbar_expect_tx(&k_full[s], ATT_KV_BYTES);
        for (int pg = 0; pg < ATT_BLK / ATT_PAGE; ++pg) {
          int pi = block_of(j) * (ATT_BLK / ATT_PAGE) + pg;
          if (pi >= npages) pi = npages - 1;  // rows past the sequence are masked by the softmax
          int page = pages[pi];
          if (page < 0) page = 0;
          const int row = ((page * 2 + 0) * p.hkv + hk) * ATT_PAGE;
          uint8_t* dst = sk + s * ATT_KV_BYTES + pg * ATT_PAGE * 128;
          tma_load_2d(dst, &tmap_kv, &k_full[s], 0, row);
          tma_load_2d(dst + ATT_KV_BYTES / 2, &tmap_kv, &k_full[s], 64, row);
        }
        // V block
        if (j >= ATT_STAGES) {
          ok = mbar_wait(&v_empty[s], ph ^ 1, abort_flag, p.status, ERR_WAIT_PRODUCER);
          if (!ok) break;
        }
        mbar_expect_tx(&v_full[s], ATT_KV_BYTES);
        for (int pg = 0; pg < ATT_BLK / ATT_PAGE; ++pg) {
          int pi = block_of(j) * (ATT_BLK / ATT_PAGE) + pg;
          if (pi >= npages) pi = npages - 1;
          int page = pages[pi];
          if (page < 0) page = 0;
          const int row = ((page * 2 + 1) * p.hkv + hk) * ATT_PAGE;
          uint8_t* dst = sv + s * ATT_KV_BYTES + pg * ATT_PAGE * 128;
          tma_load_2d(dst, &tmap_kv, &v_full[s], 0, row);
          tma_load_2d(dst + ATT_KV_BYTES / 2, &tmap_kv, &v_full[s], 64, row);
        }
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc(p.is_bf16, 128, ATT_BLK, 0, 0);
      const uint32_t idesc_pv = umma_idesc(p.is_bf16, 128, ATT_D, 0, 1);
      bool ok = mbar_wait(q_ready, 0, abort_flag, p.status, ERR_WAIT_PRODUCER);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[s], ph, abort_flag, p.status, ERR_WAIT_TMA)) return false;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (j & 1) * ATT_BLK;
#pragma unroll
        for (int kk = 0; kk < ATT_D / 16; ++kk) {
          const uint32_t half = kk >> 2, off = (kk & 3) * 32;
          const uint64_t adesc = umma_smem_desc(smem_u32(sq + half * (ATT_Q_BYTES / 2) + off), 16, 1024);
          const uint64_t bdesc =
              umma_smem_desc(smem_u32(sk + s * ATT_KV_BYTES + half * (ATT_KV_BYTES / 2) + off), 16, 1024);
          umma_f16(d_tmem, adesc, bdesc, idesc_qk, kk ? 1u : 0u);
        }
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok && nblk > 0) ok = issue_qk(0);
      if (ok && nblk > 1) ok = issue_qk(1);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        ok = mbar_wait(p_full, j & 1, abort_flag, p.status, ERR_WAIT_EPILOGUE);
        if (!ok) break;
        ok = mbar_wait(&v_full[s], ph, abort_flag, p.status, ERR_WAIT_TMA);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < ATT_BLK / 16; ++kk) {
          const uint64_t adesc = umma_smem_desc(smem_u32(sp + kk * 32), 16, 1024);
          // V: MN-major, two 64-wide atoms along head_dim (LBO), 8-row groups along kv (SBO)
          const uint64_t bdesc =
              umma_smem_desc(smem_u32(sv + s * ATT_KV_BYTES + kk * 2048), ATT_KV_BYTES / 2, 1024);
          umma_f16(tmem_o, adesc, bdesc, idesc_pv, (j | kk) ? 1u : 0u);
        }
        umma_commit(&v_empty[s]);
        umma_commit(pv_done);
        if (j + 2 < nblk) ok = issue_qk(j + 2);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue warps
    const int row = warp * 32 + lane;
    const bool row_valid = row < valid_rows;
    const bool warp_active = warp * 32 < valid_rows;
    const int tok = qstart + (row_valid ? row / G : 0);
    const int head = hk * G + (row_valid ? row % G : 0);
    // ---- stage Q (this thread's row) into the swizzled K-major layout
    {
      uint4 zero = make_uint4(0, 0, 0, 0);
      const uint4* src = reinterpret_cast<const uint4*>(
          reinterpret_cast<const uint8_t*>(p.q) + (static_cast<size_t>(tok) * p.q_stride + head * ATT_D) * 2);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint4 v = row_valid ? src[c] : zero;
        const int half = c >> 3, cc = c & 7;
        *reinterpret_cast<uint4*>(sq + half * (ATT_Q_BYTES / 2) + row * 128 + ((cc ^ (row & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);
    }
    const int kvlen = row_valid ? p.q_kvlen[tok] : 0;
    int win_start = 0;
    unsigned long long tmask = 0ull;
    if (EXT && row_valid) {
      if (p.q_kvstart) win_start = p.q_kvstart[tok];
      if (p.tree_mask) tmask = p.tree_mask[tok];
    }
    auto visible = [&](int pos) -> bool {
      if (!EXT) return pos < kvlen;
      if (pos < kvlen) return pos >= win_start || pos < p.sink;
      const int r = pos - kvlen;
      return r < 64 && ((tmask >> r) & 1ull);
    };
    float m_ref = -INFINITY;   // scaled (log2) reference maximum used for exp2
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, p.status, ERR_WAIT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float pvals[ATT_BLK];
      float mx = -INFINITY;
      if (warp_active) {
        uint32_t r0[32], r1[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + (j & 1) * ATT_BLK;
        tmem_ld32(taddr, r0);
        tmem_ld32(taddr + 32, r1);
        tmem_ld_wait();
        const int base = block_of(j) * ATT_BLK;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          float a, bq;
          if (EXT && p.cap_log2 != 0.f) {
            a = p.cap_log2 * tanh_approx(__uint_as_float(r0[c]) * p.cap_pre);
            bq = p.cap_log2 * tanh_approx(__uint_as_float(r1[c]) * p.cap_pre);
          } else {
            a = __uint_as_float(r0[c]) * p.scale_log2;
            bq = __uint_as_float(r1[c]) * p.scale_log2;
          }
          a = visible(base + c) ? a : -INFINITY;
          bq = visible(base + 32 + c) ? bq : -INFINITY;
          pvals[c] = a;
          pvals[32 + c] = bq;
          mx = fmaxf(mx, fmaxf(a, bq));
        }
      }
      // the previous P.V must be finished before P is overwritten (and before O is rescaled)
      if (j > 0) {
        ok = mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.status, ERR_WAIT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
      if (warp_active) {
        const bool grow = mx > m_ref + RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_ref, mx);
          const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
          if (j > 0) {
#pragma unroll 1
            for (int c = 0; c < ATT_D; c += 32) {
              uint32_t o[32];
              const uint32_t ta = tmem_o + (static_cast<uint32_t>(warp * 32) << 16) + c;
              tmem_ld32(ta, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(ta, o);
            }
            tmem_st_wait();
          }
          l *= alpha;
          if (m_new != -INFINITY) m_ref = m_new;
        }
        const float mr = (m_ref == -INFINITY) ? 0.f : m_ref;
        uint8_t* prow = sp + row * 128;
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float e0 = exp2f(pvals[c8 * 8 + 2 * i] - mr);
            const float e1 = exp2f(pvals[c8 * 8 + 2 * i + 1] - mr);
            l += e0 + e1;
            w[i] = pack2(e0, e1, p.is_bf16);
          }
          *reinterpret_cast<uint4*>(prow + ((c8 ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        // rows of an inactive warp contribute nothing: keep their P rows zero
        uint8_t* prow = sp + row * 128;
        if (j == 0) {
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) *reinterpret_cast<uint4*>(prow + (c8 << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l
    if (ok && nblk > 0) {
      ok = mbar_wait(pv_done, (nblk - 1) & 1, abort_flag, p.status, ERR_WAIT_MMA);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && warp_active) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) +
                      (static_cast<size_t>(tok) * p.hq + head) * ATT_D * 2;
#pragma unroll 1
      for (int c = 0; c < ATT_D; c += 32) {
        uint32_t o[32];
        if (nblk > 0) {
          tmem_ld32(tmem_o + (static_cast<uint32_t>(warp * 32) << 16) + c, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              w[k] = pack2(__uint_as_float(o[i * 8 + 2 * k]) * inv, __uint_as_float(o[i * 8 + 2 * k + 1]) * inv,
                           p.is_bf16);
            *reinterpret_cast<uint4*>(orow + c * 2 + i * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (p.lse && row_valid)
        p.lse[static_cast<size_t>(tok) * p.hq + head] =
            l > 0.f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace mlcb

using namespace mlcb;

// kv_pages: one layer's cache [num_pages, 2, hkv, 16, 128]. Tiles are (sequence, query-token range)
// pairs prepared by the caller; the grid is (tiles, hkv).
// q_kvstart / tree_mask (either may be null), sink and softcap select the masked instantiation (see
// AttnTcParams); with all of them absent the plain causal kernel runs.
MLCB_API int mlcb_attn_tc(const void* q, const void* kv_pages, void* out, float* lse, const int* tile_seq,
                          const int* tile_qstart, const int* tile_ntok, const int* q_kvlen,
                          const int* page_indptr, const int* page_indices, int num_tiles, long long q_stride,
                          int hq, int hkv, long long num_pages, float sm_scale, int dtype, int* status,
                          cudaStream_t stream, const int* q_kvstart, const unsigned long long* tree_mask,
                          int sink, float softcap) {
  if (num_tiles <= 0) return 0;
  if (hq % hkv) return -1;
  const int group = hq / hkv;
  if (group > 128 || 128 % group) return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(kv_pages)) & 15)
    return -3;
  if ((q_stride * 2) % 16) return -3;
  static bool attr_set[64] = {};
  if (first_use_on_device(attr_set)) {
    cudaFuncSetAttribute(attn_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
    cudaFuncSetAttribute(attn_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
  }
  uint64_t dims[2] = {ATT_D, static_cast<uint64_t>(num_pages) * 2 * hkv * ATT_PAGE};
  uint64_t strides[1] = {ATT_D * 2};
  uint32_t box[2] = {64, ATT_PAGE};
  const CUtensorMap* mkv = get_tensor_map(kv_pages, 2, 2, dims, strides, box, 1);
  if (!mkv) return -4;
  AttnTcParams p;
  p.q = q;
  p.out = out;
  p.lse = lse;
  p.tile_seq = tile_seq;
  p.tile_qstart = tile_qstart;
  p.tile_ntok = tile_ntok;
  p.q_kvlen = q_kvlen;
  p.page_indptr = page_indptr;
  p.page_indices = page_indices;
  p.status = status;
  p.q_stride = q_stride;
  p.hq = hq;
  p.hkv = hkv;
  p.group = group;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.is_bf16 = dtype == 1;
  p.q_kvstart = q_kvstart;
  p.tree_mask = tree_mask;
  p.sink = q_kvstart ? sink : 0;
  p.cap_pre = softcap > 0.f ? sm_scale / softcap : 0.f;
  p.cap_log2 = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  dim3 grid(num_tiles, hkv);
  if (q_kvstart || tree_mask || softcap > 0.f)
    attn_tc_kernel<true><<<grid, ATT_THREADS, ATT_SMEM, stream>>>(*mkv, p);
  else
    attn_tc_kernel<false><<<grid, ATT_THREADS, ATT_SMEM, stream>>>(*mkv, p);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
