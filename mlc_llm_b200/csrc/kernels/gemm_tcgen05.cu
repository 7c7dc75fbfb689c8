// Linear layers on the 5th-gen tensor cores:  Y[M, N] = X[M, K] . W[N, K]^T (+ bias)
//
// One persistent, warp-specialised kernel serves both serving phases and both weight formats:
//   * W dense 16-bit (fp16 / bf16), loaded by TMA straight into the 128-byte-swizzled UMMA layout;
//   * W int4 group-quantised (q4f16_1: 8 nibbles per uint32, one fp16 scale per 32 weights along K),
//     stored as tile records: the nibbles and the group scales of one 128-row x 64-k block sit in
//     4608 consecutive bytes, records of one 128-row block follow each other along K. One untiled bulk
//     copy fetches a record, "dequant" warps expand it to fp16 in the swizzled layout
//     ((nibble - 7) * scale, one rounding), and the tensor core consumes it from there.
//
// The weight tile is the UMMA "A" operand (M = 128 output features), the token tile is the "B"
// operand (N = TN tokens, 16..256), so each expanded weight tile is reused by up to 256 tokens and
// small decode batches do not pad to 128 rows. Accumulators live in TMEM (two buffers of 256
// columns, so the epilogue of one tile overlaps the main loop of the next).
//
// Roles, dense kernel (352 threads): warp 0 = TMA producer (activations + weights), warp 1 = MMA issuer
// (+TMEM owner), warps 6-9 = epilogue (TMEM -> registers -> global).
// Roles, kernels with a dequant stage (512 threads): a warp issues on scheduler (warp % 4), and the
// three single-thread control roles are serial chains of dependent instructions whose speed sets the
// pace of the whole pipeline, so they get scheduler 1 to themselves: warp 1 = MMA issuer, warp 5 = TMA
// producer of the activations, warp 9 = producer of the packed weights. Dequant group 0 = warps 0, 2,
// 3, 4, group 1 = warps 6, 7, 8, 10 (the groups take alternate K blocks), epilogue = warps 12-15.
//
// Reference counterparts: dense matmul dispatched to cuBLAS (compiler_pass/blas_dispatch.py:15-52)
// and the fused dequantize+matmul produced by compiler_pass/fuse_dequantize_matmul_ewise.py:9-85
// from quantization/group_quantization.py:390-440.
#include "common.cuh"

#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace mlcb {

constexpr int BM = 128;       // weight rows (output features) per tile == UMMA M
constexpr int BK = 64;        // K elements per pipeline stage (128 bytes of 16-bit data)
constexpr int MAX_TN = 256;   // tokens per tile == UMMA N
constexpr int STAGES = 4;     // activation / expanded-weight ring
constexpr int RAW_STAGES = 6; // packed-weight ring (q4): deeper, so TMA latency stays off the MMA loop
constexpr int X_STAGE_BYTES = MAX_TN * BK * 2;   // 32 KiB
constexpr int W_STAGE_BYTES = BM * BK * 2;       // 16 KiB
constexpr int RAW_STAGE_BYTES = BM * (BK / 2);   // 4 KiB of packed nibbles
// int4 tile record of one (128-row block, K block): [2 halves][128 rows][16 B of nibbles] then
// [128 rows][2 fp16 group scales]. Row r's first 32 weights of the block are the 16 bytes at r * 16,
// its last 32 the 16 bytes at 2048 + r * 16, its two scales the 4 bytes at 4096 + r * 4.
constexpr int Q4_REC_BYTES = BM * (BK / 2) + BM * 4;
constexpr int GEMM_THREADS = 352;      // dense kernel: warps 0-10
constexpr int GEMM_THREADS_Q4 = 512;   // kernels with a dequant stage: warps 0-15
constexpr int MAX_NST = 8;             // deepest activation / expanded-weight ring
constexpr int RING_BYTES = STAGES * (X_STAGE_BYTES + W_STAGE_BYTES);  // shared memory of that ring
constexpr int SCALE_DEPTH = 8;                   // group scales are fetched this many K blocks ahead
constexpr int SCALE_STAGE_BYTES = BM * 4;        // two fp16 scales per weight row and K block
constexpr int GEMM_SMEM = STAGES * (X_STAGE_BYTES + W_STAGE_BYTES) + RAW_STAGES * RAW_STAGE_BYTES +
                          SCALE_DEPTH * SCALE_STAGE_BYTES + 1024 + 512;

struct GemmParams {
  const void* scale;    // fp8: [N/128, K/128] fp32 block scales; int4: unused (scales travel in the tile records)
  const void* w_tiles;  // int4: tile records [ceil(rows / 128)][K / 64][Q4_REC_BYTES]
  const void* bias;     // [N] in the activation dtype, may be null
  void* y;
  int* status;
  int M, N, K;
  int ldy;              // elements
  int tn;               // tokens per tile (multiple of 16)
  int num_m_blocks, num_n_blocks;
  int out_dtype;        // 0 fp16, 1 bf16, 2 fp32
  int ab_fmt;           // 0 fp16, 1 bf16
  int splits;           // split-K factor (1 = none)
  int kb_per_split;     // K blocks handled by one work item
  int cluster_split;    // split-K siblings form one thread-block cluster and reduce through distributed shared memory
  int nst;              // ring depth: as many (activation tile + 16 KiB weight tile) stages as fit, even, <= MAX_NST
  float* workspace;     // [tiles, splits, tn, BM] fp32 partial sums (split-K only)
  int* counters;        // [tiles] arrival counters, zero between launches (split-K only)
  long long* trace;     // optional: per-role timestamps of CTA 0 (profiling aid, null = off)
  // grouped mode (mixture of experts): X rows [group_offsets[e], group_offsets[e+1]) use the weight
  // slab e, i.e. rows [e * N, (e + 1) * N) of W (and of the scales). Null = one dense problem.
  const int* group_offsets;
  int num_groups;
  // Explicit group table (expert-parallel receive layout): when group_count is set, group e covers
  // rows [group_offsets[e], group_offsets[e] + group_count[e]) and uses weight slab group_slab[e].
  const int* group_count;
  const int* group_slab;
  // ---- tensor-parallel fusion (see the "fused collectives" section below); all off when zero/null
  // Reduce-scatter epilogue: output rows go to the rank that owns them instead of to `y`.
  int rs_world, rs_rank;
  int rs_rows;                       // rows owned by each rank (multiple of 32)
  int rs_epoch;                      // call number; flags carry it, so nothing is reset
  // When set, the call number is `*epoch_base + rs_epoch` (and `*epoch_base + ag_epoch`): the base
  // lives in device memory and advances once per forward, so a captured CUDA graph of a forward can
  // be replayed with fresh call numbers.
  const int* epoch_base;
  // peer address tables live in device memory (dynamic indexing of kernel parameters would force
  // a local copy of the whole parameter block)
  const unsigned long long* rs_recv; // [world] per rank: receive buffer [world][rs_rows][N], output dtype
  const unsigned long long* rs_flag; // [world] per rank: int flags [rs_rows / 32][world]
  int* rs_count;                     // local: arrivals per 32-row chunk of the whole batch, zeroed by the last one
  void* rs_residual;                 // local: residual rows owned by this rank [rs_rows, N] (updated in place)
  const void* rs_norm_w;             // RMSNorm weight [N]
  float rs_eps, rs_w_offset;
  const unsigned long long* ag_xn;   // [world] per rank: gathered normalised activations [world * rs_rows, N]
  const unsigned long long* ag_flag; // [world] per rank: int flags [world * rs_rows / 8], one per 8-row group
  // All-gather prologue: token rows of X become readable once their 8-row group flag reaches ag_epoch.
  const int* ag_wait;
  int ag_epoch;
  // ---- all-reduce form (see ar_tail): the GEMM writes this rank's partial sums to `y`, which is this
  // rank's copy of a symmetric buffer; the kernel's tail then sums the copies of all ranks (one multimem
  // load per 16 bytes through the NVSwitch, or plain peer loads without a multicast mapping), adds the
  // residual, applies RMSNorm and leaves residual and normalised rows in local memory, on every rank.
  int ar_world, ar_rank, ar_epoch;
  const void* ar_mc;                   // multicast address of the partial-sum buffer, or null
  const unsigned long long* ar_peers;  // [world] every rank's partial-sum buffer (plain peer loads)
  const unsigned long long* ar_flags;  // [world] per rank: int arrival epochs [world]
  int* ar_counter;                     // local: CTAs of this launch that have stored their tiles
  void* ar_xn;                         // local [M, N]: normalised rows
  // CTA pairs (cta_group::2): two CTAs of a cluster share each UMMA; see gemm_kernel<.., true>.
  int pair;
};

// Where a tile lives: first weight row, first activation / output row, valid token rows, N block.
struct TileInfo {
  int w_row, x_row, m_valid, nb;
  int tile;        // linear (token block, feature block) index: split-K workspace / counter slot
  int x_load_row;  // first activation row this CTA loads (second half of the token tile for the peer CTA)
  bool dummy;      // pair mode, odd feature-block count: this CTA's half has no output
};
__device__ __forceinline__ int rs_epoch_of(const GemmParams& p) {
  return p.rs_epoch + (p.epoch_base ? __ldg(p.epoch_base) : 0);
}
__device__ __forceinline__ int ag_epoch_of(const GemmParams& p) {
  return p.ag_epoch + (p.epoch_base ? __ldg(p.epoch_base) : 0);
}
__device__ __forceinline__ int work_id(const GemmParams& p) { return p.pair ? blockIdx.x >> 1 : blockIdx.x; }
__device__ __forceinline__ int work_stride(const GemmParams& p) { return p.pair ? gridDim.x >> 1 : gridDim.x; }
__device__ __forceinline__ int feature_blocks_per_item(const GemmParams& p) {
  return p.pair ? (p.num_n_blocks + 1) >> 1 : p.num_n_blocks;
}

// `unit` counts (token block, feature block) tiles, or (token block, pair of feature blocks) in pair mode.
__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int unit) {
  TileInfo ti;
  const int per = feature_blocks_per_item(p);
  const int mbg = unit / per;
  ti.nb = unit - mbg * per;
  if (p.pair) ti.nb = 2 * ti.nb + static_cast<int>(cluster_ctarank());
  ti.dummy = ti.nb >= p.num_n_blocks;
  ti.tile = mbg * p.num_n_blocks + ti.nb;
  if (!p.group_offsets) {
    ti.w_row = ti.nb * BM;
    ti.x_row = mbg * p.tn;
    ti.m_valid = min(p.tn, p.M - ti.x_row);
    ti.x_load_row = ti.x_row + (p.pair ? static_cast<int>(cluster_ctarank()) * (p.tn >> 1) : 0);
    return ti;
  }
  int cum = 0, e = 0, begin = 0, cnt = 0;
  for (; e < p.num_groups; ++e) {
    begin = p.group_offsets[e];
    cnt = p.group_count ? p.group_count[e] : p.group_offsets[e + 1] - begin;
    const int mbs = (cnt + p.tn - 1) / p.tn;
    if (mbg < cum + mbs) break;
    cum += mbs;
  }
  const int mb = mbg - cum;
  const int slab = p.group_slab ? p.group_slab[e] : e;
  ti.w_row = slab * p.N + ti.nb * BM;
  ti.x_row = begin + mb * p.tn;
  ti.m_valid = min(p.tn, cnt - mb * p.tn);
  ti.x_load_row = ti.x_row + (p.pair ? static_cast<int>(cluster_ctarank()) * (p.tn >> 1) : 0);
  return ti;
}

// Work item `t` walks its K blocks [kb0, kb1) starting at an item-dependent offset. When many
// CTAs share one token tile (decode: a single M block) they would otherwise all fetch the same
// activation lines at the same moment; the sum over K is order-free.
__device__ __forceinline__ int rotate_k(int kb, int kb0, int kb1, int t) {
  const int n = kb1 - kb0;
  int r = (kb - kb0) + (t * 5) % n;
  if (r >= n) r -= n;
  return kb0 + r;
}

// Profiling aid: role `r` records clock64 for event slot `i` (CTA 0 only, when a buffer is given).
#ifdef MLCB_GEMM_TRACE
#define GEMM_TRACE(r, i)                                                               \
  do {                                                                                 \
    if (p.trace && blockIdx.x == 0 && (i) < 512) p.trace[(r) * 512 + (i)] = clock64(); \
  } while (0)
#else
#define GEMM_TRACE(r, i) \
  do {                   \
  } while (0)
#endif

template <typename OutT>
__device__ __forceinline__ void store_out(void* y, size_t idx, float v) {
  reinterpret_cast<OutT*>(y)[idx] = Cvt<OutT>::from_f(v);
}

// Byte address of output row `t` (feature 0). With the reduce-scatter epilogue the row lives in
// the receive buffer of the rank that owns it, in the slot of the sending rank.
__device__ __forceinline__ char* out_row_ptr(const GemmParams& p, int t, int esize) {
  if (p.rs_world == 0) return reinterpret_cast<char*>(p.y) + static_cast<size_t>(t) * p.ldy * esize;
  const int owner = t / p.rs_rows;
  const int local = t - owner * p.rs_rows;
  return reinterpret_cast<char*>(p.rs_recv[owner]) +
         (static_cast<size_t>(p.rs_rank) * p.rs_rows + local) * p.N * esize;
}

// One epilogue warp has stored its part of the 32-token chunks [first_chunk, first_chunk + nchunks)
// (global chunk indices, nchunks <= 32) of one feature tile. One system-scope fence covers all of the
// warp's stores; lanes then count one arrival per chunk, and the last of the `expected` arrivals on
// this GPU tells the owner of those rows that this rank's partial sums for the chunk are complete.
__device__ __forceinline__ void rs_signal_chunks(const GemmParams& p, int first_chunk, int nchunks,
                                                 int expected, int lane) {
  __threadfence_system();
  __syncwarp();
  if (lane < nchunks) {
    const int chunk = first_chunk + lane;
    const int prev = atomicAdd(&p.rs_count[chunk], 1);
    if (prev == expected - 1) {
      p.rs_count[chunk] = 0;
      __threadfence_system();
      const int t = chunk * 32;
      const int owner = t / p.rs_rows;
      const int local_chunk = (t - owner * p.rs_rows) >> 5;
      flag_store_release_sys(reinterpret_cast<int*>(p.rs_flag[owner]) + local_chunk * p.rs_world + p.rs_rank,
                             rs_epoch_of(p));
    }
  }
  __syncwarp();
}

template <typename T>
__device__ __forceinline__ void rs_tail_rows(const GemmParams& p, int warp, int lane, volatile int* abort_flag) {
  constexpr int VU = 4;  // 16-byte vectors in flight per operand and lane
  const int valid = max(0, min(p.rs_rows, p.M - p.rs_rank * p.rs_rows));
  const int ngroups = (valid + 7) >> 3;
  const int nvec = p.N >> 3;  // 16-byte vectors per row
  const int world = p.rs_world;
  const int* my_flags = reinterpret_cast<const int*>(p.rs_flag[p.rs_rank]);
  const char* my_recv = reinterpret_cast<const char*>(p.rs_recv[p.rs_rank]);
  T* residual = reinterpret_cast<T*>(p.rs_residual);
  const T* nw = reinterpret_cast<const T*>(p.rs_norm_w);
  const int epoch = rs_epoch_of(p);
  for (int g = blockIdx.x; g < ngroups; g += gridDim.x) {
    if (warp < 8) {
      const int row = g * 8 + warp;
      bool ok = row < valid;
      if (ok) {
        const int chunk = row >> 5;
        bool got = true;
        if (lane < world)
          got = flag_wait_ge(my_flags + chunk * world + lane, epoch, abort_flag, p.status, ERR_WAIT_PEER);
        ok = __all_sync(0xffffffffu, got);
      }
      if (ok) {
        T* res_row = residual + static_cast<size_t>(row) * p.N;
        float ss = 0.f;
        for (int v0 = lane; v0 < nvec; v0 += 32 * VU) {
          uint4 rv[VU];
          float acc[VU][8];
#pragma unroll
          for (int u = 0; u < VU; ++u) {
            const int v = v0 + 32 * u;
            rv[u] = v < nvec ? *reinterpret_cast<const uint4*>(res_row + v * 8) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int u = 0; u < VU; ++u) {
            const T* rh = reinterpret_cast<const T*>(&rv[u]);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[u][e] = Cvt<T>::to_f(rh[e]);
          }
          for (int src = 0; src < world; ++src) {
            uint4 pv[VU];
#pragma unroll
            for (int u = 0; u < VU; ++u) {
              const int v = v0 + 32 * u;
              pv[u] = v < nvec ? __ldcg(reinterpret_cast<const uint4*>(
                                     my_recv + ((static_cast<size_t>(src) * p.rs_rows + row) * p.N + v * 8) * sizeof(T)))
                               : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < VU; ++u) {
              const T* ph = reinterpret_cast<const T*>(&pv[u]);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[u][e] += Cvt<T>::to_f(ph[e]);
            }
          }
#pragma unroll
          for (int u = 0; u < VU; ++u) {
            const int v = v0 + 32 * u;
            if (v >= nvec) continue;
            uint4 ov;
            T* oh = reinterpret_cast<T*>(&ov);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              oh[e] = Cvt<T>::from_f(acc[u][e]);
              const float r = Cvt<T>::to_f(oh[e]);  // the norm sees the rounded residual
              ss += r * r;
            }
            *reinterpret_cast<uint4*>(res_row + v * 8) = ov;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / static_cast<float>(p.N) + p.rs_eps);
        const size_t grow = static_cast<size_t>(p.rs_rank) * p.rs_rows + row;  // row in the gathered batch
        for (int v0 = lane; v0 < nvec; v0 += 32 * VU) {
          uint4 rv[VU], wv[VU];
#pragma unroll
          for (int u = 0; u < VU; ++u) {
            const int v = v0 + 32 * u;
            if (v < nvec) {
              rv[u] = *reinterpret_cast<const uint4*>(res_row + v * 8);
              wv[u] = *reinterpret_cast<const uint4*>(nw + v * 8);
            }
          }
#pragma unroll
          for (int u = 0; u < VU; ++u) {
            const int v = v0 + 32 * u;
            if (v >= nvec) continue;
            const T* rh = reinterpret_cast<const T*>(&rv[u]);
            const T* wh = reinterpret_cast<const T*>(&wv[u]);
            uint4 ov;
            T* oh = reinterpret_cast<T*>(&ov);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              oh[e] = Cvt<T>::from_f(Cvt<T>::to_f(rh[e]) * inv * (Cvt<T>::to_f(wh[e]) + p.rs_w_offset));
            for (int dst = 0; dst < world; ++dst)
              *reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.ag_xn[dst]) + (grow * p.N + v * 8) * sizeof(T)) = ov;
          }
        }
      }
      __threadfence_system();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (threadIdx.x < world && g * 8 < valid)
        flag_store_release_sys(reinterpret_cast<int*>(p.ag_flag[threadIdx.x]) + ((p.rs_rank * p.rs_rows) >> 3) + g,
                               epoch);
    }
  }
}

// All-reduce tail. Every CTA of the launch has stored its tiles of this rank's partial sums when it gets
// here. (1) The last CTA of this rank to arrive tells every rank (a release store of the call number
// into slot `rank` of each rank's flag array). (2) Every CTA waits until all ranks have told this rank.
// (3) Rows are dealt to the warps of the grid: a warp sums the row over the ranks -- one
// multimem.ld_reduce per 16 bytes, reduced inside the NVSwitch with fp32 accumulation, or `world` plain
// peer loads -- adds the residual row (kept whole on every rank, updated in place), and writes the
// RMS-normalised row for the next GEMM. All waits are bounded.
template <typename T>
__device__ __forceinline__ void ar_tail_rows(const GemmParams& p, int warp, int lane, volatile int* abort_flag) {
  const int world = p.ar_world;
  const int epoch = p.ar_epoch + (p.epoch_base ? __ldg(p.epoch_base) : 0);
  if (threadIdx.x == 0) GEMM_TRACE(7, 8);
  __syncthreads();  // every output store of the CTA happens before thread 0's fence below
  if (threadIdx.x == 0) GEMM_TRACE(7, 9);
  {  // (with one rank this is the grid-wide barrier alone: a row needs the tiles of every CTA)
    if (threadIdx.x == 0) {
      __threadfence_system();
      const int prev = atomicAdd(p.ar_counter, 1);
      abort_flag[1] = (prev == static_cast<int>(gridDim.x) - 1) ? 1 : 0;
    }
    __syncthreads();
    if (abort_flag[1] && threadIdx.x < world) {
      if (threadIdx.x == 0) *p.ar_counter = 0;
      __threadfence_system();
      flag_store_release_sys(reinterpret_cast<int*>(p.ar_flags[threadIdx.x]) + p.ar_rank, epoch);
    }
    if (warp == 0) {
      const int* mine = reinterpret_cast<const int*>(p.ar_flags[p.ar_rank]);
      if (lane < world) flag_wait_ge(mine + lane, epoch, abort_flag, p.status, ERR_WAIT_PEER);
    }
    __syncthreads();
    if (threadIdx.x == 0) GEMM_TRACE(7, 10);
    if (*abort_flag) return;
  }
  // Rows are dealt to the CTAs (row = blockIdx.x, + gridDim.x, ...), RB rows at a time, so that every SM
  // pulls its share through the switch at once and every thread has several loads in flight: a thread
  // owns the 16-byte vectors threadIdx.x, + blockDim.x, ... of each row; the row's sum of squares is
  // reduced over the CTA through shared memory.
  const int nvec = p.N >> 3;  // 16-byte vectors per row
  T* residual = reinterpret_cast<T*>(p.rs_residual);
  T* xn = reinterpret_cast<T*>(p.ar_xn);
  const T* nw = reinterpret_cast<const T*>(p.rs_norm_w);
  const bool use_mc = p.ar_mc != nullptr && world > 1;
  constexpr int RB = 4;    // rows per round
  constexpr int VPT = 2;   // vectors per thread, row and pass (a wider row takes more passes)
  __shared__ float ar_ss[RB][17];
  const int nwarps = blockDim.x >> 5;
  for (int row0 = blockIdx.x * RB; row0 < p.M; row0 += gridDim.x * RB) {
    float ss[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) ss[r] = 0.f;
    for (int vb = threadIdx.x; vb < nvec; vb += blockDim.x * VPT) {
      uint4 rv[RB][VPT], sv[RB][VPT];
#pragma unroll
      for (int r = 0; r < RB; ++r)
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
          const int v = vb + u * blockDim.x;
          const bool live = row0 + r < p.M && v < nvec;
          const size_t off = static_cast<size_t>(row0 + r) * p.N + v * 8;
          rv[r][u] = live ? *reinterpret_cast<const uint4*>(residual + off) : make_uint4(0, 0, 0, 0);
          sv[r][u] = make_uint4(0, 0, 0, 0);
          if (!live) continue;
          if (use_mc) {
            const char* src = reinterpret_cast<const char*>(p.ar_mc) + off * sizeof(T);
            if (p.out_dtype == 0)
              asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                           : "=r"(sv[r][u].x), "=r"(sv[r][u].y), "=r"(sv[r][u].z), "=r"(sv[r][u].w)
                           : "l"(src));
            else
              asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                           : "=r"(sv[r][u].x), "=r"(sv[r][u].y), "=r"(sv[r][u].z), "=r"(sv[r][u].w)
                           : "l"(src));
          }
        }
      if (!use_mc) {
        // plain peer loads; the sum over the ranks is rounded to the storage type, as an all-reduce of
        // 16-bit tensors is
#pragma unroll
        for (int r = 0; r < RB; ++r)
#pragma unroll
          for (int u = 0; u < VPT; ++u) {
            const int v = vb + u * blockDim.x;
            if (row0 + r >= p.M || v >= nvec) continue;
            const size_t off = static_cast<size_t>(row0 + r) * p.N + v * 8;
            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int q = 0; q < world; ++q) {
              const uint4 pv = __ldcg(reinterpret_cast<const uint4*>(
                  reinterpret_cast<const char*>(p.ar_peers[q]) + off * sizeof(T)));
              const T* ph = reinterpret_cast<const T*>(&pv);
#pragma unroll
              for (int e = 0; e < 8; ++e) sum[e] += Cvt<T>::to_f(ph[e]);
            }
            T* sh = reinterpret_cast<T*>(&sv[r][u]);
#pragma unroll
            for (int e = 0; e < 8; ++e) sh[e] = Cvt<T>::from_f(sum[e]);
          }
      }
#pragma unroll
      for (int r = 0; r < RB; ++r)
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
          const int v = vb + u * blockDim.x;
          if (row0 + r >= p.M || v >= nvec) continue;
          const T* rh = reinterpret_cast<const T*>(&rv[r][u]);
          const T* sh = reinterpret_cast<const T*>(&sv[r][u]);
          uint4 ov;
          T* oh = reinterpret_cast<T*>(&ov);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            oh[e] = Cvt<T>::from_f(Cvt<T>::to_f(rh[e]) + Cvt<T>::to_f(sh[e]));
            const float x = Cvt<T>::to_f(oh[e]);  // the norm sees the rounded residual
            ss[r] += x * x;
          }
          *reinterpret_cast<uint4*>(residual + static_cast<size_t>(row0 + r) * p.N + v * 8) = ov;
        }
    }
#pragma unroll
    for (int r = 0; r < RB; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], o);
      if (lane == 0) ar_ss[r][warp] = ss[r];
    }
    __syncthreads();
    float inv[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      float tot = 0.f;
      for (int w = 0; w < nwarps; ++w) tot += ar_ss[r][w];
      inv[r] = rsqrtf(tot / static_cast<float>(p.N) + p.rs_eps);
    }
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 wv = *reinterpret_cast<const uint4*>(nw + v * 8);
      const T* wh = reinterpret_cast<const T*>(&wv);
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        if (row0 + r >= p.M) continue;
        const size_t off = static_cast<size_t>(row0 + r) * p.N + v * 8;
        const uint4 rv = *reinterpret_cast<const uint4*>(residual + off);  // this thread's own stores
        const T* rh = reinterpret_cast<const T*>(&rv);
        uint4 ov;
        T* oh = reinterpret_cast<T*>(&ov);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          oh[e] = Cvt<T>::from_f(Cvt<T>::to_f(rh[e]) * inv[r] * (Cvt<T>::to_f(wh[e]) + p.rs_w_offset));
        *reinterpret_cast<uint4*>(xn + off) = ov;
      }
    }
    __syncthreads();  // ar_ss is rewritten by the next round
  }
}

__device__ __forceinline__ void ar_tail(const GemmParams& p, int warp, int lane, volatile int* abort_flag) {
  if (p.out_dtype == 0) ar_tail_rows<__half>(p, warp, lane, abort_flag);
  else ar_tail_rows<__nv_bfloat16>(p, warp, lane, abort_flag);
  if (threadIdx.x == 0) GEMM_TRACE(7, 11);
}

__device__ __forceinline__ void rs_tail(const GemmParams& p, int warp, int lane, volatile int* abort_flag) {
  if (p.out_dtype == 0) rs_tail_rows<__half>(p, warp, lane, abort_flag);
  else rs_tail_rows<__nv_bfloat16>(p, warp, lane, abort_flag);
}

// Cursor over the (work item, K block) sequence of this CTA; every role advances its own copy.
// Everything that needs an integer division is computed once per work item.
struct KCursor {
  int t, kb, kb0, kb1, ka;
  TileInfo ti;
  __device__ __forceinline__ void init(const GemmParams& p, int total_kb, int num_items) {
    t = work_id(p);
    set(p, total_kb, num_items);
  }
  __device__ __forceinline__ void set(const GemmParams& p, int total_kb, int num_items) {
    if (t >= num_items) return;
    const int tile = t / p.splits;
    kb0 = (t - tile * p.splits) * p.kb_per_split;
    kb1 = min(total_kb, kb0 + p.kb_per_split);
    ti = decode_tile(p, tile);
    kb = kb0;
    ka = rotate_k(kb0, kb0, kb1, t);  // actual K block loaded at step kb (rotated start)
  }
  __device__ __forceinline__ bool valid(int num_items) const { return t < num_items; }
  __device__ __forceinline__ void next(const GemmParams& p, int total_kb, int num_items) {
    if (++kb >= kb1) {
      t += work_stride(p);
      set(p, total_kb, num_items);
    } else if (++ka >= kb1) {
      ka = kb0;
    }
  }
};

// WF: weight format. 0 = dense 16-bit, 1 = int4 groups of 32 (q4f16_1), 2 = fp8 e4m3 with one fp32
// scale per 128 x 128 block (weights expanded to the activation dtype on the way to the tensor core).
// TWO: CTA pairs. Launched as clusters of two; the pair computes 256 output features x TN tokens per
// UMMA (cta_group::2): each CTA loads its own 128-feature weight tile and HALF of the token tile, so a
// stage is 32 KiB instead of 48 and the ring is six deep; the leader (cluster rank 0) waits for both
// CTAs' tiles on its barriers, issues the MMAs, and its commits arrive on both CTAs' barriers.
template <int WF, bool TWO>
__global__ void __launch_bounds__(WF ? GEMM_THREADS_Q4 : GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
            const GemmParams p) {
  pdl_launch_dependents();      // the next kernel may be scheduled as SMs become free (it waits for this one)
  constexpr bool Q4 = WF != 0;  // "has a dequant stage"
  constexpr int W_MMA = 1;
  constexpr int W_XPROD = Q4 ? 5 : 0;
  constexpr int W_RAWPROD = 9;             // dequant kernels only
  constexpr int W_EPI0 = Q4 ? 12 : 6;      // four consecutive warps; TMEM lane quarter = warp & 3
  const int NST = p.nst;                                                 // ring depth
  const int XSB = (TWO ? p.tn >> 1 : p.tn) * BK * 2;                     // activation bytes per stage
  const uint32_t rank = TWO ? cluster_ctarank() : 0;                     // 0 = leader
  constexpr int RAW_BYTES = WF == 2 ? BM * BK : Q4_REC_BYTES;               // packed tile of one K block
  // Ring depth in the same space (int4 records carry their scales, so they also use the scale ring's
  // bytes), kept even: the two dequant groups take alternate K blocks, so with an even depth every slot
  // belongs to one group, which then observes every phase of the slot's barriers (a waiter that skipped
  // a phase could mistake an older completion for the one it needs).
  constexpr int RAW_SPACE = RAW_STAGES * RAW_STAGE_BYTES + (WF == 1 ? SCALE_DEPTH * SCALE_STAGE_BYTES : 0);
  constexpr int RAW_N = (RAW_SPACE / RAW_BYTES) & ~1;
  static_assert(RAW_N >= 2 && RAW_N <= RAW_STAGES, "packed-weight ring depth");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sx = smem;                                   // NST x XSB
  uint8_t* sw = sx + NST * XSB;                         // NST x 16 KiB
  uint8_t* sraw = smem + RING_BYTES;                    // RAW_STAGES x 4 KiB
  uint8_t* sscale = sraw + RAW_STAGES * RAW_STAGE_BYTES;  // SCALE_DEPTH x 512 B
  uint64_t* bars = reinterpret_cast<uint64_t*>(sscale + SCALE_DEPTH * SCALE_STAGE_BYTES);
  uint64_t* full = bars;                       // [NST] activation (and dense weight) tile landed
  uint64_t* empty = full + MAX_NST;            // [NST] MMA done reading the stage
  uint64_t* deq_full = empty + MAX_NST;        // [NST] expanded weight tile written
  uint64_t* raw_full = deq_full + MAX_NST;     // [RAW_STAGES] packed weight tile landed
  uint64_t* raw_empty = raw_full + RAW_STAGES; // [RAW_STAGES] dequant warps done reading it
  uint64_t* acc_full = raw_empty + RAW_STAGES; // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2]
  uint64_t* ep_bar = acc_empty + 2;            // [2] epilogue-group sync for the split-K reduction
  uint64_t* cl_bar = ep_bar + 2;               // [2] cluster split-K: all partial sums parked / all reducers done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cl_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_kb = (p.K + BK - 1) / BK;
  if (threadIdx.x == 0) GEMM_TRACE(7, 510);
  __shared__ int sh_num_items;

  if (threadIdx.x < 32) {
    // one lane per barrier index (pair mode: the leader's barriers also collect the peer CTA's arrivals)
    const int i = threadIdx.x;
    if (i < NST) {
      // full[s]: the producer's expect_tx arrival plus, with a dequant stage, one arrival per dequant warp
      // (of both CTAs in pair mode, where the leader's barrier collects everything)
      mbar_init(&full[i], Q4 ? (TWO ? 9 : 5) : 1);
      mbar_init(&empty[i], 1);
    }
    if (i < RAW_STAGES) {
      mbar_init(&raw_full[i], 1);
      mbar_init(&raw_empty[i], 4);
    }
    if (i < 2) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], TWO ? 8 : 4);
      mbar_init(&ep_bar[i], 4);
      mbar_init(&cl_bar[i], p.cluster_split ? p.splits : 1);
    }
    mbar_fence_init();
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if (p.group_offsets) {
      pdl_wait();  // the group table is written by kernels before this one
      int mbs = 0;
      for (int e = 0; e < p.num_groups; ++e) {
        const int cnt = p.group_count ? p.group_count[e] : p.group_offsets[e + 1] - p.group_offsets[e];
        mbs += (cnt + p.tn - 1) / p.tn;
      }
      sh_num_items = mbs * feature_blocks_per_item(p);
    } else {
      sh_num_items = p.num_m_blocks * feature_blocks_per_item(p) * p.splits;
    }
  }
  if (warp == W_MMA) {
    if (TWO) {
      tmem_alloc_pair(tmem_slot, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (TWO || p.cluster_split) cluster_sync_all();  // every CTA's barriers (and TMEM) exist before anyone signals a peer
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = sh_num_items;  // work items
  // Launched as a programmatic dependent, this kernel has come this far (barriers, TMEM) while its predecessor
  // was still running. Everything that reads activations, flags or tables, or writes global memory, waits here
  // for it; the packed-weight producer does not (weights are constants): it fills its ring in the meantime.
  if (!(Q4 && warp == W_RAWPROD && !p.group_offsets)) pdl_wait();

  if (warp == W_XPROD) {
    // ------------------------------------------------------------ TMA producer: activations
    // (and the dense weight tile). Ring of STAGES, recycled by the MMA.
    if (lane == 0) {
      tma_prefetch_desc(&tmap_x);
      if (!Q4) tma_prefetch_desc(&tmap_w);
    }
    // bytes credited to full[s]: in pair mode the leader's barrier counts both CTAs' tiles
    const uint32_t x_bytes = TWO ? 2u * (static_cast<uint32_t>(p.tn >> 1) * BK * 2 + (Q4 ? 0 : W_STAGE_BYTES))
                                 : static_cast<uint32_t>(p.tn) * BK * 2 + (Q4 ? 0 : W_STAGE_BYTES);
    KCursor cx;
    cx.init(p, total_kb, num_tiles);
    int gathered_row = -1;  // token tile whose rows are known to have arrived
    bool failed = false;    // no early exit: the lanes meet again at every token-tile change
    int s = 0;
    uint32_t xph = 1;  // parity of empty[s] this pass waits for (the first pass over the ring waits for nothing)
    for (uint32_t ix = 0; cx.valid(num_tiles); ++ix, cx.next(p, total_kb, num_tiles), ++s) {
      if (s == NST) {
        s = 0;
        xph ^= 1;
      }
      if (ix >= static_cast<uint32_t>(NST) && !failed) {
        const bool got = mbar_wait(&empty[s], xph, abort_flag, p.status, ERR_WAIT_PRODUCER);
        failed = !__all_sync(0xffffffffu, got);
      }
      if (p.ag_wait && cx.ti.x_row != gathered_row) {
        // rows of this token tile are pushed by their owners' kernels; one lane per 8-row group
        // (in pair mode each CTA waits for the half it loads)
        const int g0 = cx.ti.x_load_row >> 3;
        const int my_rows = TWO ? max(0, min(p.tn >> 1, cx.ti.x_row + cx.ti.m_valid - cx.ti.x_load_row))
                                : cx.ti.m_valid;
        const int ng = (my_rows + 7) >> 3;
        if (lane < ng && *abort_flag == 0)
          flag_wait_ge(p.ag_wait + g0 + lane, ag_epoch_of(p), abort_flag, p.status, ERR_WAIT_PEER);
        gathered_row = cx.ti.x_row;
        __syncwarp();
        fence_proxy_async_all();  // peer stores (generic proxy) -> TMA reads (async proxy)
        if (*abort_flag) failed = true;
      }
      if (lane == 0 && !failed) {
        GEMM_TRACE(0, ix);
        if (TWO) {
          if (rank == 0) mbar_expect_tx(&full[s], x_bytes);
          tma_load_2d_pair(sx + s * XSB, &tmap_x, &full[s], cx.ka * BK, cx.ti.x_load_row);
          if (!Q4) tma_load_2d_pair(sw + s * W_STAGE_BYTES, &tmap_w, &full[s], cx.ka * BK, cx.ti.w_row);
        } else {
          mbar_expect_tx(&full[s], x_bytes);
          tma_load_2d(sx + s * XSB, &tmap_x, &full[s], cx.ka * BK, cx.ti.x_row);
          if (!Q4) tma_load_2d(sw + s * W_STAGE_BYTES, &tmap_w, &full[s], cx.ka * BK, cx.ti.w_row);
        }
      }
    }
  } else if (Q4 && warp == W_RAWPROD) {
    // ------------------------------------------------------------ TMA producer: packed weights
    // (q4). Ring of RAW_STAGES, recycled by the dequant warps as soon as they hold the nibbles in
    // registers, so this stream runs ahead of the MMA loop.
    // (The whole warp walks the loop, lane 0 issues: uniform control flow keeps the bookkeeping cheap.)
    {
      if (WF == 2 && lane == 0) tma_prefetch_desc(&tmap_w);
      KCursor cr;
      cr.init(p, total_kb, num_tiles);
      int s = 0;
      uint32_t rph = 1;
      for (uint32_t ir = 0; cr.valid(num_tiles); ++ir, cr.next(p, total_kb, num_tiles), ++s) {
        if (s == RAW_N) {
          s = 0;
          rph ^= 1;
        }
        if (ir >= RAW_N) {
          bool ok = mbar_wait(&raw_empty[s], rph, abort_flag, p.status, ERR_WAIT_PRODUCER);
          if (!__all_sync(0xffffffffu, ok)) break;
        }
        if (lane == 0) {
          mbar_expect_tx(&raw_full[s], RAW_BYTES);
          if constexpr (WF == 2) {
            tma_load_2d(sraw + s * RAW_BYTES, &tmap_w, &raw_full[s], cr.ka * BK, cr.ti.w_row);
          } else {
            const uint8_t* rec = reinterpret_cast<const uint8_t*>(p.w_tiles) +
                                 (static_cast<size_t>(cr.ti.w_row >> 7) * total_kb + cr.ka) * Q4_REC_BYTES;
            bulk_load(sraw + s * RAW_BYTES, rec, Q4_REC_BYTES, &raw_full[s]);
          }
        }
        __syncwarp();
      }
      pdl_wait();  // (returns at once by now) this warp also takes part in the reductions and tails below
    }
  } else if (warp == W_MMA) {
    // ------------------------------------------------------------ MMA issuer
    // (pair mode: the leader CTA issues for both; the peer's warp only owns its half of the TMEM.)
    // One lane runs the loop. Its speed sets the pace of the pipeline (every tcgen05 instruction and every
    // barrier probe costs this thread some tens of cycles), so the loop carries no arithmetic that is not
    // needed: one barrier per stage, ring position and parity as counters.
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(p.ab_fmt, TWO ? 2 * BM : BM, p.tn, 0, 0);
      uint32_t tile_i = 0, it = 0;  // `it` only feeds the trace
      int s = 0;
      uint32_t ph = 0;
      const uint64_t adesc0 = umma_smem_desc(smem_u32(sw), 16, 1024);
      const uint64_t bdesc0 = umma_smem_desc(smem_u32(sx), 16, 1024);
      const uint32_t a_step = W_STAGE_BYTES >> 4, b_step = static_cast<uint32_t>(XSB) >> 4;  // per stage, 16-byte units
      uint64_t adesc = adesc0, bdesc = bdesc0;
      bool ok = true;
      auto wait_bar = [&](uint64_t* bar, uint32_t parity, int code) {
        return TWO ? mbar_wait_cluster(bar, parity, abort_flag, p.status, code)
                   : mbar_wait(bar, parity, abort_flag, p.status, code);
      };
      for (int t = work_id(p); t < num_tiles && ok; t += work_stride(p), ++tile_i) {
        const int a = tile_i & 1;
        const uint32_t aph = (tile_i >> 1) & 1;
        if (tile_i >= 2) {
          ok = wait_bar(&acc_empty[a], aph ^ 1, ERR_WAIT_EPILOGUE);
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * MAX_TN;
        const int kb0 = (t % p.splits) * p.kb_per_split;
        const int kb1 = min(total_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          GEMM_TRACE(9, it);
          // one barrier per stage: the activation tile's bytes and (with a dequant stage) the arrivals
          // of the warps that wrote the expanded weight tile
          ok = wait_bar(&full[s], ph, Q4 ? ERR_WAIT_DEQUANT : ERR_WAIT_TMA);
          if (!ok) break;
          GEMM_TRACE(2, it);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // advancing 16 elements (32 bytes) along K inside the swizzle atom: +2 in 16-byte units
            if (TWO) umma_f16_pair(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb > kb0 || kk) ? 1u : 0u);
            else umma_f16(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb > kb0 || kk) ? 1u : 0u);
          }
          GEMM_TRACE(10, it);
          if (TWO) umma_commit_pair(&empty[s]);
          else umma_commit(&empty[s]);
          GEMM_TRACE(3, it);
          adesc += a_step;
          bdesc += b_step;
          if (++s == NST) {
            s = 0;
            ph ^= 1;
            adesc = adesc0;
            bdesc = bdesc0;
          }
        }
        if (ok) {
          if (TWO) umma_commit_pair(&acc_full[a]);
          else umma_commit(&acc_full[a]);
        }
      }
    }
  } else if (Q4 && warp < 11 && warp != W_XPROD && warp != W_RAWPROD) {
    // ------------------------------------------------------------ dequant warps
    // Two groups of four warps take alternate K blocks. One iteration is a chain of long-latency steps
    // (barrier polls, shared loads, the proxy fence), longer than the tensor core needs for the block,
    // so two chains in flight keep it fed.
    {
      const int grp = warp >= 6 ? 1 : 0;
      // warps 0, 2, 3, 4 -> rows 0 / 32 / 64 / 96 of group 0; warps 6, 7, 8, 10 likewise for group 1
      const int widx = grp ? (warp == 10 ? 3 : warp - 6) : (warp == 0 ? 0 : warp - 1);
      const int row = widx * 32 + lane;  // 0..127 inside the tile
      bool ok = true;
      // K blocks this CTA walks over all of its work items (the groups need no tile bookkeeping)
      uint32_t n_iters = 0;
      for (int t = work_id(p); t < num_tiles; t += work_stride(p)) {
        const int kb0 = (t % p.splits) * p.kb_per_split;
        n_iters += static_cast<uint32_t>(min(total_kb, kb0 + p.kb_per_split) - kb0);
      }
      // fp8 only: the block scale of a K block (one fp32 per 128 x 128 block, the same word for every
      // row of the tile) is copied into shared memory SCALE_DEPTH blocks ahead with cp.async (one
      // commit group per own iteration). int4 records carry their scales with them.
      const uint32_t my_scale = smem_u32(sscale) + row * 4;
      auto fetch_scale = [&](const KCursor& c, uint32_t slot) {
        if constexpr (WF == 2) {
          const uint32_t dst = my_scale + slot * SCALE_STAGE_BYTES;
          const bool live = c.valid(num_tiles) && (c.ti.nb * BM + row < p.N);
          if (live) {
            const void* src = reinterpret_cast<const float*>(p.scale) +
                              static_cast<size_t>(c.ti.w_row / 128) * ((p.K + 127) / 128) + (c.ka >> 1);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
          } else {
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst), "r"(0u) : "memory");
          }
          asm volatile("cp.async.commit_group;" ::: "memory");
        }
      };
      auto advance2 = [&](KCursor& c) {
        if (c.valid(num_tiles)) c.next(p, total_kb, num_tiles);
        if (c.valid(num_tiles)) c.next(p, total_kb, num_tiles);
      };
      KCursor cs, cp;
      cs.init(p, total_kb, num_tiles);
      if (grp && cs.valid(num_tiles)) cs.next(p, total_kb, num_tiles);
      cp = cs;
      if constexpr (WF == 2) {
        for (int i = 0; i < SCALE_DEPTH / 2; ++i) {
          fetch_scale(cp, grp + 2 * i);
          advance2(cp);
        }
      }
      // ring positions of this group's K blocks: it = grp, grp + 2, ... (both ring depths are even)
      int s = grp, rs = grp;
      uint32_t eph = 1, rph = 0;  // parities of empty[s] (first pass: no wait) and raw_full[rs]
      for (uint32_t it = grp; it < n_iters && ok; it += 2) {
        uint32_t sc_bits = 0;
        if constexpr (WF == 2) {
          const uint32_t slot = it % SCALE_DEPTH;
          asm volatile("cp.async.wait_group %0;" ::"n"(SCALE_DEPTH / 2 - 1) : "memory");
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sc_bits) : "r"(my_scale + slot * SCALE_STAGE_BYTES) : "memory");
        }
        if constexpr (WF == 2) advance2(cs);
        if (threadIdx.x == 64) GEMM_TRACE(6, it);
        ok = mbar_wait(&raw_full[rs], rph, abort_flag, p.status, ERR_WAIT_TMA);
        ok = __all_sync(0xffffffffu, ok);  // the warp leaves together
        if (!ok) break;
        if (threadIdx.x == 64) GEMM_TRACE(4, it);
        constexpr int NWORDS = WF == 2 ? 16 : 8;  // 64 bytes of fp8 or 32 bytes of nibbles per row
        uint32_t words[NWORDS];
        if constexpr (WF == 2) {
          const uint4* raw = reinterpret_cast<const uint4*>(sraw + rs * RAW_BYTES + row * 64);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 r = raw[i];
            words[4 * i] = r.x; words[4 * i + 1] = r.y; words[4 * i + 2] = r.z; words[4 * i + 3] = r.w;
          }
        } else {
          // consecutive lanes read consecutive 16-byte words: no bank conflicts
          const uint8_t* rec = sraw + rs * RAW_BYTES;
          const uint4 r0 = *reinterpret_cast<const uint4*>(rec + row * 16);
          const uint4 r1 = *reinterpret_cast<const uint4*>(rec + BM * 16 + row * 16);
          sc_bits = *reinterpret_cast<const uint32_t*>(rec + 2 * BM * 16 + row * 4);
          words[0] = r0.x; words[1] = r0.y; words[2] = r0.z; words[3] = r0.w;
          words[4] = r1.x; words[5] = r1.y; words[6] = r1.z; words[7] = r1.w;
        }
        // The packed slot is released further down, behind the proxy fence that also publishes the
        // expanded tile: its next writer is the TMA engine (async proxy) while these reads went through
        // the generic proxy, and without a fence in between the refill was seen overtaking the reads.
        // the expanded tile may only be overwritten once the MMA that read it has finished
        if (it >= static_cast<uint32_t>(NST)) {
          ok = mbar_wait(&empty[s], eph, abort_flag, p.status, ERR_WAIT_MMA);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        if (threadIdx.x == 64 && it >= 8 && it < 500) GEMM_TRACE(7, it);
        uint8_t* dst_row = sw + s * W_STAGE_BYTES + row * 128;
        if constexpr (WF == 2) {
          const float fs = __uint_as_float(sc_bits);
#pragma unroll
          for (int w = 0; w < 8; ++w) {  // 8 fp8 values -> one 16-byte chunk of the expanded row
            uint32_t h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t pair = (words[2 * w + (j >> 1)] >> (16 * (j & 1))) & 0xffffu;
              const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(pair), __NV_E4M3);
              float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
              f.x *= fs;
              f.y *= fs;
              if (p.ab_fmt == 0) {
                const __half2 o = __float22half2_rn(f);
                h[j] = *reinterpret_cast<const uint32_t*>(&o);
              } else {
                const __nv_bfloat162 o = __float22bfloat162_rn(f);
                h[j] = *reinterpret_cast<const uint32_t*>(&o);
              }
            }
            *reinterpret_cast<uint4*>(dst_row + ((w ^ (row & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
          }
        } else {
          const __half2 sc = *reinterpret_cast<__half2*>(&sc_bits);
          // A nibble q in mantissa bits [0, 4) under exponent 0x6400 is the fp16 value 1024 + q; in bits
          // [4, 8) under exponent 0x5400 it is 64 + q. Subtracting 1031 (71) is exact, so the product
          // (q - 7) * s is rounded once. Device nibble order: pair (2j, 2j+1) of a word sits at bits
          // [4j, 4j+4) and [16+4j, 20+4j), so one shift by 8 exposes pairs 2 and 3 to the same two masks.
          const __half2 off_lo = __float2half2_rn(1031.f);
          const __half2 off_hi = __float2half2_rn(71.f);
          // bf16 models (q4bf16_1): the record's scales are bf16; (q - 7) is exact in fp16, the product with
          // the scale is formed in fp32 and rounded once to bf16
          const bool bf = p.ab_fmt == 1;
          const float fs_lo = __uint_as_float(sc_bits << 16), fs_hi = __uint_as_float(sc_bits & 0xffff0000u);
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            const __half2 s2 = __half2half2((w < 4) ? __low2half(sc) : __high2half(sc));
            const float fs = (w < 4) ? fs_lo : fs_hi;
            const uint32_t x = words[w];
            const uint32_t y = x >> 8;
            uint32_t v[4];
            v[0] = (x & 0x000f000fu) | 0x64006400u;
            v[1] = (x & 0x00f000f0u) | 0x54005400u;
            v[2] = (y & 0x000f000fu) | 0x64006400u;
            v[3] = (y & 0x00f000f0u) | 0x54005400u;
            uint32_t h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __half2 centred = __hsub2(*reinterpret_cast<__half2*>(&v[j]), (j & 1) ? off_hi : off_lo);
              if (bf) {
                float2 f = __half22float2(centred);
                f.x *= fs;
                f.y *= fs;
                const __nv_bfloat162 o = __float22bfloat162_rn(f);
                h[j] = *reinterpret_cast<const uint32_t*>(&o);
              } else {
                const __half2 hv = __hmul2(centred, s2);
                h[j] = *reinterpret_cast<const uint32_t*>(&hv);
              }
            }
            *reinterpret_cast<uint4*>(dst_row + ((w ^ (row & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[rs]);
        if (lane == 0) {
          // pair mode: the leader's barrier counts the dequant warps of both CTAs
          if (TWO) mbar_arrive_cluster(mapa_u32(smem_u32(&full[s]), 0));
          else mbar_arrive(&full[s]);
        }
        if (threadIdx.x == 64) GEMM_TRACE(5, it);
        if constexpr (WF == 2) {
          fetch_scale(cp, it % SCALE_DEPTH);  // refill the slot consumed above
          advance2(cp);
        }
        s += 2;
        if (s >= NST) {
          s -= NST;
          eph ^= 1;
        }
        rs += 2;
        if (rs >= RAW_N) {
          rs -= RAW_N;
          rph ^= 1;
        }
      }
    }
  } else if (warp >= W_EPI0 && warp < W_EPI0 + 4 && !p.cluster_split) {
    // ------------------------------------------------------------ epilogue warps
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t tile_i = 0;
    bool ok = true;
    // the accumulator buffer goes back to the MMA issuer: the leader's barrier in pair mode
    auto release_acc = [&](int a) {
      if (TWO) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[a]), 0));
      else mbar_arrive(&acc_empty[a]);
    };
    for (int t = work_id(p); t < num_tiles && ok; t += work_stride(p), ++tile_i) {
      const int sp = t % p.splits;
      const TileInfo ti = decode_tile(p, t / p.splits);
      const int tile = ti.tile;
      const int nb = ti.nb;
      const int a = tile_i & 1;
      const uint32_t aph = (tile_i >> 1) & 1;
      ok = mbar_wait(&acc_full[a], aph, abort_flag, p.status, ERR_WAIT_MMA);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below needs the whole warp
      if (!ok) break;
      if (threadIdx.x == W_EPI0 * 32) GEMM_TRACE(6, tile_i);
      tc_fence_after();
      if (ti.dummy) {  // odd feature-block count: this half of the pair tile has no output
        tc_fence_before();
        __syncwarp();
        if (lane == 0) release_acc(a);
        continue;
      }
      const int row = q * 32 + lane;     // row inside the tile
      const int n = nb * BM + row;       // output feature of this thread
      const bool n_ok = n < p.N;
      float bias = 0.f;
      if (p.bias && n_ok) {
        bias = p.ab_fmt == 0 ? __half2float(reinterpret_cast<const __half*>(p.bias)[n])
                             : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]);
      }
      const int m0 = ti.x_row;
      float* ws_tile = p.workspace + static_cast<size_t>(tile) * p.splits * p.tn * BM;
      if (p.splits > 1) {
        // park this split's partial sums: [split][token][feature] so a warp writes 128 bytes
        float* ws = ws_tile + static_cast<size_t>(sp) * p.tn * BM;
        for (int c = 0; c < p.tn; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * MAX_TN + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c + j < p.tn) ws[(c + j) * BM + row] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) release_acc(a);
        // Every split reduces its own share of the tile's tokens once all partial sums are parked,
        // so the reduction runs on `splits` SMs at once. The counter's low half counts arrivals,
        // its high half counts finished reducers; the last reducer zeroes it for the next launch.
        // Every launcher keeps tiles * splits <= CTAs in the grid whenever splits > 1, so each CTA owns at
        // most one split item and all siblings of a tile are resident at once: waiting here cannot
        // starve a sibling.
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ep_bar[0]);
        ok = mbar_wait(&ep_bar[0], 0, abort_flag, p.status, ERR_WAIT_EPILOGUE);  // two phases per tile
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (warp == W_EPI0) {
          int seen = 0;
          if (lane == 0) {
            atomicAdd(&p.counters[tile], 1);
            const unsigned long long t_start = global_timer_ns();
            uint32_t spins = 0;
            while (true) {
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.counters + tile) : "memory");
              if ((seen & 0xffff) >= p.splits || *abort_flag) break;
              if ((++spins & 0x3f) == 0 && global_timer_ns() - t_start > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                if (p.status) atomicCAS(p.status, 0, ERR_WAIT_EPILOGUE);
                break;
              }
            }
          }
          __syncwarp();
        }
        if (lane == 0) mbar_arrive(&ep_bar[1]);
        ok = mbar_wait(&ep_bar[1], tile_i & 1, abort_flag, p.status, ERR_WAIT_EPILOGUE);
        ok = ok && (*abort_flag == 0);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        {
          __threadfence();
          // this split's share of the valid tokens; thread = (token slot, 4 consecutive features)
          const int jmax = ti.m_valid;
          int per = (jmax + p.splits - 1) / p.splits;
          if (p.rs_world) per = (per + 31) & ~31;  // whole 32-token chunks, so each chunk has one reducer
          const int j_begin = min(jmax, sp * per);
          const int j_end = min(jmax, j_begin + per);
          const int f4 = lane * 4;                 // feature offset inside the tile
          const int n4 = nb * BM + f4;             // first output feature of this thread
          float b4[4] = {0.f, 0.f, 0.f, 0.f};
          if (p.bias) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (n4 + u < p.N)
                b4[u] = p.ab_fmt == 0 ? __half2float(reinterpret_cast<const __half*>(p.bias)[n4 + u])
                                      : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n4 + u]);
          }
          const int ew = warp - W_EPI0;            // epilogue warp 0..3
          for (int j0 = j_begin + ew; j0 < j_end; j0 += 16) {
            float4 acc[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] = make_float4(b4[0], b4[1], b4[2], b4[3]);
            // sixteen loads (four siblings x four tokens) in flight before the first sum
            for (int s0 = 0; s0 < p.splits; s0 += 4) {
              float4 v[4][4];
#pragma unroll
              for (int ds = 0; ds < 4; ++ds) {
                const bool s_ok = s0 + ds < p.splits;
                const float* src = ws_tile + (static_cast<size_t>(s_ok ? s0 + ds : 0) * p.tn) * BM + f4;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const int j = j0 + 4 * u;
                  v[ds][u] = (s_ok && j < j_end) ? __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(j) * BM))
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                }
              }
#pragma unroll
              for (int ds = 0; ds < 4; ++ds)
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  acc[u].x += v[ds][u].x; acc[u].y += v[ds][u].y; acc[u].z += v[ds][u].z; acc[u].w += v[ds][u].w;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int j = j0 + 4 * u;
              if (j >= j_end) continue;
              const int esize = p.out_dtype == 2 ? 4 : 2;
              char* rowp = out_row_ptr(p, m0 + j, esize);
              const float o[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
              if (n4 + 3 < p.N && (p.ldy & 3) == 0) {
                if (p.out_dtype == 0) {
                  __half2 lo = __floats2half2_rn(o[0], o[1]), hi = __floats2half2_rn(o[2], o[3]);
                  uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                  *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(rowp) + n4) = pk;
                } else if (p.out_dtype == 1) {
                  __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
                  uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                  *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(rowp) + n4) = pk;
                } else {
                  *reinterpret_cast<float4*>(reinterpret_cast<float*>(rowp) + n4) = acc[u];
                }
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  if (n4 + e >= p.N) continue;
                  if (p.out_dtype == 0) store_out<__half>(rowp, n4 + e, o[e]);
                  else if (p.out_dtype == 1) store_out<__nv_bfloat16>(rowp, n4 + e, o[e]);
                  else store_out<float>(rowp, n4 + e, o[e]);
                }
              }
            }
          }
          if (p.rs_world && j_end > j_begin)
            rs_signal_chunks(p, (m0 + j_begin) >> 5, (j_end - j_begin + 31) >> 5, p.num_n_blocks * 4, lane);
          // retire: the last reducer of the tile zeroes the counter
          __syncwarp();
          if (lane == 0) mbar_arrive(&ep_bar[0]);
          ok = mbar_wait(&ep_bar[0], 1, abort_flag, p.status, ERR_WAIT_EPILOGUE);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (warp == W_EPI0 && lane == 0) {
            const int prev = atomicAdd(&p.counters[tile], 0x10000);
            if ((prev >> 16) == p.splits - 1) p.counters[tile] = 0;
          }
        }
        continue;
      }
      // lane = output feature: a warp-wide store covers 32 consecutive features of one token.
      // Kept free of shared-memory traffic on purpose (the MMA needs that bandwidth when this
      // epilogue overlaps the next tile's main loop).
      const int jlim = ti.m_valid;
      for (int c = 0; c < p.tn; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * MAX_TN + c, r);
        tmem_ld_wait();
        if (!n_ok) continue;
        const int jn = jlim - c;  // valid tokens in this chunk (may be <= 0)
        if (jn <= 0) continue;
        // a 32-token chunk never straddles two owners (rs_rows and the tile origin are multiples of 32)
        char* rowp = out_row_ptr(p, m0 + c, p.out_dtype == 2 ? 4 : 2);
        const size_t ldy = p.rs_world ? static_cast<size_t>(p.N) : static_cast<size_t>(p.ldy);
        if (p.out_dtype == 0) {
          __half* y = reinterpret_cast<__half*>(rowp) + n;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < jn) y[static_cast<size_t>(j) * ldy] = __float2half_rn(__uint_as_float(r[j]) + bias);
        } else if (p.out_dtype == 1) {
          __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(rowp) + n;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < jn) y[static_cast<size_t>(j) * ldy] = __float2bfloat16_rn(__uint_as_float(r[j]) + bias);
        } else {
          float* y = reinterpret_cast<float*>(rowp) + n;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < jn) y[static_cast<size_t>(j) * ldy] = __uint_as_float(r[j]) + bias;
        }
      }
      if (p.rs_world && jlim > 0) rs_signal_chunks(p, m0 >> 5, (jlim + 31) >> 5, p.num_n_blocks * 4, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) release_acc(a);
      if (threadIdx.x == W_EPI0 * 32) GEMM_TRACE(7, tile_i);
    }
  }

  // ------------------------------------------------------------ split-K inside a thread-block cluster
  // The siblings of a tile are the CTAs of one cluster (cluster rank = split index), one work item
  // each. Once its main loop is done every warp of a CTA helps: the partial sums go from TMEM to the
  // CTA's own shared memory (the rings are idle by then), and each CTA reduces its share of the tile's
  // tokens by reading every sibling's copy through distributed shared memory. No global scratch, no
  // global-memory flags; remote shared memory answers slowly, so many warps keep many loads in flight.
  if (p.cluster_split) {
    constexpr int NW = Q4 ? 16 : 8;  // participating warps: the same number for each TMEM lane quarter
    __syncwarp();
    bool ok = true;
    const int t = work_id(p);
    const bool have = t < num_tiles;  // every CTA of the cluster has an item (grid = tiles * splits)
    const int sp = have ? t % p.splits : 0;
    TileInfo ti = {};
    if (have) ti = decode_tile(p, t / p.splits);
    float* stage = reinterpret_cast<float*>(smem);  // [token][feature] fp32, tn x 128
    if (have && warp < NW) {
      ok = mbar_wait(&acc_full[0], 0, abort_flag, p.status, ERR_WAIT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const int q = warp & 3, g = warp >> 2;
        const int row = q * 32 + lane;
        for (int c = g * 32; c < p.tn; c += (NW / 4) * 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c + j < p.tn) stage[(c + j) * BM + row] = __uint_as_float(r[j]);
        }
        tc_fence_before();
      }
    }
    if (threadIdx.x == 0) GEMM_TRACE(7, 2);
    asm volatile("fence.acq_rel.cluster;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0)
      for (int r2 = 0; r2 < p.splits; ++r2) mbar_arrive_cluster(mapa_u32(smem_u32(&cl_bar[0]), r2));
    if (have && warp < NW) {
      const bool got = mbar_wait_cluster(&cl_bar[0], 0, abort_flag, p.status, ERR_WAIT_EPILOGUE);
      ok = __all_sync(0xffffffffu, got && ok && *abort_flag == 0);
      if (threadIdx.x == 0) GEMM_TRACE(7, 3);
      if (ok) {
        const int nb = ti.nb, m0 = ti.x_row;
        const int jmax = ti.m_valid;
        int per = (jmax + p.splits - 1) / p.splits;
        if (p.rs_world) per = (per + 31) & ~31;  // whole 32-token chunks, so each chunk has one reducing CTA
        const int j_begin = min(jmax, sp * per);
        const int j_end = min(jmax, j_begin + per);
        const int f4 = lane * 4;                 // feature offset inside the tile
        const int n4 = nb * BM + f4;             // first output feature of this thread
        float b4[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.bias) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (n4 + u < p.N)
              b4[u] = p.ab_fmt == 0 ? __half2float(reinterpret_cast<const __half*>(p.bias)[n4 + u])
                                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n4 + u]);
        }
        const uint32_t stage_u32 = smem_u32(stage) + f4 * 4;
        // warp w takes tokens j_begin + w, + NW, ...; four tokens x four siblings = sixteen loads in flight
        for (int j0 = j_begin + warp; j0 < j_end; j0 += 4 * NW) {
          float4 acc[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[u] = make_float4(b4[0], b4[1], b4[2], b4[3]);
          for (int s0 = 0; s0 < p.splits; s0 += 4) {
            float4 v[4][4];
#pragma unroll
            for (int ds = 0; ds < 4; ++ds) {
              const bool s_ok = s0 + ds < p.splits;
              const uint32_t src = mapa_u32(stage_u32, s_ok ? s0 + ds : 0);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int j = j0 + NW * u;
                v[ds][u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (s_ok && j < j_end)
                  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                               : "=f"(v[ds][u].x), "=f"(v[ds][u].y), "=f"(v[ds][u].z), "=f"(v[ds][u].w)
                               : "r"(src + static_cast<uint32_t>(j) * (BM * 4)));
              }
            }
#pragma unroll
            for (int ds = 0; ds < 4; ++ds)
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                acc[u].x += v[ds][u].x; acc[u].y += v[ds][u].y; acc[u].z += v[ds][u].z; acc[u].w += v[ds][u].w;
              }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = j0 + NW * u;
            if (j >= j_end) continue;
            const int esize = p.out_dtype == 2 ? 4 : 2;
            char* rowp = out_row_ptr(p, m0 + j, esize);
            const float o[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
            if (n4 + 3 < p.N && (p.ldy & 3) == 0) {
              if (p.out_dtype == 0) {
                __half2 lo = __floats2half2_rn(o[0], o[1]), hi = __floats2half2_rn(o[2], o[3]);
                uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(rowp) + n4) = pk;
              } else if (p.out_dtype == 1) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
                uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(rowp) + n4) = pk;
              } else {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(rowp) + n4) = acc[u];
              }
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (n4 + e >= p.N) continue;
                if (p.out_dtype == 0) store_out<__half>(rowp, n4 + e, o[e]);
                else if (p.out_dtype == 1) store_out<__nv_bfloat16>(rowp, n4 + e, o[e]);
                else store_out<float>(rowp, n4 + e, o[e]);
              }
            }
          }
        }
        if (p.rs_world && j_end > j_begin)
          rs_signal_chunks(p, (m0 + j_begin) >> 5, (j_end - j_begin + 31) >> 5, p.num_n_blocks * NW, lane);
      }
    }
    if (threadIdx.x == 0) GEMM_TRACE(7, 4);
    // A CTA's shared memory must outlive its siblings' reads: every CTA reports when it has finished
    // reading (a CTA that gave up reports as well) and waits for all reports before it leaves.
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int r2 = 0; r2 < p.splits; ++r2) mbar_arrive_cluster(mapa_u32(smem_u32(&cl_bar[1]), r2));
      mbar_wait_cluster(&cl_bar[1], 0, abort_flag, p.status, ERR_WAIT_EPILOGUE);
      GEMM_TRACE(7, 5);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (TWO) cluster_sync_all();  // the peer's shared memory and TMEM stay valid until both are done
  if (warp == W_MMA) {
    tc_fence_after();
    if (TWO) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0) GEMM_TRACE(7, 511);

  // ------------------------------------------------------------ fused collectives: tail
  // Reduce-scatter + residual + RMSNorm + all-gather for the rows this rank owns. The main loop
  // above pushed this rank's partial sums to the owners; here each CTA takes 8-row groups of the
  // owned rows (one warp per row), waits for every rank's partial sums of the row's 32-row chunk,
  // adds them to the residual stream (kept only on the owner), normalises, and writes the
  // normalised row into every rank's gather buffer, followed by the group's flag.
  if (p.rs_world && *abort_flag == 0) rs_tail(p, warp, lane, abort_flag);
  if (p.ar_world && *abort_flag == 0) ar_tail(p, warp, lane, abort_flag);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

struct MapKey {
  uint64_t v[14];
  bool operator==(const MapKey& o) const {
    for (int i = 0; i < 14; ++i)
      if (v[i] != o.v[i]) return false;
    return true;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 14; ++i) h = (h ^ k.v[i]) * 1099511628211ull;
    return static_cast<size_t>(h);
  }
};

const CUtensorMap* get_tensor_map(const void* base, int elem_bytes, int rank, const uint64_t* dims,
                                  const uint64_t* strides_bytes, const uint32_t* box,
                                  int swizzle_128, int is_fp8) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap*, MapKeyHash> cache;
  MapKey key{};
  key.v[0] = reinterpret_cast<uint64_t>(base);
  key.v[1] = static_cast<uint64_t>(elem_bytes) | (static_cast<uint64_t>(rank) << 8) |
             (static_cast<uint64_t>(swizzle_128) << 16) | (static_cast<uint64_t>(is_fp8) << 24);
  for (int i = 0; i < rank; ++i) {
    key.v[2 + i] = dims[i];
    key.v[6 + i] = i + 1 < rank ? strides_bytes[i] : 0;
    key.v[10 + i] = box[i];
  }
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return nullptr;
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[5];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstrides[i] = strides_bytes[i];
  }
  CUtensorMap* m = new CUtensorMap;
  CUresult r = fn(m, dt, rank, const_cast<void*>(base), gdims, gstrides, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    delete m;
    return nullptr;
  }
  if (cache.size() > 65536) cache.clear();  // bounded; entries are tiny and re-creatable
  cache.emplace(key, m);
  return m;
}

long long g_launch_count = 0;

int sm_count() {
  static int n[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (n[dev] == 0) {
    cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
    if (n[dev] <= 0) n[dev] = 148;
  }
  return n[dev];
}

// Ring depth for a token tile of `tn` rows (half of it per CTA in pair mode): as many stages as fit.
static int pick_nst(int tn, bool pair) {
  const int xsb = (pair ? tn / 2 : tn) * BK * 2;
  int n = (RING_BYTES / (xsb + W_STAGE_BYTES)) & ~1;
  return n > MAX_NST ? MAX_NST : (n < 2 ? 2 : n);
}

static int pick_tn(int M) {
  if (M <= 16) return 16;
  int blocks = (M + MAX_TN - 1) / MAX_TN;
  int tn = (M + blocks - 1) / blocks;
  tn = (tn + 15) / 16 * 16;
  return tn > MAX_TN ? MAX_TN : tn;
}

}  // namespace mlcb

using namespace mlcb;

static long long* g_gemm_trace = nullptr;
// Debug hook: device buffer of 12 x 512 int64 that receives CTA 0's role timestamps (null = off;
// only builds with MLCB_GEMM_TRACE record anything).
MLCB_API void mlcb_gemm_set_trace(long long* buf) { g_gemm_trace = buf; }

// Returns 0 on success, a negative value for a rejected shape, a positive CUDA error otherwise.
// x: [M, K] row-major (ldx elements) fp16/bf16.  w: dense [N, K] (same dtype) or, with
// scale != nullptr, int4 tile records [ceil(N / 128)][K / 64][4608 bytes] (nibbles in device order
// and fp16 group scales interleaved per 128-row x 64-k block, see Q4_REC_BYTES; `scale` only selects
// the format and is not read).
// Arguments of the fused tensor-parallel forms (mirrored by a ctypes structure on the Python side).
struct MlcbFusedArgs {
  int rs_world, rs_rank, rs_rows, rs_epoch;
  const unsigned long long* rs_recv;  // device arrays of `rs_world` peer addresses
  const unsigned long long* rs_flag;
  void* rs_count;
  void* rs_residual;
  const void* rs_norm_w;
  float rs_eps, rs_w_offset;
  const unsigned long long* ag_xn;
  const unsigned long long* ag_flag;
  const void* ag_wait;
  int ag_epoch, reserved;
  const int* epoch_base;  // optional device word added to rs_epoch / ag_epoch (CUDA-graph replays)
  // all-reduce form (ar_world > 0; uses rs_residual, rs_norm_w, rs_eps, rs_w_offset as well): `y` must be
  // this rank's partial-sum buffer
  int ar_world, ar_rank, ar_epoch, ar_pad;
  const void* ar_mc;
  const unsigned long long* ar_peers;
  const unsigned long long* ar_flags;
  void* ar_counter;
  void* ar_xn;
};

// CTA-pair kernels: MLCB_GEMM_PAIR = "0" never, "1" every weight format, unset = dense 16-bit weights
// only (measured: +5..18 % on dense shapes; with a dequant stage the leader has to wait for both CTAs'
// expanded tiles every K block and the pair form is slower than two independent CTAs).
static int g_pair_mode = -1;  // -1 unread, 0 off, 1 all formats, 2 dense only
static bool pair_mode_enabled(int wf) {
  if (g_pair_mode < 0) {
    const char* e = getenv("MLCB_GEMM_PAIR");
    g_pair_mode = !e ? 2 : (e[0] == '1' ? 1 : 0);
  }
  return g_pair_mode == 1 || (g_pair_mode == 2 && wf == 0);
}
// Test hook: 1 = every format, 0 = off, 2 = default policy.
MLCB_API void mlcb_gemm_set_pair_mode(int mode) { g_pair_mode = mode; }

// Split-K reduction inside thread-block clusters (MLCB_GEMM_CLUSTER_SPLIT=0 falls back to the
// reduction through global scratch, which the CTA-pair kernels and the allocation-free entry point use).
static int g_cluster_split = -1;
// MLCB_PDL=1 launches the GEMMs as programmatic dependents of their predecessors (set-up and packed-weight
// prefetch overlap the predecessor's tail). Off by default: on the serving benchmark it measured within noise of
// the ordinary launches (15 322 vs 15 293 tok/s on one B200; the decode step's kernels fill all SMs to their end, so
// there is little tail to overlap), and ordinary launches keep the ordering rules simple.
static bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("MLCB_PDL");
    on = (e && e[0] == '1') ? 1 : 0;
  }
  return on == 1;
}

static bool cluster_split_enabled() {
  if (g_cluster_split < 0) {
    const char* e = getenv("MLCB_GEMM_CLUSTER_SPLIT");
    g_cluster_split = (e && e[0] == '0') ? 0 : 1;
  }
  return g_cluster_split == 1;
}
MLCB_API void mlcb_gemm_set_cluster_split(int on) { g_cluster_split = on ? 1 : 0; }

// How many clusters of `size` CTAs of the single-CTA kernel the current device holds at once (cached).
static int max_active_clusters(int wf, int size) {
  static int cache[64][3][9] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (size < 1 || size > 8) return 0;
  int& slot = cache[dev][wf][size];
  if (slot == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(size * 64);
    cfg.blockDim = dim3(wf ? GEMM_THREADS_Q4 : GEMM_THREADS);
    cfg.dynamicSmemBytes = GEMM_SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t err = wf == 1   ? cudaOccupancyMaxActiveClusters(&n, gemm_kernel<1, false>, &cfg)
                      : wf == 2 ? cudaOccupancyMaxActiveClusters(&n, gemm_kernel<2, false>, &cfg)
                                : cudaOccupancyMaxActiveClusters(&n, gemm_kernel<0, false>, &cfg);
    if (err != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    slot = n > 0 ? n : -1;
  }
  return slot > 0 ? slot : 0;
}
MLCB_API int mlcb_gemm_max_active_clusters(int wf, int size) { return max_active_clusters(wf, size); }

static int gemm_launch(const void* x, const void* w, const void* scale, const void* bias, void* y,
                       int M, int N, int K, int ldx, int ldy, int ab_fmt, int out_dtype,
                       int* status, float* workspace, long long workspace_bytes, int* counters,
                       int num_counters, cudaStream_t stream, const MlcbFusedArgs* f, int wf_hint = 0) {
  if (M <= 0 || N <= 0) return 0;
  const bool rs = f && f->rs_world > 0;
  if (f && f->ar_world > 0 && (f->ar_world > 8 || N % 8 != 0 || out_dtype > 1 || ldy != N || rs || !f->ar_xn ||
                              !f->rs_residual || !f->rs_norm_w || !f->ar_flags || !f->ar_counter || !f->ar_peers))
    return -5;
  if (rs && (f->rs_world > 8 || f->rs_rows % 32 != 0 || N % 8 != 0 || out_dtype > 1 ||
             static_cast<long long>(f->rs_rows) * f->rs_world < M))
    return -5;
  const int wf = scale == nullptr ? 0 : ((wf_hint == 2 || (f && f->reserved == 2)) ? 2 : 1);
  const bool q4 = wf == 1;
  if (K % 8 != 0 || ldx % 8 != 0) return -1;
  if (q4 && K % 64 != 0) return -2;  // (scales in the tile records are in the activation dtype)
  if (wf == 2 && K % 64 != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -3;
  static bool attr_set[64] = {};
  if (first_use_on_device(attr_set)) {
    cudaFuncSetAttribute(gemm_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(gemm_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(gemm_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(gemm_kernel<0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(gemm_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(gemm_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
  }
  GemmParams p = {};
  p.scale = scale;
  p.w_tiles = q4 ? w : nullptr;
  p.bias = bias;
  p.y = y;
  p.status = status;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.tn = pick_tn(M);
  if (rs) p.tn = (p.tn + 31) & ~31;  // 32-token chunks must not straddle tiles
  // CTA pairs: each CTA loads half of the token tile, so the tile must split into two halves of whole
  // swizzle atoms; tiny batches stay on the single-CTA kernel.
  const bool pair = pair_mode_enabled(wf) && M > 32;
  if (pair) p.tn = (p.tn + 31) & ~31;
  p.pair = pair ? 1 : 0;
  p.nst = pick_nst(p.tn, pair);
  p.num_m_blocks = (M + p.tn - 1) / p.tn;
  p.num_n_blocks = (N + BM - 1) / BM;
  p.out_dtype = out_dtype;
  p.ab_fmt = ab_fmt;
  if (f) {
    p.rs_world = f->rs_world;
    p.rs_rank = f->rs_rank;
    p.rs_rows = f->rs_rows;
    p.rs_epoch = f->rs_epoch;
    p.rs_recv = f->rs_recv;
    p.rs_flag = f->rs_flag;
    p.ag_xn = f->ag_xn;
    p.ag_flag = f->ag_flag;
    p.rs_count = static_cast<int*>(f->rs_count);
    p.rs_residual = f->rs_residual;
    p.rs_norm_w = f->rs_norm_w;
    p.rs_eps = f->rs_eps;
    p.rs_w_offset = f->rs_w_offset;
    p.ag_wait = static_cast<const int*>(f->ag_wait);
    p.ag_epoch = f->ag_epoch;
    p.epoch_base = f->epoch_base;
    p.ar_world = f->ar_world;
    p.ar_rank = f->ar_rank;
    p.ar_epoch = f->ar_epoch;
    p.ar_mc = f->ar_mc;
    p.ar_peers = f->ar_peers;
    p.ar_flags = f->ar_flags;
    p.ar_counter = static_cast<int*>(f->ar_counter);
    p.ar_xn = f->ar_xn;
  }
  // split-K when the output tiles alone cannot fill the GPU (decode-sized M with a narrow N)
  {
    const int tiles = p.num_m_blocks * p.num_n_blocks;
    const int total_kb = (K + BK - 1) / BK;
    int splits = 1;
    // work items that exist without splitting, and the CTAs (or CTA pairs) that can take one each
    const int units = pair ? p.num_m_blocks * ((p.num_n_blocks + 1) / 2) : tiles;
    const int workers = pair ? sm_count() / 2 : sm_count();
    if (workspace && counters && units * 2 <= workers && tiles <= num_counters) {
      int max_splits = workers / units;
      if (max_splits > 8) max_splits = 8;
      if (max_splits > total_kb / 4) max_splits = total_kb / 4;
      if (max_splits < 1) max_splits = 1;
      while (max_splits > 1 && static_cast<long long>(tiles) * max_splits * p.tn * BM * 4 > workspace_bytes)
        --max_splits;
      // A K block costs a CTA about 0.31 us, the reduction over the siblings about 6 us whatever their
      // number (measured on B200): split only where the shorter main loop pays for it, and no further
      // than it pays.
      float best = total_kb * 0.31f;
      for (int sp = 2; sp <= max_splits; ++sp) {
        const float cost = ((total_kb + sp - 1) / sp) * 0.31f + 6.0f;
        if (cost < best - 1.0f) {
          best = cost;
          splits = sp;
        }
      }
    }
    p.kb_per_split = (total_kb + splits - 1) / splits;
    p.splits = (total_kb + p.kb_per_split - 1) / p.kb_per_split;
    p.workspace = workspace;
    p.counters = counters;
    p.trace = g_gemm_trace;
    p.group_offsets = nullptr;
    p.num_groups = 0;
  }

  uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  uint64_t xs[1] = {static_cast<uint64_t>(ldx) * 2};
  uint32_t xb[2] = {BK, static_cast<uint32_t>(pair ? p.tn / 2 : p.tn)};
  const CUtensorMap* mx = get_tensor_map(x, 2, 2, xd, xs, xb, 1);
  const CUtensorMap* mw;
  if (q4) {
    mw = mx;  // tile records are fetched with untiled bulk copies; the kernel ignores this map
  } else if (wf == 2) {
    uint64_t wd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t ws[1] = {static_cast<uint64_t>(K)};
    uint32_t wb[2] = {BK, BM};
    mw = get_tensor_map(w, 1, 2, wd, ws, wb, 0);
  } else {
    uint64_t wd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t ws[1] = {static_cast<uint64_t>(K) * 2};
    uint32_t wb[2] = {BK, BM};
    mw = get_tensor_map(w, 2, 2, wd, ws, wb, 1);
  }
  if (!mx || !mw) return -4;
  if (pair) {
    const int items = p.num_m_blocks * ((p.num_n_blocks + 1) / 2) * p.splits;
    const int pairs = items < sm_count() / 2 ? items : sm_count() / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(wf ? GEMM_THREADS_Q4 : GEMM_THREADS);
    cfg.dynamicSmemBytes = GEMM_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t err;
    if (q4) err = cudaLaunchKernelEx(&cfg, gemm_kernel<1, true>, *mx, *mw, p);
    else if (wf == 2) err = cudaLaunchKernelEx(&cfg, gemm_kernel<2, true>, *mx, *mw, p);
    else err = cudaLaunchKernelEx(&cfg, gemm_kernel<0, true>, *mx, *mw, p);
    count_launch();
    return static_cast<int>(err != cudaSuccess ? err : cudaGetLastError());
  }
  // Clusters of `splits` CTAs: only as many as the GPU can hold at once (the clusters of a second wave
  // would double the run time); with fewer, split less or fall back to the reduction through global scratch.
  if (p.splits > 1 && cluster_split_enabled()) {
    const int out_tiles = p.num_m_blocks * p.num_n_blocks;
    const int total_kb = (K + BK - 1) / BK;
    int sp = p.splits;
    while (sp > 1 && max_active_clusters(wf, sp) < out_tiles) --sp;
    if (sp > 1 && sp != p.splits) {
      p.kb_per_split = (total_kb + sp - 1) / sp;
      p.splits = (total_kb + p.kb_per_split - 1) / p.kb_per_split;
    }
    if (sp <= 1 || max_active_clusters(wf, p.splits) < out_tiles) p.cluster_split = -1;  // not this time
  }
  int tiles = p.num_m_blocks * p.num_n_blocks * p.splits;
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (p.splits > 1 && cluster_split_enabled() && p.cluster_split == 0) {
    // the `splits` siblings of a tile are consecutive work items: one cluster each, reduced on chip
    p.cluster_split = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles);
    cfg.blockDim = dim3(wf ? GEMM_THREADS_Q4 : GEMM_THREADS);
    cfg.dynamicSmemBytes = GEMM_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t err;
    if (q4) err = cudaLaunchKernelEx(&cfg, gemm_kernel<1, false>, *mx, *mw, p);
    else if (wf == 2) err = cudaLaunchKernelEx(&cfg, gemm_kernel<2, false>, *mx, *mw, p);
    else err = cudaLaunchKernelEx(&cfg, gemm_kernel<0, false>, *mx, *mw, p);
    count_launch();
    return static_cast<int>(err != cudaSuccess ? err : cudaGetLastError());
  }
  p.cluster_split = 0;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(wf ? GEMM_THREADS_Q4 : GEMM_THREADS);
    cfg.dynamicSmemBytes = GEMM_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaError_t err;
    if (q4) err = cudaLaunchKernelEx(&cfg, gemm_kernel<1, false>, *mx, *mw, p);
    else if (wf == 2) err = cudaLaunchKernelEx(&cfg, gemm_kernel<2, false>, *mx, *mw, p);
    else err = cudaLaunchKernelEx(&cfg, gemm_kernel<0, false>, *mx, *mw, p);
    count_launch();
    return static_cast<int>(err != cudaSuccess ? err : cudaGetLastError());
  }
}

MLCB_API int mlcb_gemm(const void* x, const void* w, const void* scale, const void* bias, void* y,
                       int M, int N, int K, int ldx, int ldy, int ab_fmt, int out_dtype,
                       int* status, float* workspace, long long workspace_bytes, int* counters,
                       int num_counters, cudaStream_t stream) {
  return gemm_launch(x, w, scale, bias, y, M, N, K, ldx, ldy, ab_fmt, out_dtype, status, workspace,
                     workspace_bytes, counters, num_counters, stream, nullptr);
}

// Weights in fp8 e4m3 [N, K] with one fp32 scale per 128 x 128 block (`scale_inv` [ceil(N/128),
// ceil(K/128)], the "weight_scale_inv" tensor of block-scaled fp8 checkpoints); activations and the
// tensor-core math stay 16-bit. Reference: quantization/block_scale_quantization.py with the
// CUTLASS / Triton fp8 group GEMMs (op/cutlass.py, op/triton.py).
MLCB_API int mlcb_gemm_fp8(const void* x, const void* w, const void* scale_inv, const void* bias, void* y,
                           int M, int N, int K, int ldx, int ldy, int ab_fmt, int out_dtype, int* status,
                           float* workspace, long long workspace_bytes, int* counters, int num_counters,
                           cudaStream_t stream) {
  if (!scale_inv) return -2;
  return gemm_launch(x, w, scale_inv, bias, y, M, N, K, ldx, ldy, ab_fmt, out_dtype, status, workspace,
                     workspace_bytes, counters, num_counters, stream, nullptr, 2);
}

// Tensor-parallel forms of the same kernel (one launch each, collective included):
//  * reduce-scatter form (f->rs_world > 0): this rank's partial products go straight from the
//    epilogue into the receive buffers of the ranks that own the rows (peer stores over NVLink,
//    overlapping the remaining tiles); the kernel's tail then sums the partial sums of the rows it
//    owns, adds the residual, applies RMSNorm and writes the normalised rows to every rank.
//    `y` is unused.  Replaces GEMM + all-reduce + add + RMSNorm (reference:
//    model/llama/llama_model.py:211-214 with compiler_pass/fuse_add_norm.py).
//  * all-gather form (f->ag_wait != null): `x` is this rank's gather buffer; the activation
//    producer waits per 8-row group for the owners' pushes, so the GEMM starts on the rows that
//    have arrived while the rest is still in flight.
// All peer accesses are plain loads / stores from this kernel; no TMA touches peer memory.
MLCB_API int mlcb_gemm_fused(const void* x, const void* w, const void* scale, const void* bias, void* y,
                             int M, int N, int K, int ldx, int ldy, int ab_fmt, int out_dtype,
                             int* status, float* workspace, long long workspace_bytes, int* counters,
                             int num_counters, const MlcbFusedArgs* f, cudaStream_t stream) {
  return gemm_launch(x, w, scale, bias, y, M, N, K, ldx, ldy, ab_fmt, out_dtype, status, workspace,
                     workspace_bytes, counters, num_counters, stream, f);
}

// Bounded wait until the gather flags of rows [0, rows) have reached `epoch` (for consumers of a
// gather buffer that are not this library's GEMM, e.g. the row gather before the LM head).
__global__ void flag_wait_kernel(const int* flags, int groups, int epoch, const int* epoch_base, int* status) {
  if (epoch_base) epoch += __ldg(epoch_base);
  for (int g = threadIdx.x; g < groups; g += blockDim.x)
    flag_wait_ge(flags + g, epoch, nullptr, status, ERR_WAIT_PEER);
}
MLCB_API int mlcb_flag_wait(const int* flags, int rows, int epoch, const int* epoch_base, int* status,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  flag_wait_kernel<<<1, 256, 0, stream>>>(flags, (rows + 7) / 8, epoch, epoch_base, status);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// `*word += delta` in stream order: advances the device-resident call-number base of the fused
// collectives at the end of a forward (captured into the forward's CUDA graph).
__global__ void epoch_add_kernel(int* word, int delta) { *word += delta; }
MLCB_API int mlcb_epoch_add(int* word, int delta, cudaStream_t stream) {
  epoch_add_kernel<<<1, 1, 0, stream>>>(word, delta);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API long long mlcb_launch_count() { return mlcb::g_launch_count; }

// Grouped GEMM for mixture-of-experts layers: rows [offsets[e], offsets[e+1]) of x (expert-major
// permuted tokens, `total_rows` in all) are multiplied by expert e's weight slab w[e] ([N, K] dense
// 16-bit, or int4 tile records of the stacked slabs, selected by scale != nullptr); y has the same row
// order, [total_rows, N].
// `offsets` is a device array of num_groups + 1 ints; the kernel derives its tile list from it, so
// no host synchronisation is needed between routing and the expert matmuls.
static int gemm_grouped_launch(const void* x, const void* w, const void* scale, void* y, const int* offsets,
                               const int* group_count, const int* group_slab, int num_groups, int num_slabs,
                               int total_rows, int rows_hint, int N, int K, int ldx, int ldy, int ab_fmt,
                               int out_dtype, int* status, cudaStream_t stream, bool fp8 = false) {
  if (total_rows <= 0 || N <= 0 || num_groups <= 0) return 0;
  // weight format: packed int4 records (scale != null), e4m3 with fp32 128 x 128 block scales (fp8; `scale` holds
  // them, slab after slab), or dense 16-bit
  const bool q4 = scale != nullptr && !fp8;
  if (fp8 && (!scale || K % 128 != 0)) return -2;
  if (K % 8 != 0 || ldx % 8 != 0 || N % BM != 0) return -1;
  if (q4 && K % 64 != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -3;
  static bool attr_set[64] = {};
  if (first_use_on_device(attr_set)) {
    cudaFuncSetAttribute(gemm_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(gemm_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(gemm_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
  }
  GemmParams p = {};
  p.scale = scale;
  p.w_tiles = q4 ? w : nullptr;
  p.bias = nullptr;
  p.y = y;
  p.status = status;
  p.M = total_rows;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  // token tile sized for the average expert load (the box of the activation tensor map is fixed)
  const int avg = (rows_hint + num_groups - 1) / num_groups;
  p.tn = avg >= 192 ? 256 : avg >= 96 ? 128 : avg >= 48 ? 64 : avg >= 24 ? 32 : 16;
  p.nst = pick_nst(p.tn, false);
  p.num_m_blocks = 0;
  p.num_n_blocks = N / BM;
  p.out_dtype = out_dtype;
  p.ab_fmt = ab_fmt;
  p.splits = 1;
  p.kb_per_split = (K + BK - 1) / BK;
  p.workspace = nullptr;
  p.counters = nullptr;
  p.trace = nullptr;
  p.group_offsets = offsets;
  p.num_groups = num_groups;
  p.group_count = group_count;
  p.group_slab = group_slab;
  uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(total_rows)};
  uint64_t xs[1] = {static_cast<uint64_t>(ldx) * 2};
  uint32_t xb[2] = {BK, static_cast<uint32_t>(p.tn)};
  const CUtensorMap* mx = get_tensor_map(x, 2, 2, xd, xs, xb, 1);
  const CUtensorMap* mw;
  const uint64_t wrows = static_cast<uint64_t>(num_slabs) * N;
  if (q4) {
    mw = mx;  // slab e's records start at tile row e * N / 128 (N is a multiple of 128 here)
  } else if (fp8) {
    uint64_t wd[2] = {static_cast<uint64_t>(K), wrows};
    uint64_t ws[1] = {static_cast<uint64_t>(K)};
    uint32_t wb[2] = {BK, BM};
    mw = get_tensor_map(w, 1, 2, wd, ws, wb, 0);
  } else {
    uint64_t wd[2] = {static_cast<uint64_t>(K), wrows};
    uint64_t ws[1] = {static_cast<uint64_t>(K) * 2};
    uint32_t wb[2] = {BK, BM};
    mw = get_tensor_map(w, 2, 2, wd, ws, wb, 1);
  }
  if (!mx || !mw) return -4;
  // upper bound of useful CTAs: every expert may add one partial token block
  const long long max_tiles = (static_cast<long long>(rows_hint) / p.tn + num_groups) * p.num_n_blocks;
  const int grid = max_tiles < sm_count() ? static_cast<int>(max_tiles) : sm_count();
  if (q4)
    gemm_kernel<1, false><<<grid, GEMM_THREADS_Q4, GEMM_SMEM, stream>>>(*mx, *mw, p);
  else if (fp8)
    gemm_kernel<2, false><<<grid, GEMM_THREADS_Q4, GEMM_SMEM, stream>>>(*mx, *mw, p);
  else
    gemm_kernel<0, false><<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(*mx, *mw, p);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// Grouped GEMM over block-scaled e4m3 expert weights [slabs, N, K] with fp32 scales [slabs, N / 128, K / 128]
// (weights expanded to the activation dtype on the way to the tensor core; reference: the grouped fp8 GEMM of
// python/mlc_llm/op/cutlass.py:281-375). group_count / group_slab may be null (groups = consecutive slabs).
MLCB_API int mlcb_gemm_grouped_fp8(const void* x, const void* w, const void* scale, void* y, const int* group_begin,
                                   const int* group_count, const int* group_slab, int num_groups, int num_slabs,
                                   int buffer_rows, int rows_hint, int N, int K, int ldx, int ldy, int ab_fmt,
                                   int out_dtype, int* status, cudaStream_t stream) {
  return gemm_grouped_launch(x, w, scale, y, group_begin, group_count, group_slab, num_groups, num_slabs,
                             buffer_rows, rows_hint > 0 ? rows_hint : 1, N, K, ldx, ldy, ab_fmt, out_dtype, status,
                             stream, true);
}

MLCB_API int mlcb_gemm_grouped(const void* x, const void* w, const void* scale, void* y, const int* offsets,
                               int num_groups, int total_rows, int N, int K, int ldx, int ldy, int ab_fmt,
                               int out_dtype, int* status, cudaStream_t stream) {
  return gemm_grouped_launch(x, w, scale, y, offsets, nullptr, nullptr, num_groups, num_groups, total_rows,
                             total_rows, N, K, ldx, ldy, ab_fmt, out_dtype, status, stream);
}

// Grouped GEMM over an explicit group table (device arrays of num_groups ints each): group g covers
// rows [group_begin[g], group_begin[g] + group_count[g]) of x / y and uses weight slab group_slab[g]
// out of num_slabs. `buffer_rows` is the height of x / y, `rows_hint` the expected number of live
// rows (sizes the token tile and the grid; any value is safe). Used by the expert-parallel path,
// whose receive buffer holds one expert-major region per sending rank.
MLCB_API int mlcb_gemm_grouped_table(const void* x, const void* w, const void* scale, void* y,
                                     const int* group_begin, const int* group_count, const int* group_slab,
                                     int num_groups, int num_slabs, int buffer_rows, int rows_hint, int N, int K,
                                     int ldx, int ldy, int ab_fmt, int out_dtype, int* status, cudaStream_t stream) {
  return gemm_grouped_launch(x, w, scale, y, group_begin, group_count, group_slab, num_groups, num_slabs,
                             buffer_rows, rows_hint > 0 ? rows_hint : 1, N, K, ldx, ldy, ab_fmt, out_dtype, status,
                             stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in gemm_noalloc.h). Same kernel, but the split-K scratch
// is a fixed array in this translation unit instead of caller-provided memory.
// ---------------------------------------------------------------------------------------------
#include "gemm_noalloc.h"

#include <cstdio>

namespace {
// Partial sums first, tile counters behind them. In host code this name is only a handle for
// cudaGetSymbolAddress; the kernel receives the looked-up device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MLCB_NOALLOC_SCRATCH_BYTES +
                                                                 MLCB_NOALLOC_MAX_TILES * sizeof(int)];
constexpr int kMaxDevices = 64;
unsigned char* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;
thread_local char g_noalloc_err[256] = {0};

int noalloc_fail(int code, const char* fmt, long long a = 0, long long b = 0, long long c = 0) {
  snprintf(g_noalloc_err, sizeof(g_noalloc_err), fmt, a, b, c);
  return code;
}

// Encodes a 2-D tiled tensor map into caller-provided storage (no heap, no cache).
bool encode_map_local(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

MLCB_API const char* mlcb_gemm_noalloc_last_error(void) { return g_noalloc_err; }

MLCB_API int mlcb_gemm_noalloc(const void* x, const void* w, void* y, int M, int N, int K, int ldx, int ldy,
                               int ab_fmt, int* status, cudaStream_t stream) {
  g_noalloc_err[0] = 0;
  if (M <= 0 || N <= 0) return 0;
  if (!x || !w || !y || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldx < K || ldy < N || (ab_fmt != 0 && ab_fmt != 1))
    return noalloc_fail(MLCB_NOALLOC_BAD_ARGUMENT,
                        "mlcb_gemm_noalloc: bad argument (K=%lld and ldx must be multiples of 8, ldx >= K, ldy >= N=%lld)",
                        K, N);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15)
    return noalloc_fail(MLCB_NOALLOC_BAD_ARGUMENT, "mlcb_gemm_noalloc: pointers must be 16-byte aligned");

  // ---- one-time set-up per device: device address of the built-in scratch
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return noalloc_fail(static_cast<int>(err), "mlcb_gemm_noalloc: cudaGetDevice failed (%lld)", err);
  if (dev < 0 || dev >= kMaxDevices)
    return noalloc_fail(MLCB_NOALLOC_BAD_ARGUMENT, "mlcb_gemm_noalloc: device index %lld out of range", dev);
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      void* p = nullptr;
      err = cudaGetSymbolAddress(&p, g_noalloc_scratch);  // with `dev` current
      if (err != cudaSuccess || !p)
        return noalloc_fail(static_cast<int>(err ? err : cudaErrorInvalidSymbol),
                            "mlcb_gemm_noalloc: cudaGetSymbolAddress failed (%lld)", err);
      // once per device (this block runs once per device): the attribute is per device
      cudaFuncSetAttribute(gemm_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
      g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
    }
    scratch = g_noalloc_ptr[dev];
  }

  // ---- tiling and split-K, bounded by the built-in scratch
  GemmParams p = {};
  p.scale = nullptr;
  p.bias = nullptr;
  p.y = y;
  p.status = status;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.tn = pick_tn(M);
  p.nst = pick_nst(p.tn, false);
  p.num_m_blocks = (M + p.tn - 1) / p.tn;
  p.num_n_blocks = (N + BM - 1) / BM;
  p.out_dtype = ab_fmt;
  p.ab_fmt = ab_fmt;
  p.trace = nullptr;
  p.group_offsets = nullptr;
  p.num_groups = 0;
  const long long tiles = static_cast<long long>(p.num_m_blocks) * p.num_n_blocks;
  if (tiles > MLCB_NOALLOC_MAX_TILES)
    return noalloc_fail(MLCB_NOALLOC_TOO_LARGE,
                        "mlcb_gemm_noalloc: %lld output tiles exceed the built-in limit of %lld; use mlcb_gemm with "
                        "caller-provided scratch",
                        tiles, MLCB_NOALLOC_MAX_TILES);
  const int total_kb = (K + BK - 1) / BK;
  // Split K only while every (tile, split) item gets a CTA of its own (tiles * splits <= SMs): the
  // kernel's reducer waits for its sibling splits, which is only starvation-free when all of them
  // are resident at once. Problems with more than SMs / 2 tiles, or a single K block, run unsplit
  // and touch no scratch at all.
  int splits = sm_count() / static_cast<int>(tiles);
  if (splits > 8) splits = 8;
  if (splits > total_kb) splits = total_kb;
  if (splits < 1) splits = 1;
  p.kb_per_split = (total_kb + splits - 1) / splits;
  p.splits = (total_kb + p.kb_per_split - 1) / p.kb_per_split;
  const long long need = p.splits > 1 ? tiles * p.splits * p.tn * BM * 4 : 0;
  if (need > static_cast<long long>(MLCB_NOALLOC_SCRATCH_BYTES))
    return noalloc_fail(MLCB_NOALLOC_TOO_LARGE,
                        "mlcb_gemm_noalloc: split-K scratch of %lld bytes exceeds the built-in %lld bytes "
                        "(M x N too large for this entry point; use mlcb_gemm)",
                        need, MLCB_NOALLOC_SCRATCH_BYTES);
  p.workspace = reinterpret_cast<float*>(scratch);
  p.counters = reinterpret_cast<int*>(scratch + MLCB_NOALLOC_SCRATCH_BYTES);
  // the counters must start at zero; the partial sums are fully overwritten before they are read
  err = cudaMemsetAsync(p.counters, 0, static_cast<size_t>(tiles) * sizeof(int), stream);
  if (err != cudaSuccess) return noalloc_fail(static_cast<int>(err), "mlcb_gemm_noalloc: cudaMemsetAsync failed (%lld)", err);

  CUtensorMap mx, mw;
  if (!encode_map_local(&mx, x, K, M, static_cast<uint64_t>(ldx) * 2, BK, p.tn) ||
      !encode_map_local(&mw, w, K, N, static_cast<uint64_t>(K) * 2, BK, BM))
    return noalloc_fail(MLCB_NOALLOC_NO_DRIVER_ENTRY, "mlcb_gemm_noalloc: could not encode the TMA tensor maps");
  const int items = static_cast<int>(tiles) * p.splits;
  const int grid = items < sm_count() ? items : sm_count();
  gemm_kernel<0, false><<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(mx, mw, p);
  count_launch();
  err = cudaGetLastError();
  if (err != cudaSuccess) return noalloc_fail(static_cast<int>(err), "mlcb_gemm_noalloc: launch failed (%lld)", err);
  return 0;
}
