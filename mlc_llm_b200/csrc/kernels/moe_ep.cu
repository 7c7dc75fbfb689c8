// Expert parallelism: token dispatch and result combine as all-to-all exchanges over peer memory.
//
// Every rank owns a contiguous range of experts and a slice of the batch's tokens. The dispatch
// kernel sends each (token, slot) pair's hidden row straight into the receive region of the rank that
// owns the chosen expert (peer stores over NVLink), expert-major within the sender's region, together
// with the per-expert counts and the pair ids; the receiver turns the counts into the group table of
// the grouped tensor-core GEMM. The combine kernel sends every expert output row to the slot of its
// (token, slot) pair on every rank, and every rank takes the weighted sum over the k slots of all tokens:
// the tensor-parallel attention that follows wants every token on every rank, so no gather is needed.
// Buffers are written by exactly one sender per region and guarded by epoch flags (release / acquire
// at system scope); all waits are bounded.
//
// The reference has no expert parallelism (its MoE is tensor-parallel over the expert width,
// model/mixtral/mixtral_model.py:144-145); routing semantics follow op/moe_misc.py.
#include "common.cuh"

namespace mlcb {

struct EpParams {
  int world, rank, e_local, k, hidden, cap, epoch, pairs;
  const unsigned long long* disp_x;     // [world] rows  [world(src)][cap][hidden]
  const unsigned long long* disp_meta;  // [world] ints  [world(src)][e_local + 1]: rows per local expert, total
  const unsigned long long* disp_pair;  // [world] ints  [world(src)][cap]: pair id of each row at its home rank
  const unsigned long long* disp_flag;  // [world] ints  [world(src)]
  const unsigned long long* comb_y;     // [world] rows  [pairs of all ranks][hidden]
  const unsigned long long* comb_flag;  // [world] ints  [world(expert rank)]
  int* done_counter;                    // local, zero between launches
  int* status;
  // The call number of an exchange lives in device memory, so that a captured forward stays valid when it is
  // replayed: every kernel of a call uses *epoch_base + epoch, and the call's last kernel (the flag wait of the
  // combine) moves *epoch_base on. A null epoch_base means `epoch` is the absolute number.
  int* epoch_base;
  int pair_base;                        // global id of this rank's first (token, slot) pair
  __device__ __forceinline__ int call_epoch() const { return epoch + (epoch_base ? *epoch_base : 0); }
};

// One warp per (token, slot) pair.
template <typename T>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const T* __restrict__ x, const int* __restrict__ experts, const int* __restrict__ sorted_pos,
                   const int* __restrict__ offsets, const EpParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x * 8 + warp;
  if (pair < p.pairs) {
    const int e = experts[pair];
    const int dst = e / p.e_local;
    const int row = sorted_pos[pair] - offsets[dst * p.e_local];
    if (row < p.cap) {
      const int token = pair / p.k;
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(token) * p.hidden);
      uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.disp_x[dst]) +
                                            (static_cast<size_t>(p.rank) * p.cap + row) * p.hidden * sizeof(T));
      for (int v = lane; v < p.hidden / 8; v += 32) out[v] = src[v];
      if (lane == 0) reinterpret_cast<int*>(p.disp_pair[dst])[p.rank * p.cap + row] = p.pair_base + pair;
    } else if (lane == 0 && p.status) {
      atomicCAS(p.status, 0, ERR_CAPACITY);
    }
  }
  if (blockIdx.x == 0) {
    // rows per (destination rank, local expert), then the total
    for (int i = threadIdx.x; i < p.world * (p.e_local + 1); i += blockDim.x) {
      const int dst = i / (p.e_local + 1), el = i % (p.e_local + 1);
      const int first = dst * p.e_local;
      const int v = el < p.e_local ? offsets[first + el + 1] - offsets[first + el]
                                   : offsets[first + p.e_local] - offsets[first];
      reinterpret_cast<int*>(p.disp_meta[dst])[p.rank * (p.e_local + 1) + el] = v;
    }
  }
  // the last CTA to finish publishes this rank's regions to every destination
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(p.done_counter, 1);
    is_last = prev == static_cast<int>(gridDim.x) - 1;
    if (is_last) *p.done_counter = 0;
  }
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    if (threadIdx.x < p.world)
      flag_store_release_sys(reinterpret_cast<int*>(p.disp_flag[threadIdx.x]) + p.rank, p.call_epoch());
  }
}

// Receiver: wait for every sender's flag, then lay the received rows out expert by expert. A sender's region
// holds its rows expert-major, so the rows of local expert e arrive as `world` segments (one per sender).
// The table describes them in expert-major order, segment g = e * world + src: where the segment sits in the
// receive buffer (seg_src), where it goes in the compact buffer (seg_dst), how long it is (seg_cnt). The
// grouped GEMM then sees one group per local expert (group e = compact rows [group_begin[e], + group_count[e]),
// weight slab e), so every expert's weights are streamed once, not once per sender. live[0] = rows received.
__global__ void ep_build_groups_kernel(const EpParams p, int* __restrict__ group_begin, int* __restrict__ group_count,
                                       int* __restrict__ group_slab, int* __restrict__ seg_src,
                                       int* __restrict__ seg_dst, int* __restrict__ seg_cnt, int* __restrict__ live) {
  const int* flags = reinterpret_cast<const int*>(p.disp_flag[p.rank]);
  const int* meta = reinterpret_cast<const int*>(p.disp_meta[p.rank]);
  if (threadIdx.x < p.world) flag_wait_ge(flags + threadIdx.x, p.call_epoch(), nullptr, p.status, ERR_WAIT_PEER);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < p.e_local; ++e) {
      group_begin[e] = run;
      group_slab[e] = e;
      for (int src = 0; src < p.world; ++src) {
        const int* m = meta + src * (p.e_local + 1);
        int begin = src * p.cap;
        for (int i = 0; i < e; ++i) begin += __ldcg(m + i);
        const int cnt = __ldcg(m + e);
        const int g = e * p.world + src;
        seg_src[g] = begin;
        seg_dst[g] = run;
        seg_cnt[g] = cnt;
        run += cnt;
      }
      group_count[e] = run - group_begin[e];
    }
    live[0] = run;
  }
}

// One warp per compact row: copy the row (and its pair id) from its segment of the receive buffer.
template <typename T>
__global__ void __launch_bounds__(256)
ep_compact_kernel(const T* __restrict__ recv, T* __restrict__ xc, const int* __restrict__ pair_in,
                  int* __restrict__ pair_out, const int* __restrict__ seg_src, const int* __restrict__ seg_dst,
                  const int* __restrict__ seg_cnt, const int* __restrict__ live, int segments, int hidden) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  if (r >= live[0]) return;
  int g = 0;
  while (g + 1 < segments && r >= seg_dst[g] + seg_cnt[g]) ++g;  // segments are in compact-row order
  const int src_row = seg_src[g] + (r - seg_dst[g]);
  const uint4* in = reinterpret_cast<const uint4*>(recv + static_cast<size_t>(src_row) * hidden);
  uint4* out = reinterpret_cast<uint4*>(xc + static_cast<size_t>(r) * hidden);
  for (int v = lane; v < hidden / 8; v += 32) out[v] = __ldcg(in + v);
  if (lane == 0) pair_out[r] = __ldcg(pair_in + src_row);
}

// One warp per compact row: send the expert output to its pair's slot on every rank.
template <typename T>
__global__ void __launch_bounds__(256)
ep_combine_send_kernel(const T* __restrict__ y, const int* __restrict__ live, const int* __restrict__ pairs,
                       const EpParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int idx = blockIdx.x * 8 + warp;  // compact row
  // the grid covers the worst case; only the CTAs that hold rows (and CTA 0, so that the flags are always
  // written) take part in the completion count
  const int rows = live[0];
  const int ctas = max(1, (rows + 7) / 8);
  if (static_cast<int>(blockIdx.x) >= ctas) return;
  if (idx < rows) {
    const int pair = pairs[idx];
    const uint4* in = reinterpret_cast<const uint4*>(y + static_cast<size_t>(idx) * p.hidden);
    // every rank sums every token (the attention that follows wants all tokens everywhere): the row goes to
    // all ranks, at its global pair slot
    for (int v = lane; v < p.hidden / 8; v += 32) {
      const uint4 val = in[v];
      for (int dst = 0; dst < p.world; ++dst)
        reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.comb_y[dst]) +
                                 static_cast<size_t>(pair) * p.hidden * sizeof(T))[v] = val;
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(p.done_counter, 1);
    is_last = prev == ctas - 1;
    if (is_last) *p.done_counter = 0;
  }
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    if (threadIdx.x < p.world)
      flag_store_release_sys(reinterpret_cast<int*>(p.comb_flag[threadIdx.x]) + p.rank, p.call_epoch());
  }
}

// Last kernel of an exchange: waits for every expert rank's combine flag, then moves the call number on.
__global__ void ep_wait_flags_kernel(const int* flags, int n, int epoch, int* epoch_base, int* status) {
  const int want = epoch + (epoch_base ? *epoch_base : 0);
  if (threadIdx.x < n) flag_wait_ge(flags + threadIdx.x, want, nullptr, status, ERR_WAIT_PEER);
  __syncthreads();
  if (threadIdx.x == 0 && epoch_base) *epoch_base = want;
}

}  // namespace mlcb

using namespace mlcb;

struct MlcbEpArgs {
  int world, rank, e_local, k, hidden, cap, epoch, pairs;
  const unsigned long long* disp_x;
  const unsigned long long* disp_meta;
  const unsigned long long* disp_pair;
  const unsigned long long* disp_flag;
  const unsigned long long* comb_y;
  const unsigned long long* comb_flag;
  void* done_counter;
  void* status;
  void* epoch_base;
  int pair_base;
};

static EpParams to_params(const MlcbEpArgs* a) {
  EpParams p;
  p.world = a->world; p.rank = a->rank; p.e_local = a->e_local; p.k = a->k; p.hidden = a->hidden;
  p.cap = a->cap; p.epoch = a->epoch; p.pairs = a->pairs;
  p.disp_x = a->disp_x; p.disp_meta = a->disp_meta; p.disp_pair = a->disp_pair; p.disp_flag = a->disp_flag;
  p.comb_y = a->comb_y; p.comb_flag = a->comb_flag;
  p.done_counter = static_cast<int*>(a->done_counter);
  p.status = static_cast<int*>(a->status);
  p.epoch_base = static_cast<int*>(a->epoch_base);
  p.pair_base = a->pair_base;
  return p;
}

// x [tokens, hidden] local rows; experts / sorted_pos [pairs]; offsets [E + 1] from mlcb_moe_permute.
MLCB_API int mlcb_ep_dispatch(const void* x, const int* experts, const int* sorted_pos, const int* offsets,
                              const MlcbEpArgs* a, int dtype, cudaStream_t stream) {
  if (a->hidden % 8 != 0 || a->world > 8) return -1;
  const EpParams p = to_params(a);
  const int grid = p.pairs > 0 ? (p.pairs + 7) / 8 : 1;
  if (dtype == 0)
    ep_dispatch_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), experts, sorted_pos, offsets, p);
  else
    ep_dispatch_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), experts,
                                                                 sorted_pos, offsets, p);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_ep_build_groups(const MlcbEpArgs* a, int* group_begin, int* group_count, int* group_slab,
                                  int* seg_src, int* seg_dst, int* seg_cnt, int* live, cudaStream_t stream) {
  ep_build_groups_kernel<<<1, 32, 0, stream>>>(to_params(a), group_begin, group_count, group_slab, seg_src, seg_dst,
                                               seg_cnt, live);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// recv / pair_in: this rank's receive buffer [rows_max, hidden] and the pair ids of its rows; xc / pair_out: the
// compact, expert-major copy (rows [0, live[0])).
MLCB_API int mlcb_ep_compact(const void* recv, void* xc, const int* pair_in, int* pair_out, const int* seg_src,
                             const int* seg_dst, const int* seg_cnt, const int* live, int segments, int rows_max,
                             int hidden, int dtype, cudaStream_t stream) {
  if (rows_max <= 0) return 0;
  if (hidden % 8) return -1;
  const int grid = (rows_max + 7) / 8;
  if (dtype == 0)
    ep_compact_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(recv), static_cast<__half*>(xc),
                                                        pair_in, pair_out, seg_src, seg_dst, seg_cnt, live, segments,
                                                        hidden);
  else
    ep_compact_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(recv),
                                                               static_cast<__nv_bfloat16*>(xc), pair_in, pair_out,
                                                               seg_src, seg_dst, seg_cnt, live, segments, hidden);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// y [.., hidden]: expert outputs of the compact rows [0, live[0]); pairs: their global pair ids.
MLCB_API int mlcb_ep_combine_send(const void* y, const int* live, const int* pairs, const MlcbEpArgs* a, int dtype,
                                  cudaStream_t stream) {
  const EpParams p = to_params(a);
  const int grid = (p.world * p.cap + 7) / 8;
  if (dtype == 0)
    ep_combine_send_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(y), live, pairs, p);
  else
    ep_combine_send_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), live, pairs, p);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_ep_wait_flags(const int* flags, int n, int epoch, int* epoch_base, int* status,
                                cudaStream_t stream) {
  ep_wait_flags_kernel<<<1, 32, 0, stream>>>(flags, n, epoch, epoch_base, status);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
