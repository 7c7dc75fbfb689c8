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

// Receiver: wait for every sender's flag, then build the group table of the grouped GEMM. Group
// g = src * e_local + e covers rows [begin, begin + count) of this rank's receive buffer and uses
// weight slab e. rows_of_src[src] = rows received from src.
__global__ void ep_build_groups_kernel(const EpParams p, int* __restrict__ group_begin, int* __restrict__ group_count,
                                       int* __restrict__ group_slab, int* __restrict__ rows_of_src) {
  const int* flags = reinterpret_cast<const int*>(p.disp_flag[p.rank]);
  const int* meta = reinterpret_cast<const int*>(p.disp_meta[p.rank]);
  if (threadIdx.x < p.world) flag_wait_ge(flags + threadIdx.x, p.call_epoch(), nullptr, p.status, ERR_WAIT_PEER);
  __syncthreads();
  for (int g = threadIdx.x; g < p.world * p.e_local; g += blockDim.x) {
    const int src = g / p.e_local, e = g % p.e_local;
    const int* m = meta + src * (p.e_local + 1);
    int begin = src * p.cap;
    for (int i = 0; i < e; ++i) begin += __ldcg(m + i);
    group_begin[g] = begin;
    group_count[g] = __ldcg(m + e);
    group_slab[g] = e;
  }
  if (threadIdx.x < p.world) rows_of_src[threadIdx.x] = __ldcg(meta + threadIdx.x * (p.e_local + 1) + p.e_local);
}

// One warp per received row: send the expert output back to its pair's slot at the home rank.
template <typename T>
__global__ void __launch_bounds__(256)
ep_combine_send_kernel(const T* __restrict__ y, const int* __restrict__ rows_of_src, const EpParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int idx = blockIdx.x * 8 + warp;  // src * cap + row
  const int src = idx / p.cap, row = idx % p.cap;
  if (src < p.world && row < min(p.cap, rows_of_src[src])) {
    const int pair = __ldcg(reinterpret_cast<const int*>(p.disp_pair[p.rank]) + idx);
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
    is_last = prev == static_cast<int>(gridDim.x) - 1;
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
                                  int* rows_of_src, cudaStream_t stream) {
  ep_build_groups_kernel<<<1, 256, 0, stream>>>(to_params(a), group_begin, group_count, group_slab, rows_of_src);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// y [world * cap, hidden]: expert outputs in the receive layout.
MLCB_API int mlcb_ep_combine_send(const void* y, const int* rows_of_src, const MlcbEpArgs* a, int dtype,
                                  cudaStream_t stream) {
  const EpParams p = to_params(a);
  const int grid = (p.world * p.cap + 7) / 8;
  if (dtype == 0)
    ep_combine_send_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(y), rows_of_src, p);
  else
    ep_combine_send_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), rows_of_src, p);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

MLCB_API int mlcb_ep_wait_flags(const int* flags, int n, int epoch, int* epoch_base, int* status,
                                cudaStream_t stream) {
  ep_wait_flags_kernel<<<1, 32, 0, stream>>>(flags, n, epoch, epoch_base, status);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
