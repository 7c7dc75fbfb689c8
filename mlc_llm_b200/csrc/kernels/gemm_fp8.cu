// Block-scaled fp8 linear layers with fp8 activations (W8A8) on the 5th-gen tensor cores.
//
//   Y[M, N] = sum over K groups g of 128:  sa[m, g] * sw[n / 128, g] * (Xq[m, g] . Wq[n, g]^T)
//
// Wq: e4m3 [N, K] with one fp32 scale per 128 x 128 block (the "weight_scale_inv" tensor of block-scaled
// checkpoints). Xq: e4m3 [M, K] with one fp32 scale per row and 128-element group, produced on the fly by
// act_quant_fp8_kernel below (scale = max(|x|, eps) / 448, stored transposed [K / 128][M] so that the
// scales of a token tile and one group are contiguous).
//
// Both operands reach the tensor core as fp8 (tcgen05.mma kind::f8f6f4, twice the 16-bit rate), 128
// bytes of K per pipeline stage = exactly one scale group. The scale of a group's partial product varies
// with the token and the group, so it cannot stay inside one TMEM accumulator: every group is
// multiplied into a fresh accumulator (two of them take turns) and eight "promotion" warps add it,
// scaled, to fp32 registers while the tensor core works on the next group (the weight tile is the UMMA
// A operand, so a thread owns one output feature and 64 of the tile's up to 128 tokens). Measured: a
// 256-token tile with sixteen promotion warps is slower (0.75 vs 0.96 PFLOP/s at 8192 x 10240 x 8192), the
// promotion arithmetic then outweighs what the wider tensor-core instruction saves.
//
// Roles (320 threads): warp 0 = TMA producer (fp8 weights, fp8 activations, activation scales), warp 1 =
// MMA issuer (+ TMEM owner), warps 2-9 = promotion / epilogue.
//
// Reference counterparts: quantization/block_scale_quantization.py:285-318 (weights), :603-700
// (rowwise_group_quant_fp8), op/cutlass.py:138-279 (fp8 block-scale GEMM).
#include "common.cuh"

namespace mlcb {

constexpr int F8_BM = 128;        // weight rows per tile == UMMA M
constexpr int F8_BK = 128;        // fp8 elements per stage == one scale group == 128 bytes
constexpr int F8_TN = 128;        // tokens per tile (UMMA N), at most
constexpr int F8_STAGES = 6;
constexpr int F8_PROMO = 8;       // promotion warps: two per TMEM lane quarter, 64 token columns each
constexpr int F8_W_BYTES = F8_BM * F8_BK;   // 16 KiB
constexpr int F8_X_BYTES = F8_TN * F8_BK;   // 16 KiB
constexpr int F8_S_BYTES = F8_TN * 4;       // activation scales of the stage's group
constexpr int F8_STAGE_BYTES = F8_W_BYTES + F8_X_BYTES;
constexpr int F8_THREADS = 64 + 32 * F8_PROMO;
constexpr int F8_SMEM = F8_STAGES * (F8_STAGE_BYTES + F8_S_BYTES) + 1024 + 256;

struct Fp8Params {
  const float* w_scale;   // [ceil(N / 128), ceil(K / 128)]
  const float* x_scale;   // [K / 128][x_scale_ld] (transposed)
  const void* bias;       // [N] in the output dtype, may be null
  void* y;
  int* status;
  int M, N, K, ldy, x_scale_ld;
  int tn, num_m_blocks, num_n_blocks;
  int out_dtype;          // 0 fp16, 1 bf16
};

// 32 lanes x 16 columns of 32-bit values: thread t of the warp gets lane (base_lane + t).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sw = smem;                                   // STAGES x 16 KiB
  uint8_t* sx = sw + F8_STAGES * F8_W_BYTES;            // STAGES x 16 KiB
  float* ss = reinterpret_cast<float*>(sx + F8_STAGES * F8_X_BYTES);  // STAGES x TN scales
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(ss) + F8_STAGES * F8_S_BYTES);
  uint64_t* empty = full + F8_STAGES;      // MMA done with the tiles and the promotion warps with the scales
  uint64_t* acc_full = empty + F8_STAGES;  // [2] one group's product is complete
  uint64_t* acc_empty = acc_full + 2;      // [2] the promotion warps have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = (p.K + F8_BK - 1) / F8_BK;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;

  if (threadIdx.x < F8_STAGES) {
    mbar_init(&full[threadIdx.x], 1);
    mbar_init(&empty[threadIdx.x], 1 + F8_PROMO);
  }
  if (threadIdx.x < 2) {
    mbar_init(&acc_full[threadIdx.x], 1);
    mbar_init(&acc_empty[threadIdx.x], F8_PROMO);
  }
  if (threadIdx.x == 0) *abort_flag = 0;
  if (threadIdx.x < 32) mbar_fence_init();
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_x);
      tma_prefetch_desc(&tmap_w);
      const uint32_t bytes = F8_W_BYTES + static_cast<uint32_t>(p.tn) * F8_BK + static_cast<uint32_t>(p.tn) * 4;
      int s = 0;
      uint32_t eph = 1;
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int mb = t / p.num_n_blocks, nb = t - mb * p.num_n_blocks;
        for (int g = 0; g < groups; ++g, ++it) {
          if (it >= F8_STAGES && !mbar_wait(&empty[s], eph, abort_flag, p.status, ERR_WAIT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], bytes);
          tma_load_2d(sw + s * F8_W_BYTES, &tmap_w, &full[s], g * F8_BK, nb * F8_BM);
          tma_load_2d(sx + s * F8_X_BYTES, &tmap_x, &full[s], g * F8_BK, mb * p.tn);
          bulk_load(ss + s * F8_TN, p.x_scale + static_cast<size_t>(g) * p.x_scale_ld + mb * p.tn,
                    static_cast<uint32_t>(p.tn) * 4, &full[s]);
          if (++s == F8_STAGES) {
            s = 0;
            eph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer: one fresh accumulator per group
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(0, F8_BM, p.tn, 0, 0);  // e4m3 x e4m3, fp32 accumulate
      int s = 0;
      uint32_t ph = 0, ga = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int g = 0; g < groups; ++g, ++ga) {
          const int a = ga & 1;
          if (ga >= 2) {
            ok = mbar_wait(&acc_empty[a], ((ga >> 1) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EPILOGUE);
            if (!ok) break;
          }
          ok = mbar_wait(&full[s], ph, abort_flag, p.status, ERR_WAIT_TMA);
          if (!ok) break;
          tc_fence_after();
          const uint64_t adesc = umma_smem_desc(smem_u32(sw + s * F8_W_BYTES), 16, 1024);
          const uint64_t bdesc = umma_smem_desc(smem_u32(sx + s * F8_X_BYTES), 16, 1024);
          const uint32_t d_tmem = tmem_base + a * F8_TN;
#pragma unroll
          for (int kk = 0; kk < F8_BK / 32; ++kk)  // 32 fp8 elements (32 bytes) per instruction
            umma_f8(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, kk ? 1u : 0u);
          umma_commit(&empty[s]);
          umma_commit(&acc_full[a]);
          if (++s == F8_STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ promotion + epilogue
    const int q = warp & 3;             // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;   // which 64 of the tile's (up to) 128 tokens
    const int row = q * 32 + lane;      // output feature inside the tile
    int s = 0;
    uint32_t ga = 0;
    bool ok = true;
    __shared__ __align__(16) float comb_all[F8_PROMO][64];
    float* comb = comb_all[warp - 2];
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int mb = t / p.num_n_blocks, nb = t - mb * p.num_n_blocks;
      const int m0 = mb * p.tn, n = nb * F8_BM + row;
      const int c0 = half * 64;
      const bool cols_live = c0 < p.tn;  // narrow tiles: the warps of the higher column ranges have nothing to do
      float acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0.f;
      const float* wrow = p.w_scale + static_cast<size_t>(nb) * groups;
      for (int g = 0; g < groups; ++g, ++ga) {
        const int a = ga & 1;
        const float swg = __ldg(wrow + g);
        ok = mbar_wait(&acc_full[a], (ga >> 1) & 1, abort_flag, p.status, ERR_WAIT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // token scale x weight-block scale of this warp's 64 columns, formed once per column (two per lane)
        // instead of once per lane and column
        {
          const float2 sa2 = *reinterpret_cast<const float2*>(ss + s * F8_TN + c0 + 2 * lane);
          *reinterpret_cast<float2*>(comb + 2 * lane) = make_float2(sa2.x * swg, sa2.y * swg);
          __syncwarp();
        }
        if (cols_live) {
#pragma unroll
          for (int c = 0; c < 64; c += 16) {
            if (c0 + c >= p.tn) continue;
            uint32_t r[16];
            tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * F8_TN + c0 + c, r);
            tmem_ld_wait();
            const float4* sv = reinterpret_cast<const float4*>(comb + c);
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const float4 sa = sv[j4];  // the same address for every lane: a broadcast
              acc[c + 4 * j4 + 0] = fmaf(__uint_as_float(r[4 * j4 + 0]), sa.x, acc[c + 4 * j4 + 0]);
              acc[c + 4 * j4 + 1] = fmaf(__uint_as_float(r[4 * j4 + 1]), sa.y, acc[c + 4 * j4 + 1]);
              acc[c + 4 * j4 + 2] = fmaf(__uint_as_float(r[4 * j4 + 2]), sa.z, acc[c + 4 * j4 + 2]);
              acc[c + 4 * j4 + 3] = fmaf(__uint_as_float(r[4 * j4 + 3]), sa.w, acc[c + 4 * j4 + 3]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();  // (also: every lane is done with `comb` before the next group rewrites it)
        if (lane == 0) {
          mbar_arrive(&acc_empty[a]);
          mbar_arrive(&empty[s]);  // the stage's scales have been read
        }
        if (++s == F8_STAGES) s = 0;
      }
      if (!ok) break;
      // ---- epilogue: lane = output feature, a warp-wide store covers 32 consecutive features of a token
      if (cols_live && n < p.N) {
        float bias = 0.f;
        if (p.bias)
          bias = p.out_dtype == 0 ? __half2float(reinterpret_cast<const __half*>(p.bias)[n])
                                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]);
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int m = m0 + c0 + j;
          if (c0 + j >= p.tn || m >= p.M) continue;
          const size_t idx = static_cast<size_t>(m) * p.ldy + n;
          if (p.out_dtype == 0) reinterpret_cast<__half*>(p.y)[idx] = __float2half_rn(acc[j] + bias);
          else reinterpret_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(acc[j] + bias);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// Per row and 128-element group: scale = max(|x|, eps) / 448, q = clamp(x / scale, +-448) as e4m3.
// One warp per (row, group); a lane converts 4 consecutive elements. Scales are stored transposed,
// [K / 128][scale_ld], so the GEMM fetches the scales of a token tile and a group as one contiguous run.
template <typename T>
__global__ void act_quant_fp8_kernel(const T* __restrict__ x, uint8_t* __restrict__ xq, float* __restrict__ scale_t,
                                     int M, int K, long long ldx, int scale_ld) {
  const int groups = (K + 127) / 128;
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(M) * groups) return;
  const int m = static_cast<int>(w / groups), g = static_cast<int>(w - static_cast<long long>(m) * groups);
  const int k0 = g * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (k0 + 3 < K) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + m * ldx + k0);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = Cvt<T>::to_f(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (k0 + i < K) v[i] = Cvt<T>::to_f(x[m * ldx + k0 + i]);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = fmaxf(warp_max(amax), 1e-10f);
  const float scale = __fdiv_rn(amax, 448.f);
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float qv = fminf(fmaxf(__fdiv_rn(v[i], scale), -448.f), 448.f);  // the quotient, as the reference forms it
    packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  }
  if (k0 + 3 < K) {
    *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(m) * K + k0) = packed;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (k0 + i < K) xq[static_cast<size_t>(m) * K + k0 + i] = static_cast<uint8_t>(packed >> (8 * i));
  }
  if (lane == 0) scale_t[static_cast<size_t>(g) * scale_ld + m] = scale;
}

}  // namespace mlcb

using namespace mlcb;

// x: [M, K] fp16 (dtype 0) / bf16 (1), row stride ldx elements (a multiple of 4). xq: [M, K] e4m3.
// scale_t: [ceil(K / 128)][scale_ld] fp32 with scale_ld >= M.
MLCB_API int mlcb_act_quant_fp8(const void* x, void* xq, float* scale_t, int M, int K, long long ldx, int scale_ld,
                                int dtype, cudaStream_t stream) {
  if (M <= 0 || K <= 0) return 0;
  if (ldx % 4 || K % 4 || scale_ld < M || (reinterpret_cast<uintptr_t>(x) & 7) || (reinterpret_cast<uintptr_t>(xq) & 3))
    return -1;
  const long long warps = static_cast<long long>(M) * ((K + 127) / 128);
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
  if (dtype == 0)
    act_quant_fp8_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<const __half*>(x), static_cast<uint8_t*>(xq),
                                                             scale_t, M, K, ldx, scale_ld);
  else
    act_quant_fp8_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                    static_cast<uint8_t*>(xq), scale_t, M, K, ldx,
                                                                    scale_ld);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// xq: [M, K] e4m3 with x_scale_t [K / 128][x_scale_ld] (from mlcb_act_quant_fp8; x_scale_ld a multiple of 4 and
// >= M rounded up to the token tile). w: [N, K] e4m3 with w_scale [ceil(N / 128), ceil(K / 128)]. K must be a
// multiple of 128 (one scale group per pipeline stage). y: [M, N] fp16 / bf16.
MLCB_API int mlcb_gemm_fp8_w8a8(const void* xq, const float* x_scale_t, const void* w, const float* w_scale,
                                const void* bias, void* y, int M, int N, int K, int ldy, int x_scale_ld,
                                int out_dtype, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 != 0 || out_dtype > 1 || !x_scale_t || !w_scale) return -2;
  if ((reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x_scale_t)) & 15)
    return -3;
  static bool attr_set[64] = {};
  if (first_use_on_device(attr_set))
    cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM);
  Fp8Params p = {};
  p.w_scale = w_scale;
  p.x_scale = x_scale_t;
  p.bias = bias;
  p.y = y;
  p.status = status;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.x_scale_ld = x_scale_ld;
  // token tile: as even a split of M as fits 128, in multiples of 16
  const int blocks = (M + F8_TN - 1) / F8_TN;
  int tn = ((M + blocks - 1) / blocks + 15) / 16 * 16;
  if (tn > F8_TN) tn = F8_TN;
  p.tn = tn;
  p.num_m_blocks = (M + tn - 1) / tn;
  p.num_n_blocks = (N + F8_BM - 1) / F8_BM;
  p.out_dtype = out_dtype;
  if (x_scale_ld % 4 || x_scale_ld < p.num_m_blocks * tn) return -5;  // the last token tile reads a whole run of scales
  uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  uint64_t xs[1] = {static_cast<uint64_t>(K)};
  uint32_t xb[2] = {F8_BK, static_cast<uint32_t>(tn)};
  const CUtensorMap* mx = get_tensor_map(xq, 1, 2, xd, xs, xb, 1);
  uint64_t wd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
  uint64_t ws[1] = {static_cast<uint64_t>(K)};
  uint32_t wb[2] = {F8_BK, F8_BM};
  const CUtensorMap* mw = get_tensor_map(w, 1, 2, wd, ws, wb, 1);
  if (!mx || !mw) return -4;
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_fp8_kernel<<<grid, F8_THREADS, F8_SMEM, stream>>>(*mx, *mw, p);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
