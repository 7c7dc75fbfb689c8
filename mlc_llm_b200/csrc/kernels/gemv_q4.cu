// Memory-bound matrix-vector product for int4-group weights (q4f16_1) and one to four tokens: the
// single-stream decode case, where the tensor-core kernel's dequantise-to-shared-memory stage, not
// HBM, sets the pace.  Reference behaviour: the fused dequantize + GEMV schedule that dlight gives
// ``fuse_dequantize_matmul_ewise`` outputs at batch 1 (python/mlc_llm/compiler_pass/
// fuse_dequantize_matmul_ewise.py:9-85, low_batch_specialization.py).
//
// One warp owns R = 4 consecutive output rows.  A lane takes one 32-weight group of each row per
// step: a 16-byte load of packed nibbles per row, one fp16 scale per row, and the 32 activations of
// that group for every token (64 bytes per token, shared by the four rows and, through L1, by the
// other warps).  Weights are expanded with the 0x6400 trick (1024 + q is exact in fp16), multiplied
// with the activations in half2 four products at a time, and accumulated in fp32.  No shared memory,
// no barriers.
//
// Weight layout: the device nibble order of the tensor-core kernel (word w of a row holds elements
// 8w .. 8w+7; pair (2j, 2j+1) at bits [4j, 4j+4) and [16+4j, 20+4j)).
#include "common.cuh"

namespace mlcb {

constexpr int GEMV_ROWS = 4;    // rows per warp
constexpr int GEMV_WARPS = 8;   // warps per CTA

// Eight weights of one packed word -> four half2 values (q - 7), in element order.  Pairs 0 and 2 sit in
// the low nibble of each half-word (of the word, and of the word shifted right by 8): 0x6400 | q is
// 1024 + q.  Pairs 1 and 3 sit one nibble higher: 0x6400 | (q << 4) is 1024 + 16 q, and one fused
// multiply-add (x 1/16, - 71) brings it to q - 7.  One shift, four logic ops and four arithmetic ops
// per word; every step is exact in fp16.
__device__ __forceinline__ void unpack8_q4(uint32_t wv, __half2 (&hv)[4]) {
  const __half2 off = __float2half2_rn(1031.f);
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  const __half2 off_hi = __float2half2_rn(-71.f);
  const uint32_t w8 = wv >> 8;
  uint32_t a = (wv & 0x000f000fu) | 0x64006400u;
  uint32_t b = (wv & 0x00f000f0u) | 0x64006400u;
  uint32_t c = (w8 & 0x000f000fu) | 0x64006400u;
  uint32_t d = (w8 & 0x00f000f0u) | 0x64006400u;
  hv[0] = __hsub2(*reinterpret_cast<__half2*>(&a), off);
  hv[1] = __hfma2(*reinterpret_cast<__half2*>(&b), sixteenth, off_hi);
  hv[2] = __hsub2(*reinterpret_cast<__half2*>(&c), off);
  hv[3] = __hfma2(*reinterpret_cast<__half2*>(&d), sixteenth, off_hi);
}

template <typename TO, int MMAX>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
    gemv_q4_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ w, const __half* __restrict__ scale,
                   const __half* __restrict__ bias, TO* __restrict__ y, int m_count, int N, int K, int ldx,
                   int ldy) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * GEMV_WARPS + warp) * GEMV_ROWS;
  if (row0 >= N) return;
  const int groups = K >> 5;            // 32-weight groups (= 16-byte chunks of nibbles) per row
  const size_t words_per_row = static_cast<size_t>(K) >> 3;
  float acc[GEMV_ROWS][MMAX];
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MMAX; ++m) acc[r][m] = 0.f;
  const __half2 off = __float2half2_rn(1031.f);
  for (int g = lane; g < groups; g += 32) {
    uint4 q[GEMV_ROWS];
    float s[GEMV_ROWS];
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) {
      const int row = row0 + r;
      if (row < N) {
        q[r] = __ldg(reinterpret_cast<const uint4*>(w + row * words_per_row) + g);
        s[r] = __half2float(__ldg(scale + static_cast<size_t>(row) * groups + g));
      } else {
        q[r] = make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);  // q - 7 == 0
        s[r] = 0.f;
      }
    }
    __half2 xv[MMAX][16];
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      if (m < m_count) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * ldx + (g << 5));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 t = __ldg(xp + i);
          xv[m][4 * i] = *reinterpret_cast<const __half2*>(&t.x);
          xv[m][4 * i + 1] = *reinterpret_cast<const __half2*>(&t.y);
          xv[m][4 * i + 2] = *reinterpret_cast<const __half2*>(&t.z);
          xv[m][4 * i + 3] = *reinterpret_cast<const __half2*>(&t.w);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) xv[m][i] = __float2half2_rn(0.f);
      }
    }
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) {
      const uint32_t words[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
#pragma unroll
      for (int wd = 0; wd < 4; wd += 2) {   // two words (16 weights) per trip to fp32
        __half2 ha[4], hb[4];
        unpack8_q4(words[wd], ha);
        unpack8_q4(words[wd + 1], hb);
#pragma unroll
        for (int m = 0; m < MMAX; ++m) {
          __half2 p = __hmul2(ha[0], xv[m][4 * wd]);
          p = __hfma2(ha[1], xv[m][4 * wd + 1], p);
          p = __hfma2(ha[2], xv[m][4 * wd + 2], p);
          p = __hfma2(ha[3], xv[m][4 * wd + 3], p);
          p = __hfma2(hb[0], xv[m][4 * wd + 4], p);
          p = __hfma2(hb[1], xv[m][4 * wd + 5], p);
          p = __hfma2(hb[2], xv[m][4 * wd + 6], p);
          p = __hfma2(hb[3], xv[m][4 * wd + 7], p);
          const float2 f = __half22float2(p);
          acc[r][m] += s[r] * (f.x + f.y);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      const int row = row0 + r;
      if (lane == 0 && row < N && m < m_count) {
        if (bias) v += __half2float(bias[row]);
        y[static_cast<size_t>(m) * ldy + row] = Cvt<TO>::from_f(v);
      }
    }
}

// Second form: KS warps of a CTA share each group of four rows and split K between them (narrow layers
// have too few rows to fill the GPU with one warp per row group), and the loads of the next step are
// issued before the arithmetic of the current one (PREFETCH; measured slower than relying on occupancy:
// 119 us vs 100 us on the 128256 x 4096 LM head, so the launcher does not select it).
template <typename TO, int MMAX, int KS, bool PREFETCH>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
    gemv_q4_split_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ w,
                         const __half* __restrict__ scale, const __half* __restrict__ bias, TO* __restrict__ y,
                         int m_count, int N, int K, int ldx, int ldy, const int* __restrict__ slab_of_row) {
  __shared__ float partial[GEMV_WARPS][GEMV_ROWS][MMAX];
  if (slab_of_row) {
    // grouped form (mixture-of-experts decode): blockIdx.y is a row of x / y, multiplied by the weight slab
    // (expert) named for it; w / scale hold the slabs one after the other, [slabs, N, K / 8] and [slabs, N, K / 32]
    const size_t slab = static_cast<size_t>(slab_of_row[blockIdx.y]);
    w += slab * N * (static_cast<size_t>(K) >> 3);
    scale += slab * N * (static_cast<size_t>(K) >> 5);
    x += static_cast<size_t>(blockIdx.y) * ldx;
    y += static_cast<size_t>(blockIdx.y) * ldy;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int GROUPS_PER_CTA = GEMV_WARPS / KS;     // row groups per CTA
  const int rg = warp / KS, ks = warp % KS;           // row group inside the CTA, K slice of this warp
  const int row0 = (blockIdx.x * GROUPS_PER_CTA + rg) * GEMV_ROWS;
  const int groups = K >> 5;
  const size_t words_per_row = static_cast<size_t>(K) >> 3;
  float acc[GEMV_ROWS][MMAX];
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MMAX; ++m) acc[r][m] = 0.f;
  const __half2 off = __float2half2_rn(1031.f);

  uint4 q[GEMV_ROWS], qn[GEMV_ROWS];
  float s[GEMV_ROWS], sn[GEMV_ROWS];
  uint4 xr[MMAX][4], xn[MMAX][4];
  auto load = [&](int g, uint4 (&qq)[GEMV_ROWS], float (&ss)[GEMV_ROWS], uint4 (&xx)[MMAX][4]) {
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) {
      const int row = row0 + r;
      if (row < N && g < groups) {
        qq[r] = __ldg(reinterpret_cast<const uint4*>(w + row * words_per_row) + g);
        ss[r] = __half2float(__ldg(scale + static_cast<size_t>(row) * groups + g));
      } else {
        qq[r] = make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
        ss[r] = 0.f;
      }
    }
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      if (m < m_count && g < groups) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * ldx + (g << 5));
#pragma unroll
        for (int i = 0; i < 4; ++i) xx[m][i] = __ldg(xp + i);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) xx[m][i] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  auto compute = [&](const uint4 (&qq)[GEMV_ROWS], const float (&ss)[GEMV_ROWS], const uint4 (&xx)[MMAX][4]) {
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) {
      const uint32_t words[4] = {qq[r].x, qq[r].y, qq[r].z, qq[r].w};
#pragma unroll
      for (int wd = 0; wd < 4; wd += 2) {
        __half2 ha[4], hb[4];
        unpack8_q4(words[wd], ha);
        unpack8_q4(words[wd + 1], hb);
#pragma unroll
        for (int m = 0; m < MMAX; ++m) {
          const uint32_t xa[4] = {xx[m][wd].x, xx[m][wd].y, xx[m][wd].z, xx[m][wd].w};
          const uint32_t xb[4] = {xx[m][wd + 1].x, xx[m][wd + 1].y, xx[m][wd + 1].z, xx[m][wd + 1].w};
          __half2 p = __hmul2(ha[0], *reinterpret_cast<const __half2*>(&xa[0]));
          p = __hfma2(ha[1], *reinterpret_cast<const __half2*>(&xa[1]), p);
          p = __hfma2(ha[2], *reinterpret_cast<const __half2*>(&xa[2]), p);
          p = __hfma2(ha[3], *reinterpret_cast<const __half2*>(&xa[3]), p);
          p = __hfma2(hb[0], *reinterpret_cast<const __half2*>(&xb[0]), p);
          p = __hfma2(hb[1], *reinterpret_cast<const __half2*>(&xb[1]), p);
          p = __hfma2(hb[2], *reinterpret_cast<const __half2*>(&xb[2]), p);
          p = __hfma2(hb[3], *reinterpret_cast<const __half2*>(&xb[3]), p);
          const float2 f = __half22float2(p);
          acc[r][m] += ss[r] * (f.x + f.y);
        }
      }
    }
  };
  const int step = 32 * KS;
  int g = ks * 32 + lane;
  if (row0 < N) {
    if (PREFETCH) {
      load(g, q, s, xr);
      while (g < groups) {
        load(g + step, qn, sn, xn);   // past the end: zero weights, no memory access
        compute(q, s, xr);
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r) { q[r] = qn[r]; s[r] = sn[r]; }
#pragma unroll
        for (int m = 0; m < MMAX; ++m)
#pragma unroll
          for (int i = 0; i < 4; ++i) xr[m][i] = xn[m][i];
        g += step;
      }
    } else {
      for (; g < groups; g += step) {
        load(g, q, s, xr);
        compute(q, s, xr);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) partial[warp][r][m] = v;
    }
  __syncthreads();
  // one thread per (row group, row, token) adds the K slices
  const int items = GROUPS_PER_CTA * GEMV_ROWS * MMAX;
  for (int i = threadIdx.x; i < items; i += blockDim.x) {
    const int g2 = i / (GEMV_ROWS * MMAX), r = (i / MMAX) % GEMV_ROWS, m = i % MMAX;
    const int row = (blockIdx.x * GROUPS_PER_CTA + g2) * GEMV_ROWS + r;
    if (row < N && m < m_count) {
      float v = 0.f;
#pragma unroll
      for (int k2 = 0; k2 < KS; ++k2) v += partial[g2 * KS + k2][r][m];
      if (bias) v += __half2float(bias[row]);
      y[static_cast<size_t>(m) * ldy + row] = Cvt<TO>::from_f(v);
    }
  }
}

}  // namespace mlcb

using namespace mlcb;

static int g_gemv_form = -1;  // -1 unread; 1 = one warp per row group; 2 = K split across warps + prefetch
static int gemv_form() {
  if (g_gemv_form < 0) {
    const char* e = getenv("MLCB_GEMV_FORM");
    g_gemv_form = (e && e[0] == '1') ? 1 : 2;
  }
  return g_gemv_form;
}
// Test / benchmark hook.
MLCB_API void mlcb_gemv_set_form(int form) { g_gemv_form = form; }

// x: [M, K] fp16 (row stride ldx, 16-byte aligned rows), w: packed int4 [N, K/8] in the device nibble
// order, scale: [N, K/32] fp16, y: [M, N] (row stride ldy) fp16 (out_dtype 0) or fp32 (out_dtype 2).
// Returns -1 for shapes it does not take (M > 4, K not a multiple of 32, misaligned rows); the caller
// then uses the tensor-core kernel.
MLCB_API int mlcb_gemv_q4(const void* x, const void* w, const void* scale, const void* bias, void* y, int M,
                          int N, int K, int ldx, int ldy, int out_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 4 || K <= 0 || K % 32 != 0 || ldx % 8 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -1;
  if (out_dtype != 0 && out_dtype != 2) return -1;
  if (gemv_form() == 2) {
    // K slices per row group: enough warps to cover the SMs several times over, at least one step each
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long row_groups = (N + GEMV_ROWS - 1) / GEMV_ROWS;
    int ks = 1;
    while (ks < GEMV_WARPS && row_groups * ks < static_cast<long long>(sms) * 32 && (K >> 5) >= 32 * ks * 2) ks *= 2;
    const int groups_per_cta = GEMV_WARPS / ks;
    const int grid2 = static_cast<int>((row_groups + groups_per_cta - 1) / groups_per_cta);
#define GEMV_SPLIT(TO, MM, KS, PF)                                                                          \
  gemv_q4_split_kernel<TO, MM, KS, PF><<<grid2, GEMV_WARPS * 32, 0, stream>>>(                               \
      static_cast<const __half*>(x), static_cast<const uint32_t*>(w), static_cast<const __half*>(scale),     \
      static_cast<const __half*>(bias), static_cast<TO*>(y), M, N, K, ldx, ldy, nullptr)
#define GEMV_SPLIT_KS(TO, MM, PF)                                     \
  do {                                                                \
    if (ks == 1) GEMV_SPLIT(TO, MM, 1, PF);                           \
    else if (ks == 2) GEMV_SPLIT(TO, MM, 2, PF);                      \
    else if (ks == 4) GEMV_SPLIT(TO, MM, 4, PF);                      \
    else GEMV_SPLIT(TO, MM, 8, PF);                                   \
  } while (0)
    if (out_dtype == 0) {
      if (M == 1) GEMV_SPLIT_KS(__half, 1, false);
      else if (M == 2) GEMV_SPLIT_KS(__half, 2, false);
      else GEMV_SPLIT_KS(__half, 4, false);
    } else {
      if (M == 1) GEMV_SPLIT_KS(float, 1, false);
      else if (M == 2) GEMV_SPLIT_KS(float, 2, false);
      else GEMV_SPLIT_KS(float, 4, false);
    }
#undef GEMV_SPLIT_KS
#undef GEMV_SPLIT
    count_launch();
    return static_cast<int>(cudaGetLastError());
  }
  const int rows_per_cta = GEMV_WARPS * GEMV_ROWS;
  const int grid = (N + rows_per_cta - 1) / rows_per_cta;
#define GEMV_LAUNCH(TO, MM)                                                                             \
  gemv_q4_kernel<TO, MM><<<grid, GEMV_WARPS * 32, 0, stream>>>(                                         \
      static_cast<const __half*>(x), static_cast<const uint32_t*>(w), static_cast<const __half*>(scale), \
      static_cast<const __half*>(bias), static_cast<TO*>(y), M, N, K, ldx, ldy)
  if (out_dtype == 0) {
    if (M == 1) GEMV_LAUNCH(__half, 1);
    else if (M == 2) GEMV_LAUNCH(__half, 2);
    else GEMV_LAUNCH(__half, 4);
  } else {
    if (M == 1) GEMV_LAUNCH(float, 1);
    else if (M == 2) GEMV_LAUNCH(float, 2);
    else GEMV_LAUNCH(float, 4);
  }
#undef GEMV_LAUNCH
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// Grouped matrix-vector products for mixture-of-experts decode (reference: the single-token expert GEMV of
// python/mlc_llm/op/moe_matmul.py:12-74): row r of x [rows, K] is multiplied by slab slab_of_row[r] of the stacked
// weights w [slabs, N, K / 8] / scale [slabs, N, K / 32]; y [rows, N]. One grid row per row of x, so a handful
// of (token, expert) pairs stream only the experts they use, at the GEMV's memory-bound rate.
MLCB_API int mlcb_gemv_q4_grouped(const void* x, const void* w, const void* scale, void* y, const int* slab_of_row,
                                  int rows, int N, int K, int ldx, int ldy, int out_dtype, cudaStream_t stream) {
  if (rows <= 0 || N <= 0) return 0;
  if (rows > 64 || K <= 0 || K % 32 != 0 || ldx % 8 != 0 || !slab_of_row) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -1;
  if (out_dtype != 0 && out_dtype != 2) return -1;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long row_groups = (N + GEMV_ROWS - 1) / GEMV_ROWS;
  int ks = 1;
  while (ks < GEMV_WARPS && row_groups * ks * rows < static_cast<long long>(sms) * 32 && (K >> 5) >= 32 * ks * 2) ks *= 2;
  const int groups_per_cta = GEMV_WARPS / ks;
  dim3 grid(static_cast<unsigned>((row_groups + groups_per_cta - 1) / groups_per_cta), static_cast<unsigned>(rows));
#define GEMV_GROUPED(TO, KS)                                                                                 \
  gemv_q4_split_kernel<TO, 1, KS, false><<<grid, GEMV_WARPS * 32, 0, stream>>>(                               \
      static_cast<const __half*>(x), static_cast<const uint32_t*>(w), static_cast<const __half*>(scale), nullptr, \
      static_cast<TO*>(y), 1, N, K, ldx, ldy, slab_of_row)
#define GEMV_GROUPED_KS(TO)               \
  do {                                    \
    if (ks == 1) GEMV_GROUPED(TO, 1);     \
    else if (ks == 2) GEMV_GROUPED(TO, 2); \
    else if (ks == 4) GEMV_GROUPED(TO, 4); \
    else GEMV_GROUPED(TO, 8);             \
  } while (0)
  if (out_dtype == 0) GEMV_GROUPED_KS(__half);
  else GEMV_GROUPED_KS(float);
#undef GEMV_GROUPED_KS
#undef GEMV_GROUPED
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------
// Five to sixteen tokens: warp-level tensor-core form.  The tcgen05 kernel expands weights through shared
// memory at a rate sized for 256-token tiles, so for a handful of tokens it takes as long as for 256; here the
// nibbles are expanded in registers straight into the A fragments of mma.sync.m16n8k16 (weights are A,
// 16 output rows x 16 k; activations are B, 16 k x 8 tokens; fp32 accumulators).
//
// Fragment layout (PTX ISA, m16n8k16, .f16): with g = lane / 4 and t = lane % 4,
//   A regs: {row g, k 2t..2t+1}, {row g+8, k 2t..2t+1}, {row g, k 2t+8..2t+9}, {row g+8, k 2t+8..2t+9}
//   B regs: {k 2t..2t+1, token g}, {k 2t+8..2t+9, token g}
//   C regs: {row g, tokens 2t, 2t+1}, {row g+8, tokens 2t, 2t+1}
// In the device nibble order a packed word holds eight consecutive k with the pair (2j, 2j+1) at bits
// [4j, 4j+4) and [16+4j, 20+4j), so the A register for k 2t..2t+1 of a 16-k block is pair j = t of the block's
// first word and the one for k 2t+8..2t+9 is pair t of its second word: one shift, one mask-or, one subtract.
// A lane reads the 16 bytes (32 k, one scale group) of its two rows per step; the four lanes of a row read
// the same bytes.  The group scale is applied to the group's partial accumulator in fp32.
namespace mlcb {

__device__ __forceinline__ uint32_t unpack_pair_q4(uint32_t word, int shift) {
  uint32_t v = ((word >> shift) & 0x000f000fu) | 0x64006400u;
  const __half2 off = __float2half2_rn(1031.f);
  __half2 h = __hsub2(*reinterpret_cast<__half2*>(&v), off);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int MMV_WARPS = 8;

// NT token tiles of eight (1: up to 8 tokens, 2: up to 16); KS warps share a 16-row group and split K.
template <typename TO, int NT, int KS>
__global__ void __launch_bounds__(MMV_WARPS * 32)
    gemm_q4_lowm_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ w, const __half* __restrict__ scale,
                        const __half* __restrict__ bias, TO* __restrict__ y, int m_count, int N, int K, int ldx,
                        int ldy) {
  __shared__ float partial[MMV_WARPS][16][NT * 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  constexpr int GROUPS_PER_CTA = MMV_WARPS / KS;
  const int rg = warp / KS, ks = warp % KS;
  const int row0 = (blockIdx.x * GROUPS_PER_CTA + rg) * 16;
  const int groups = K >> 5;                               // 32-k scale groups per row
  const size_t words_per_row = static_cast<size_t>(K) >> 3;
  const int ra = row0 + g, rb = row0 + g + 8;              // this lane's two rows
  const bool va = ra < N, vb = rb < N;
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
  const int shift = 4 * t;
  if (row0 < N) {
    for (int gi = ks; gi < groups; gi += KS) {
      const uint4 qa = va ? __ldg(reinterpret_cast<const uint4*>(w + ra * words_per_row) + gi)
                          : make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
      const uint4 qb = vb ? __ldg(reinterpret_cast<const uint4*>(w + rb * words_per_row) + gi)
                          : make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
      const float sa = va ? __half2float(__ldg(scale + static_cast<size_t>(ra) * groups + gi)) : 0.f;
      const float sb = vb ? __half2float(__ldg(scale + static_cast<size_t>(rb) * groups + gi)) : 0.f;
      // two 16-k blocks of this 32-k group: words (x, y) and (z, w)
      const uint32_t a_lo[4] = {unpack_pair_q4(qa.x, shift), unpack_pair_q4(qb.x, shift),
                                unpack_pair_q4(qa.y, shift), unpack_pair_q4(qb.y, shift)};
      const uint32_t a_hi[4] = {unpack_pair_q4(qa.z, shift), unpack_pair_q4(qb.z, shift),
                                unpack_pair_q4(qa.w, shift), unpack_pair_q4(qb.w, shift)};
      const int k0 = gi << 5;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int tok = n * 8 + g;
        uint32_t b[4] = {0u, 0u, 0u, 0u};
        if (tok < m_count) {
          const __half* xp = x + static_cast<size_t>(tok) * ldx + k0 + 2 * t;
          b[0] = __ldg(reinterpret_cast<const uint32_t*>(xp));        // k0 + 2t, +1
          b[1] = __ldg(reinterpret_cast<const uint32_t*>(xp + 8));    // k0 + 2t + 8, +9
          b[2] = __ldg(reinterpret_cast<const uint32_t*>(xp + 16));   // second block
          b[3] = __ldg(reinterpret_cast<const uint32_t*>(xp + 24));
        }
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        mma_m16n8k16(c, a_lo, b[0], b[1]);
        mma_m16n8k16(c, a_hi, b[2], b[3]);
        acc[n][0] += sa * c[0];
        acc[n][1] += sa * c[1];
        acc[n][2] += sb * c[2];
        acc[n][3] += sb * c[3];
      }
    }
  }
  // C layout: regs 0,1 = (row g, tokens 2t, 2t+1); regs 2,3 = (row g+8, same tokens)
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    partial[warp][g][n * 8 + 2 * t] = acc[n][0];
    partial[warp][g][n * 8 + 2 * t + 1] = acc[n][1];
    partial[warp][g + 8][n * 8 + 2 * t] = acc[n][2];
    partial[warp][g + 8][n * 8 + 2 * t + 1] = acc[n][3];
  }
  __syncthreads();
  const int items = GROUPS_PER_CTA * 16 * NT * 8;
  for (int i = threadIdx.x; i < items; i += blockDim.x) {
    const int tok = i % (NT * 8), r = (i / (NT * 8)) % 16, g2 = i / (NT * 8 * 16);
    const int row = (blockIdx.x * GROUPS_PER_CTA + g2) * 16 + r;
    if (row < N && tok < m_count) {
      float v = 0.f;
#pragma unroll
      for (int k2 = 0; k2 < KS; ++k2) v += partial[g2 * KS + k2][r][tok];
      if (bias) v += __half2float(bias[row]);
      y[static_cast<size_t>(tok) * ldy + row] = Cvt<TO>::from_f(v);
    }
  }
}

}  // namespace mlcb

// Same contract as mlcb_gemv_q4 for 1 <= M <= 16 (K a multiple of 32, rows of x 16-byte aligned).
MLCB_API int mlcb_gemm_q4_lowm(const void* x, const void* w, const void* scale, const void* bias, void* y, int M,
                               int N, int K, int ldx, int ldy, int out_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 != 0 || ldx % 8 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -1;
  if (out_dtype != 0 && out_dtype != 2) return -1;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long row_groups = (N + 15) / 16;
  int ks = 1;
  while (ks < MMV_WARPS && row_groups * ks < static_cast<long long>(sms) * 24 && (K >> 5) >= ks * 8) ks *= 2;
  const int groups_per_cta = MMV_WARPS / ks;
  const int grid = static_cast<int>((row_groups + groups_per_cta - 1) / groups_per_cta);
#define LOWM_LAUNCH(TO, NT, KS)                                                                            \
  mlcb::gemm_q4_lowm_kernel<TO, NT, KS><<<grid, mlcb::MMV_WARPS * 32, 0, stream>>>(                         \
      static_cast<const __half*>(x), static_cast<const uint32_t*>(w), static_cast<const __half*>(scale),    \
      static_cast<const __half*>(bias), static_cast<TO*>(y), M, N, K, ldx, ldy)
#define LOWM_KS(TO, NT)                                \
  do {                                                 \
    if (ks == 1) LOWM_LAUNCH(TO, NT, 1);               \
    else if (ks == 2) LOWM_LAUNCH(TO, NT, 2);          \
    else if (ks == 4) LOWM_LAUNCH(TO, NT, 4);          \
    else LOWM_LAUNCH(TO, NT, 8);                       \
  } while (0)
  if (out_dtype == 0) {
    if (M <= 8) LOWM_KS(__half, 1);
    else LOWM_KS(__half, 2);
  } else {
    if (M <= 8) LOWM_KS(float, 1);
    else LOWM_KS(float, 2);
  }
#undef LOWM_KS
#undef LOWM_LAUNCH
  mlcb::count_launch();
  return static_cast<int>(cudaGetLastError());
}
