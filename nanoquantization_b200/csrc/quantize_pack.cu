// Quantise and pack on the GPU: group-wise asymmetric int4 quantisation of an
// nn.Linear weight [N, K] and packing into the AWQ checkpoint layout, in one
// kernel.  It reproduces, rounding for rounding, what the reference does in two
// Python steps: pseudo_quantize (nanoquantization/utils/quantization.py:20-41:
// scale = clamp(max - min, 1e-5) / 15, zero = clamp(-round(min / scale), 0, 15),
// q = clamp(round(w / scale) + zero, 0, 15), w' = (q - zero) * scale, every
// operation rounded to the weight dtype) followed by WQLinear_GEMM.from_linear
// (nanoquantization/layers/gemm.py:478-548: round(w' / scale + zero), no clamp,
// eight columns per int32 in the order 0,2,4,6,1,3,5,7).
//
// One CTA takes 64 output columns x one group of k: warp w reduces min and max of
// rows 8w..8w+7 (each lane 4 consecutive k... for group size 128), the quantised
// values go through shared memory, and the packed words of one k are written
// as 32 contiguous bytes.
#include "common.cuh"

namespace nqb200 {

template <int DT> struct QT;  // 0 f16, 1 bf16, 2 f32
template <> struct QT<0> { using T = __half;
  static __device__ __forceinline__ float ld(const void* p, size_t i) { return __half2float(reinterpret_cast<const __half*>(p)[i]); }
  static __device__ __forceinline__ float rnd(float v) { return __half2float(__float2half_rn(v)); } };
template <> struct QT<1> { using T = __nv_bfloat16;
  static __device__ __forceinline__ float ld(const void* p, size_t i) { return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]); }
  static __device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); } };
template <> struct QT<2> { using T = float;
  static __device__ __forceinline__ float ld(const void* p, size_t i) { return reinterpret_cast<const float*>(p)[i]; }
  static __device__ __forceinline__ float rnd(float v) { return v; } };

constexpr int kQCols = 64;  // output columns (weight rows) per CTA

// WDT: dtype of the weight (arithmetic is rounded to it); ODT: dtype of the stored scales (0 f16, 1 bf16)
template <int WDT, int ODT>
__global__ void __launch_bounds__(256) quantize_pack_kernel(const void* __restrict__ weight, uint32_t* __restrict__ qweight,
                                                            uint16_t* __restrict__ qscales, uint32_t* __restrict__ qzeros,
                                                            int N, int K, int g) {
  extern __shared__ uint8_t qs[];  // [kQCols][g] quantised values, then [kQCols] zero-points
  uint8_t* zs = qs + (size_t)kQCols * g;
  using W = QT<WDT>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kQCols, grp = blockIdx.y;
  const int k0 = grp * g;
  for (int r = warp; r < kQCols; r += 8) {
    const int n = n0 + r;
    if (n >= N) break;
    const size_t base = (size_t)n * K + k0;
    float mx = -INFINITY, mn = INFINITY;
    for (int k = lane; k < g; k += 32) { const float v = W::ld(weight, base + k); mx = fmaxf(mx, v); mn = fminf(mn, v); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o)); mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o)); }
    // every step rounded to the weight dtype, as the elementwise tensor operations of the reference are
    float range = W::rnd(mx - mn);
    range = W::rnd(fmaxf(range, 1e-5f));
    const float scale = W::rnd(range / 15.f);
    float zero = W::rnd(-rintf(W::rnd(mn / scale)));
    zero = fminf(fmaxf(zero, 0.f), 15.f);
    for (int k = lane; k < g; k += 32) {
      const float v = W::ld(weight, base + k);
      float q = W::rnd(rintf(W::rnd(v / scale)) + zero);
      q = fminf(fmaxf(q, 0.f), 15.f);
      const float wdq = W::rnd(W::rnd(q - zero) * scale);              // the fake-quantised weight
      const float iw = rintf(W::rnd(W::rnd(wdq / scale) + zero));      // what the packer recomputes from it
      qs[(size_t)r * g + k] = (uint8_t)((int)iw & 0xF);
    }
    if (lane == 0) {
      zs[r] = (uint8_t)(int)zero;
      // scales.clone().to(output_dtype)
      qscales[(size_t)grp * N + n] = ODT ? __bfloat16_as_ushort(__float2bfloat16_rn(scale)) : __half_as_ushort(__float2half_rn(scale));
    }
  }
  __syncthreads();
  const int NW = N >> 3;
  constexpr int kWordsPerRow = kQCols / 8;
  for (int idx = threadIdx.x; idx < g * kWordsPerRow; idx += blockDim.x) {
    const int k = idx / kWordsPerRow, wi = idx % kWordsPerRow;
    const int wcol = (n0 >> 3) + wi;
    if (wcol >= NW) continue;
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = (j < 4) ? 2 * j : 2 * (j - 4) + 1;  // nibble j holds column e
      word |= (uint32_t)qs[(size_t)(8 * wi + e) * g + k] << (4 * j);
    }
    qweight[(size_t)(k0 + k) * NW + wcol] = word;
  }
  if (threadIdx.x < kWordsPerRow) {
    const int wi = threadIdx.x, wcol = (n0 >> 3) + wi;
    if (wcol < NW) {
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = (j < 4) ? 2 * j : 2 * (j - 4) + 1;
        word |= (uint32_t)zs[8 * wi + e] << (4 * j);
      }
      qzeros[(size_t)grp * NW + wcol] = word;
    }
  }
}

}  // namespace nqb200

using namespace nqb200;

extern "C" int nqb200_quantize_pack(const void* weight, int weight_dtype, void* qweight, void* qscales, void* qzeros,
                                    int64_t N, int64_t K, int64_t g, int scales_dtype, void* stream) {
  if (N <= 0 || K <= 0 || g <= 0 || K % g != 0 || N % 8 != 0 || N > INT32_MAX || K > INT32_MAX) return NQB200_ERR_BAD_SHAPE;
  if (weight_dtype < 0 || weight_dtype > 2 || (scales_dtype != NQB200_F16 && scales_dtype != NQB200_BF16)) return NQB200_ERR_BAD_DTYPE;
  if (!weight || !qweight || !qscales || !qzeros) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(weight) || !aligned16(qweight) || !aligned16(qscales) || !aligned16(qzeros)) return NQB200_ERR_MISALIGNED;
  const size_t smem = (size_t)kQCols * g + kQCols;
  if (smem > 200 * 1024 || K / g > 65535) return NQB200_ERR_TOO_LARGE;
  dim3 grid((unsigned)((N + kQCols - 1) / kQCols), (unsigned)(K / g));
  cudaStream_t st = (cudaStream_t)stream;
#define NQ_LAUNCH(W, O)                                                                                              \
  do {                                                                                                               \
    if (smem > 48 * 1024 &&                                                                                          \
        cudaFuncSetAttribute(quantize_pack_kernel<W, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { \
      cudaGetLastError();                                                                                            \
      return NQB200_ERR_LAUNCH;                                                                                      \
    }                                                                                                                \
    quantize_pack_kernel<W, O><<<grid, 256, smem, st>>>(weight, (uint32_t*)qweight, (uint16_t*)qscales, (uint32_t*)qzeros, \
                                                       (int)N, (int)K, (int)g);                                     \
  } while (0)
  if (weight_dtype == 0) { if (scales_dtype) NQ_LAUNCH(0, 1); else NQ_LAUNCH(0, 0); }
  else if (weight_dtype == 1) { if (scales_dtype) NQ_LAUNCH(1, 1); else NQ_LAUNCH(1, 0); }
  else { if (scales_dtype) NQ_LAUNCH(2, 1); else NQ_LAUNCH(2, 0); }
#undef NQ_LAUNCH
  return check_launch();
}
