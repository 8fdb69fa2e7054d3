// int4 unpack and dense dequantise: HBM-bound byte/word kernels.
//
// A packed word holds 8 adjacent columns; nibble j (bits 4j..4j+3) is column
// {0,2,4,6,1,3,5,7}[j] of the group, so column e sits at bit {0,16,4,20,8,24,12,28}[e].
#include "common.cuh"

namespace nqb200 {

// One thread per packed word: 4 B in, 8 B out (one 64-bit store); a warp reads
// 128 B and writes 256 B, both contiguous.
__global__ void __launch_bounds__(256) unpack_int4_kernel(const uint32_t* __restrict__ words,
                                                          uint2* __restrict__ out, int64_t nwords) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < nwords; i += stride) {
    const uint32_t w = __ldg(words + i);
    const uint32_t ev = w & 0x0F0F0F0Fu;         // bytes: e0, e4, e1, e5
    const uint32_t od = (w >> 4) & 0x0F0F0F0Fu;  // bytes: e2, e6, e3, e7
    // bytes 0-3 of `ev` are selector 0-3, bytes of `od` are 4-7
    uint2 o;
    o.x = __byte_perm(ev, od, 0x6420);  // e0 e1 e2 e3  <- ev.b0, ev.b2, od.b0, od.b2
    o.y = __byte_perm(ev, od, 0x7531);  // e4 e5 e6 e7  <- ev.b1, ev.b3, od.b1, od.b3
    out[i] = o;
  }
}

// One thread per packed word: reads the word, its zero-point word and 8
// scales (16 B), writes 8 dequantised values (16 B).  The integer difference
// times a 16-bit scale is exact in fp32, so the single conversion back gives
// the one rounding of `dtype(q - z) * s`.
template <bool BF16>
__global__ void __launch_bounds__(256) dequant_kernel(const uint32_t* __restrict__ qw,
                                                      const uint4* __restrict__ sc,
                                                      const uint32_t* __restrict__ qz,
                                                      uint4* __restrict__ out, int K, int NW, int g) {
  const int64_t total = (int64_t)K * NW;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int k = (int)(i / NW);
    const int c = (int)(i - (int64_t)k * NW);
    const int gi = k / g;
    const uint32_t w = __ldg(qw + i);
    const uint32_t z = __ldg(qz + (int64_t)gi * NW + c);
    const uint4 s4 = __ldg(sc + (int64_t)gi * NW + c);
    const uint32_t s[4] = {s4.x, s4.y, s4.z, s4.w};
    uint32_t o[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      // columns 2p and 2p+1 sit at bits 4p and 4p+16
      const int d0 = (int)((w >> (4 * p)) & 0xF) - (int)((z >> (4 * p)) & 0xF);
      const int d1 = (int)((w >> (4 * p + 16)) & 0xF) - (int)((z >> (4 * p + 16)) & 0xF);
      const float s0 = raw16_to_float<BF16>((uint16_t)(s[p] & 0xFFFF));
      const float s1 = raw16_to_float<BF16>((uint16_t)(s[p] >> 16));
      o[p] = (uint32_t)float_to_raw16<BF16>((float)d0 * s0) |
             ((uint32_t)float_to_raw16<BF16>((float)d1 * s1) << 16);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace nqb200

using namespace nqb200;

extern "C" int nqb200_unpack_int4(const void* words, void* out_u8, int64_t rows, int64_t cols_packed,
                                  void* stream) {
  if (rows < 0 || cols_packed < 0) return NQB200_ERR_BAD_SHAPE;
  if (rows == 0 || cols_packed == 0) return NQB200_OK;
  if (!words || !out_u8) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(words) || !aligned16(out_u8)) return NQB200_ERR_MISALIGNED;
  const int64_t n = rows * cols_packed;
  const int64_t blocks = (n + 255) / 256;
  const int grid = (int)(blocks < (int64_t)kNumSMs * 16 ? blocks : (int64_t)kNumSMs * 16);
  unpack_int4_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint32_t*)words, (uint2*)out_u8, n);
  return check_launch();
}

extern "C" int nqb200_dequant(const void* qweight, const void* qscales, const void* qzeros, void* out,
                              int64_t K, int64_t N, int64_t g, int dtype, void* stream) {
  if (K <= 0 || N <= 0 || g <= 0 || K % g != 0 || N % 8 != 0 || K > INT32_MAX || N > INT32_MAX)
    return NQB200_ERR_BAD_SHAPE;
  if (dtype != NQB200_F16 && dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  if (!qweight || !qscales || !qzeros || !out) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(qweight) || !aligned16(qscales) || !aligned16(qzeros) || !aligned16(out))
    return NQB200_ERR_MISALIGNED;
  const int NW = (int)(N / 8);
  const int64_t n = K * (int64_t)NW;
  const int64_t blocks = (n + 255) / 256;
  const int grid = (int)(blocks < (int64_t)kNumSMs * 16 ? blocks : (int64_t)kNumSMs * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == NQB200_BF16)
    dequant_kernel<true><<<grid, 256, 0, st>>>((const uint32_t*)qweight, (const uint4*)qscales,
                                               (const uint32_t*)qzeros, (uint4*)out, (int)K, NW, (int)g);
  else
    dequant_kernel<false><<<grid, 256, 0, st>>>((const uint32_t*)qweight, (const uint4*)qscales,
                                                (const uint32_t*)qzeros, (uint4*)out, (int)K, NW, (int)g);
  return check_launch();
}
