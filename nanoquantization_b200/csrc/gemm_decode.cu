// Decode-side W4A16 kernel: skinny GEMM (up to 16 tokens per CTA) that streams
// the packed weights once and is bound by HBM bandwidth.
//
// The B200 has few issue slots per weight byte (about 2.8 lane-instructions per
// int4 weight at full bandwidth), so the weights are never expanded into
// dequantised fp16 values with a subtract and a multiply each.  Instead:
//
//   y[m,n] = sum_g s[g,n] * ( sum_{k in g} x[m,k] q[k,n]  -  z[g,n] * sum_{k in g} x[m,k] )
//
//   * the inner sums run on the tensor cores (mma.sync m16n8k16, weights as the
//     16-row A operand, tokens as the 8-column B operand, fp32 accumulate);
//   * q is fed as raw nibbles: for fp16, (word & 0x000F000F) read as half2 is
//     q * 2^-24 (a subnormal) and (word & 0x00F000F0) is q * 2^-20, both exact,
//     so one AND per pair of weights is the whole int4 -> fp16 conversion; for
//     bf16 the nibble is OR-ed into 128.0 and the offset is removed with the
//     same sum of x that removes the zero-point;
//   * sum_{k in g} x[m,k] comes from one extra mma per k-step with an all-ones
//     A operand, which lands it in exactly the accumulator layout that needs it;
//   * the scale, the power of two and the zero-point are applied once per
//     group per output in fp32.
//
// The mma wants two adjacent k of one column in a register while a packed word
// holds eight columns of one k.  One PRMT per pair of rows interleaves byte b of
// rows k and k+1, after which the two masks give k-paired operands directly.
// The k index inside a 16-row step is permuted (thread tig owns rows 4*tig..4*tig+3)
// consistently for both operands, so every thread reads whole packed words with
// 128-bit (or 64-bit) loads and x with one 64-bit load.
//
// Split-K: the 4 warps of a CTA take alternate groups and are summed in shared
// memory in a fixed order; CTAs along K write fp32 partials to the workspace
// and the last one to arrive (a counter per output tile) sums them in a fixed
// order, adds the bias and writes the result, so the output is deterministic.
#include "common.cuh"

namespace nqb200 {

constexpr int kDecodeThreads = 128;
constexpr int kDecodeWarps = 4;
constexpr int kTargetCtas = kNumSMs * 3;

bool decode_mma_supports(int64_t M, int64_t N, int64_t K, int64_t g) {
  (void)M;
  return N % 16 == 0 && g % 16 == 0 && K % g == 0;
}

DecodePlan plan_decode(int64_t M, int64_t N, int64_t K, int64_t g) {
  DecodePlan p;
  p.mt = M > 8 ? 2 : 1;
  p.ng = (p.mt == 1 && N % 32 == 0) ? 4 : 2;
  p.tile_n = 64 * p.ng;
  p.ntiles = (int)((N + p.tile_n - 1) / p.tile_n);
  p.mchunks = (int)((M + 8 * p.mt - 1) / (8 * p.mt));
  const int G = (int)(K / g);
  const int64_t base = (int64_t)p.ntiles * p.mchunks;
  int want = (int)((kTargetCtas + base - 1) / base);
  if (want < 1) want = 1;
  if (want > G) want = G;
  p.gpc = (G + want - 1) / want;
  p.ksplit = (G + p.gpc - 1) / p.gpc;
  // the counters always occupy the same fixed head of the workspace, so that one call's
  // partial sums can never be read as another call's counters
  p.counter_bytes = kCounterBytes;
  if (base * 4 > (int64_t)kCounterBytes) { p.gpc = G; p.ksplit = 1; }
  p.partial_bytes = p.ksplit > 1 ? (size_t)p.mchunks * p.ksplit * 8 * p.mt * (size_t)N * 4 : 0;
  return p;
}

struct DecodeParams {
  const uint16_t* x; const uint32_t* qw; const uint16_t* sc; const uint32_t* qz;
  const void* bias; int bias_dtype; uint16_t* out;
  int M, N, K, g, gpc, ksplit, ntiles;
  int* counters; float* partials;
};

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

template <int NG> struct WordVec;
template <> struct WordVec<4> {
  uint32_t v[4];
  __device__ __forceinline__ void load(const uint32_t* p) {
    const uint4 t = __ldg(reinterpret_cast<const uint4*>(p)); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ __forceinline__ void zero() { v[0] = v[1] = v[2] = v[3] = 0; }
};
template <> struct WordVec<2> {
  uint32_t v[2];
  __device__ __forceinline__ void load(const uint32_t* p) {
    const uint2 t = __ldg(reinterpret_cast<const uint2*>(p)); v[0] = t.x; v[1] = t.y;
  }
  __device__ __forceinline__ void zero() { v[0] = v[1] = 0; }
};

template <int MT, int NG, bool BF16>
__global__ void __launch_bounds__(kDecodeThreads) decode_mma_kernel(const DecodeParams p) {
  constexpr int TILE_N = 64 * NG;
  constexpr int ROWS = 8 * MT;
  constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u;
  constexpr uint32_t ONES = BF16 ? 0x3F803F80u : 0x3C003C00u;
  // value fed to the mma for nibble q is (q + OFF) / MULT
  constexpr float MULT_LO = BF16 ? 1.f : 16777216.f;  // 2^24
  constexpr float MULT_HI = BF16 ? 1.f : 1048576.f;   // 2^20
  constexpr float OFF = BF16 ? 128.f : 0.f;

  __shared__ float red[ROWS][TILE_N + 8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tig = lane & 3;
  const int tile_n0 = blockIdx.x * TILE_N;
  const int n0 = tile_n0 + gq * 8 * NG;
  const bool n_ok = n0 < p.N;
  const int NW = p.N >> 3;
  const int wc0 = n0 >> 3;
  const int mbase = blockIdx.z * ROWS;
  const int G = p.K / p.g;
  const int g_begin = blockIdx.y * p.gpc;
  const int g_end = min(G, g_begin + p.gpc);
  const int ksteps = p.g >> 4;

  const uint16_t* xrow[MT];
  bool m_ok[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int m = mbase + 8 * mt + gq;
    m_ok[mt] = m < p.M;
    xrow[mt] = p.x + (size_t)(m_ok[mt] ? m : 0) * p.K;
  }

  float total[MT][NG][4][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int c = 0; c < NG; ++c)
#pragma unroll
      for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[mt][c][b][i] = 0.f;

  for (int grp = g_begin + warp; grp < g_end; grp += kDecodeWarps) {
    float acc[MT][NG][4][4];
    float xs[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) xs[mt][i] = 0.f;
#pragma unroll
      for (int c = 0; c < NG; ++c)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[mt][c][b][i] = 0.f;
    }

    uint4 sv[NG];
    WordVec<NG> zw;
    if (n_ok) {
#pragma unroll
      for (int c = 0; c < NG; ++c)
        sv[c] = __ldg(reinterpret_cast<const uint4*>(p.sc + (size_t)grp * p.N + n0 + 8 * c));
      zw.load(p.qz + (size_t)grp * NW + wc0);
    } else {
#pragma unroll
      for (int c = 0; c < NG; ++c) sv[c] = make_uint4(0, 0, 0, 0);
      zw.zero();
    }

    const int kb0 = grp * p.g + 4 * tig;
    WordVec<NG> wa[4], wb[4];
    uint2 xa[MT], xb[MT];

    auto load_step = [&](WordVec<NG> (&w)[4], uint2 (&xf)[MT], int ks) {
      const int kb = kb0 + 16 * ks;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (n_ok) w[i].load(p.qw + (size_t)(kb + i) * NW + wc0); else w[i].zero();
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
        xf[mt] = m_ok[mt] ? __ldg(reinterpret_cast<const uint2*>(xrow[mt] + kb)) : make_uint2(0, 0);
    };

    auto compute_step = [&](const WordVec<NG> (&w)[4], const uint2 (&xf)[MT]) {
#pragma unroll
      for (int c = 0; c < NG; ++c) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          // byte b of rows k0,k1 (resp. k2,k3) into bytes 0 and 2: nibbles 2b and 2b+1, k-paired
          const uint32_t sel = (uint32_t)b | ((uint32_t)b << 4) | ((uint32_t)(4 + b) << 8) | ((uint32_t)(4 + b) << 12);
          const uint32_t p01 = __byte_perm(w[0].v[c], w[1].v[c], sel);
          const uint32_t p23 = __byte_perm(w[2].v[c], w[3].v[c], sel);
          uint32_t a0, a1, a2, a3;
          if (BF16) {
            a0 = (p01 & LO) | 0x43004300u; a1 = ((p01 >> 4) & LO) | 0x43004300u;
            a2 = (p23 & LO) | 0x43004300u; a3 = ((p23 >> 4) & LO) | 0x43004300u;
          } else {
            a0 = p01 & LO; a1 = p01 & HI; a2 = p23 & LO; a3 = p23 & HI;
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma16816<BF16>(acc[mt][c][b], a0, a1, a2, a3, xf[mt].x, xf[mt].y);
        }
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) mma16816<BF16>(xs[mt], ONES, ONES, ONES, ONES, xf[mt].x, xf[mt].y);
    };

    load_step(wa, xa, 0);
    for (int ks = 0; ks < ksteps; ks += 2) {
      const bool has1 = ks + 1 < ksteps;
      if (has1) load_step(wb, xb, ks + 1);
      compute_step(wa, xa);
      if (has1) {
        if (ks + 2 < ksteps) load_step(wa, xa, ks + 2);
        compute_step(wb, xb);
      }
    }

    // once per group: scale, power of two and zero-point, in fp32
#pragma unroll
    for (int c = 0; c < NG; ++c) {
      const uint32_t sw[4] = {sv[c].x, sv[c].y, sv[c].z, sv[c].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int b = j >> 1, r = j & 1;
        const int e = (j < 4) ? 2 * j : 2 * (j - 4) + 1;  // column held by nibble j
        const float s = raw16_to_float<BF16>((uint16_t)((sw[e >> 1] >> (16 * (e & 1))) & 0xFFFF));
        const float z = (float)((zw.v[c] >> (4 * j)) & 0xF);
        const float A = s * (r ? MULT_HI : MULT_LO);
        const float B = s * (z + OFF);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int t = 0; t < 2; ++t)
            total[mt][c][b][2 * r + t] += A * acc[mt][c][b][2 * r + t] - B * xs[mt][t];
      }
    }
  }

  // warps summed in order 0,1,2,3
#pragma unroll 1
  for (int w = 0; w < kDecodeWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < NG; ++c)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int b = j >> 1, r = j & 1;
            const int e = (j < 4) ? 2 * j : 2 * (j - 4) + 1;
            const int col = gq * 8 * NG + 8 * c + e;
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int row = 8 * mt + 2 * tig + t;
              const float v = total[mt][c][b][2 * r + t];
              if (w == 0) red[row][col] = v; else red[row][col] += v;
            }
          }
    }
    __syncthreads();
  }

  const int rows = min(ROWS, p.M - mbase);
  constexpr int HALF_N = TILE_N / 2;
  if (p.ksplit == 1) {
    for (int idx = threadIdx.x; idx < ROWS * HALF_N; idx += kDecodeThreads) {
      const int row = idx / HALF_N, n = tile_n0 + 2 * (idx % HALF_N);
      if (row < rows && n < p.N) {
        float v0 = red[row][n - tile_n0], v1 = red[row][n - tile_n0 + 1];
        if (p.bias) { v0 += bias_to_float(p.bias, p.bias_dtype, n); v1 += bias_to_float(p.bias, p.bias_dtype, n + 1); }
        const uint32_t o = (uint32_t)float_to_raw16<BF16>(v0) | ((uint32_t)float_to_raw16<BF16>(v1) << 16);
        *reinterpret_cast<uint32_t*>(p.out + (size_t)(mbase + row) * p.N + n) = o;
      }
    }
    return;
  }

  float* part = p.partials + ((size_t)blockIdx.z * p.ksplit) * ROWS * (size_t)p.N;
  for (int idx = threadIdx.x; idx < ROWS * HALF_N; idx += kDecodeThreads) {
    const int row = idx / HALF_N, n = tile_n0 + 2 * (idx % HALF_N);
    if (row < rows && n < p.N)
      __stcg(reinterpret_cast<float2*>(part + ((size_t)blockIdx.y * ROWS + row) * p.N + n),
             make_float2(red[row][n - tile_n0], red[row][n - tile_n0 + 1]));
  }
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  int* counter = p.counters + blockIdx.z * p.ntiles + blockIdx.x;
  if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1) == p.ksplit - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < ROWS * HALF_N; idx += kDecodeThreads) {
    const int row = idx / HALF_N, n = tile_n0 + 2 * (idx % HALF_N);
    if (row < rows && n < p.N) {
      float v0 = 0.f, v1 = 0.f;
      for (int ks = 0; ks < p.ksplit; ++ks) {
        const float2 t = __ldcg(reinterpret_cast<const float2*>(part + ((size_t)ks * ROWS + row) * p.N + n));
        v0 += t.x; v1 += t.y;
      }
      if (p.bias) { v0 += bias_to_float(p.bias, p.bias_dtype, n); v1 += bias_to_float(p.bias, p.bias_dtype, n + 1); }
      const uint32_t o = (uint32_t)float_to_raw16<BF16>(v0) | ((uint32_t)float_to_raw16<BF16>(v1) << 16);
      *reinterpret_cast<uint32_t*>(p.out + (size_t)(mbase + row) * p.N + n) = o;
    }
  }
  if (threadIdx.x == 0) *counter = 0;  // leave the workspace as it was found
}

template <int MT, int NG, bool BF16>
static int launch_one(const DecodeParams& dp, const DecodePlan& pl, cudaStream_t st) {
  dim3 grid(pl.ntiles, pl.ksplit, pl.mchunks);
  decode_mma_kernel<MT, NG, BF16><<<grid, kDecodeThreads, 0, st>>>(dp);
  return check_launch();
}

int launch_decode_mma(const GemmArgs& a) {
  const DecodePlan pl = plan_decode(a.M, a.N, a.K, a.g);
  if (pl.mchunks > 65535 || pl.ksplit > 65535) return NQB200_ERR_TOO_LARGE;
  if (pl.ksplit > 1) {
    if (!a.ws || a.ws_bytes < pl.counter_bytes + pl.partial_bytes) return NQB200_ERR_WORKSPACE;
    if (!aligned16(a.ws)) return NQB200_ERR_MISALIGNED;
  }
  DecodeParams dp;
  dp.x = (const uint16_t*)a.x; dp.qw = a.qw; dp.sc = (const uint16_t*)a.sc; dp.qz = a.qz;
  dp.bias = a.bias; dp.bias_dtype = a.bias_dtype; dp.out = (uint16_t*)a.out;
  dp.M = a.M; dp.N = a.N; dp.K = a.K; dp.g = a.g; dp.gpc = pl.gpc; dp.ksplit = pl.ksplit; dp.ntiles = pl.ntiles;
  dp.counters = (int*)a.ws;
  dp.partials = (float*)((char*)a.ws + pl.counter_bytes);
  const bool bf = a.dtype == NQB200_BF16;
  if (pl.mt == 1 && pl.ng == 4) return bf ? launch_one<1, 4, true>(dp, pl, a.stream) : launch_one<1, 4, false>(dp, pl, a.stream);
  if (pl.mt == 1 && pl.ng == 2) return bf ? launch_one<1, 2, true>(dp, pl, a.stream) : launch_one<1, 2, false>(dp, pl, a.stream);
  return bf ? launch_one<2, 2, true>(dp, pl, a.stream) : launch_one<2, 2, false>(dp, pl, a.stream);
}

// ---------------------------------------------------------------------------
// Fallback for shapes the tiled kernels do not take (N % 16 != 0 or a group size
// that is not a multiple of 16): one thread per (token, packed word), weights
// rounded to the 16-bit type exactly as the reference does, fp32 accumulate.
// ---------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(128) generic_kernel(const uint16_t* __restrict__ x, const uint32_t* __restrict__ qw,
                                                      const uint16_t* __restrict__ sc, const uint32_t* __restrict__ qz,
                                                      const void* bias, int bias_dtype, uint16_t* __restrict__ out,
                                                      int M, int N, int K, int g) {
  const int NW = N >> 3;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int m = blockIdx.y;
  if (c >= NW || m >= M) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float s[8]; int z[8];
  for (int k = 0; k < K; ++k) {
    if (k % g == 0) {
      const int gi = k / g;
      const uint32_t zw = qz[(size_t)gi * NW + c];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int sh = (e >> 1) * 4 + (e & 1) * 16;
        z[e] = (zw >> sh) & 0xF;
        s[e] = raw16_to_float<BF16>(sc[(size_t)gi * N + 8 * c + e]);
      }
    }
    const uint32_t w = qw[(size_t)k * NW + c];
    const float xv = raw16_to_float<BF16>(x[(size_t)m * K + k]);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int sh = (e >> 1) * 4 + (e & 1) * 16;
      const float wv = raw16_to_float<BF16>(float_to_raw16<BF16>((float)((int)((w >> sh) & 0xF) - z[e]) * s[e]));
      acc[e] = fmaf(xv, wv, acc[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float v = acc[e];
    if (bias) v += bias_to_float(bias, bias_dtype, 8 * c + e);
    out[(size_t)m * N + 8 * c + e] = float_to_raw16<BF16>(v);
  }
}

int launch_generic(const GemmArgs& a) {
  if (a.M > 65535) return NQB200_ERR_TOO_LARGE;
  dim3 grid((a.N / 8 + 127) / 128, a.M);
  if (a.dtype == NQB200_BF16)
    generic_kernel<true><<<grid, 128, 0, a.stream>>>((const uint16_t*)a.x, a.qw, (const uint16_t*)a.sc, a.qz, a.bias,
                                                     a.bias_dtype, (uint16_t*)a.out, a.M, a.N, a.K, a.g);
  else
    generic_kernel<false><<<grid, 128, 0, a.stream>>>((const uint16_t*)a.x, a.qw, (const uint16_t*)a.sc, a.qz, a.bias,
                                                      a.bias_dtype, (uint16_t*)a.out, a.M, a.N, a.K, a.g);
  return check_launch();
}

}  // namespace nqb200
