// Streaming decode kernel: W4A16 skinny GEMM for up to 16 tokens, group size 128.
//
// One persistent CTA per SM.  The packed matrix is cut into units of 128 rows
// (one quantisation group) by 512 columns; unit u = tile * G + group, so that a
// CTA's contiguous range of units walks down K inside a column tile.  The 148
// CTAs take equal contiguous ranges (sizes differ by at most one unit).
//
//   producer warp : for each unit, four TMA tensor loads into a shared-memory
//                   ring (two 128x128-byte boxes of packed weights with the
//                   128-byte swizzle, the group's scales and zero-points),
//                   completion on an mbarrier.  About 190 KB per SM is in flight
//                   from the first cycle, which is what keeps HBM busy at these
//                   sizes.  It reads nothing another kernel writes, so under
//                   programmatic stream serialisation it starts before the
//                   kernel ahead of it has finished.
//   activation warp : the group's 128 k of every token by plain loads into the
//                   stage (swizzled like a TMA tile), and their sum per token
//                   (the tensor pipe is this kernel's scarce resource, so the sum
//                   is not done with an all-ones mma).
//   8 consumer warps : warp w owns columns 64w..64w+63 of the tile for the whole
//                   group; arithmetic as in the register-fed kernel (raw nibbles
//                   as fp16 subnormals into mma.sync m16n8k16, scale and
//                   zero-point applied once per group in fp32).  The 128-byte swizzle and
//                   the mma's own k order (2t, 2t+1, 2t+8, 2t+9) make every
//                   shared-memory load conflict-free.
//
// A CTA whose range covers a tile's whole K writes the output itself.  Other
// segments go to a per-CTA slot (fp32) in the workspace, and a second, small
// kernel adds a tile's slots in CTA order (so the result does not depend on
// timing), adds the bias and writes the output.  Both kernels are launched with
// programmatic stream serialisation: the second is resident before the first
// ends, and the next layer's weights start to stream while it runs.
//
// Every wait is bounded; on expiry the kernel records NQB200_ERR_WAIT_TIMEOUT in
// the workspace status word and drains instead of spinning.
#include "common.cuh"
#include "tma_utils.cuh"
#include "peer_layout.cuh"
#include <mutex>

namespace nqb200 {

constexpr int kUnitN = 512, kUnitK = 128;
constexpr int kConsumerWarps = 8;
constexpr int kStreamThreads = (kConsumerWarps + 2) * 32;  // consumers, TMA producer, sum(x) warp
constexpr int kOffW0 = 0, kOffW1 = 16384, kOffX0 = 32768;

// Up to 8 tokens (MT = 1): two CTAs per SM with three stages each, so that 16 consumer warps
// share an SM's issue slots.  Up to 16 tokens (MT = 2): one CTA per SM with five stages.
template <int MT> struct StreamCfg {
  static constexpr int kCtasPerSm = MT == 1 ? 2 : 1;
  static constexpr int kStages = MT == 1 ? 3 : 5;
  static constexpr int kXBox = 8 * MT * 128;                 // bytes of one activation box
  static constexpr int kOffX1 = kOffX0 + kXBox;
  static constexpr int kOffSc = kOffX0 + 2 * kXBox;
  static constexpr int kOffZ = kOffSc + 1024;
  static constexpr int kOffXs = kOffZ + 256;                  // sum over the group's k of each token, fp32
  static constexpr int kStageBytes = (kOffXs + 64 + 1023) / 1024 * 1024;
  static constexpr int kSmem = kStages * kStageBytes + 1024;
  static constexpr int kSlotFloats = 8 * MT * kUnitN;         // one segment's slot
  static constexpr uint32_t kStageTx = 2 * 16384 + 1024 + 256;  // what TMA brings: weights, scales, zero-points
};
constexpr int kStatusWord = kCounterBytes / 4 - 1;  // last word of the counter region

struct StreamParams {
  const void* bias; int bias_dtype; uint16_t* out;
  const uint16_t* x;
  int M, N, K, G, ntiles, nctas;
  uint32_t U;
  int* counters; float* slots;
  // Optional prologue: x is a residual stream h and the GEMM input is RMSNorm(h) * norm_weight, with
  // mean(h^2) given as sums of squares per (token, 512-column tile of h): norm_ssq[M][norm_tiles].
  const float* norm_ssq; int norm_tiles; const uint16_t* norm_weight; float norm_eps;
  // Optional epilogue of the reducing kernel: out = 16-bit(16-bit(y) + residual_in) (the new residual
  // stream) and its sums of squares per (token, tile) into ssq_out[M][ntiles].
  const uint16_t* residual_in; float* ssq_out;
};

int stream_tile_columns() { return kUnitN; }

bool stream_supports(int64_t M, int64_t N, int64_t K, int64_t g) {
  return M >= 1 && M <= 16 && g == 128 && K % 128 == 0 && N % 32 == 0 && (N + kUnitN - 1) / kUnitN < kStatusWord;
}

size_t stream_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const long long U = ((N + kUnitN - 1) / kUnitN) * (K / 128);
  const long long cap = (long long)kNumSMs * (M > 8 ? 1 : 2);
  const long long C = U < cap ? U : cap;
  return (size_t)kCounterBytes + (size_t)C * 2 * (size_t)(M > 8 ? 16 : 8) * kUnitN * sizeof(float);
}

template <bool BF16>
__device__ __forceinline__ void mma16816s(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// unit ranges in 32-bit arithmetic (the host checks U * C < 2^31): 64-bit division is a long
// dependent instruction sequence on the GPU and these run on the critical path of the tail
__device__ __forceinline__ uint32_t cta_begin(uint32_t c, uint32_t U, uint32_t C) { return (c * U) / C; }
__device__ __forceinline__ int cta_of_unit(uint32_t u, uint32_t U, uint32_t C) { return (int)(((u + 1) * C - 1) / U); }

// value of column e (0..7) of a thread's 8-column group, row t of the token pair
#define NQ_TOTAL_AT(tot, e, t) tot[((e) & 1 ? 4 + ((e) >> 1) : ((e) >> 1)) >> 1][2 * (((e) & 1 ? 4 + ((e) >> 1) : ((e) >> 1)) & 1) + (t)]

template <int MT, bool BF16, bool NORM>
__global__ void __launch_bounds__(kStreamThreads, StreamCfg<MT>::kCtasPerSm)
stream_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_sc,
              const __grid_constant__ CUtensorMap tm_z, const StreamParams p) {
  constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u;
  constexpr float MULT_LO = BF16 ? 1.f : 16777216.f, MULT_HI = BF16 ? 1.f : 1048576.f, OFF = BF16 ? 128.f : 0.f;
  using Cfg = StreamCfg<MT>;
  constexpr int kStages = Cfg::kStages, kStageBytes = Cfg::kStageBytes, kOffX1 = Cfg::kOffX1, kOffSc = Cfg::kOffSc,
                kOffZ = Cfg::kOffZ, kOffXs = Cfg::kOffXs, kSlotFloats = Cfg::kSlotFloats;
  constexpr uint32_t kStageTx = Cfg::kStageTx;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages], bar_empty[kStages], bar_xs[kStages];

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));  // same place, generic pointer
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t U = p.U, C = (uint32_t)p.nctas;
  const uint32_t u_begin = cta_begin(blockIdx.x, U, C), u_end = cta_begin(blockIdx.x + 1, U, C);
  const int nunits = (int)(u_end - u_begin);
  const int G = p.G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), kConsumerWarps); mbar_init(smem_u32(&bar_xs[s]), 1);
    }
    mbar_fence_init();
  }
  __syncthreads();

  grid_launch_dependents();
  if (warp != kConsumerWarps) grid_dependency_wait();  // all but the TMA producer touch what the kernel ahead may still write

  if (warp == kConsumerWarps) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      prefetch_tmap(&tm_w); prefetch_tmap(&tm_sc); prefetch_tmap(&tm_z);
      int tile = (int)(u_begin / G), grp = (int)(u_begin % G);
      int issued = 0;
      bool ok = true;
      // Everything this thread requests (packed weights, scales, zero-points) is read-only, so it
      // does not wait for the kernel ahead of this one on the stream; the activations come through
      // the activation warp, which does.
      for (int i = 0; i < nunits; ++i) {
        const int s = i % kStages;
        if (i >= kStages && !mbar_wait(smem_u32(&bar_empty[s]), ((i / kStages) - 1) & 1)) { ok = false; break; }
        const uint32_t st = smem_base + s * kStageBytes, bar = smem_u32(&bar_full[s]);
        mbar_expect_tx(bar, kStageTx);
        tma_load_2d(st + kOffW0, &tm_w, tile * 64, grp * kUnitK, bar);
        tma_load_2d(st + kOffW1, &tm_w, tile * 64 + 32, grp * kUnitK, bar);
        tma_load_2d(st + kOffSc, &tm_sc, tile * 256, grp, bar);
        tma_load_2d(st + kOffZ, &tm_z, tile * 64, grp, bar);
        ++issued;
        if (++grp == G) { grp = 0; ++tile; }
      }
      if (!ok) { grid_dependency_wait(); atomicExch(p.counters + kStatusWord, NQB200_ERR_WAIT_TIMEOUT); }
      // do not leave while a copy of ours may still be landing in this CTA's shared memory
      for (int i = issued > kStages ? issued - kStages : 0; i < issued; ++i)
        mbar_wait(smem_u32(&bar_full[i % kStages]), (i / kStages) & 1);
    }
    return;
  }
  if (warp == kConsumerWarps + 1) {
    // --------------------------------------------------------- activation warp
    // Brings the group's 128 k of every token from global memory with plain loads (they are small,
    // L2-resident and must not queue behind the weight boxes), stores them in the layout of a
    // 128-byte-swizzled tile (16-byte chunk c of row m at chunk c ^ (m & 7)), and leaves each
    // token's sum over the group beside them.  Lanes 0-15 hold one token's 256 bytes, lanes 16-31
    // the next token's.
    const int cc = lane & 15, half = lane >> 4;
    int grp = (int)(u_begin % G);
    // With the RMSNorm prologue: 1 / rms of token `lane` from the per-tile sums of squares (added
    // in tile order), handed to the lanes that need it by shuffles.
    float inv_mine = 0.f;
    if (NORM && lane < p.M) {
      float tot = 0.f;
      for (int tl = 0; tl < p.norm_tiles; ++tl) tot += __ldcg(p.norm_ssq + (size_t)lane * p.norm_tiles + tl);
      inv_mine = rsqrtf(tot / (float)p.K + p.norm_eps);
    }
    float inv_tok[4 * MT];
#pragma unroll
    for (int j = 0; j < 4 * MT; ++j) inv_tok[j] = __shfl_sync(0xFFFFFFFFu, inv_mine, (2 * j + half) & 31);
    for (int i = 0; i < nunits; ++i) {
      const int s = i % kStages;
      if (i >= kStages && !mbar_wait(smem_u32(&bar_empty[s]), ((i / kStages) - 1) & 1)) {
        atomicExch(p.counters + kStatusWord, NQB200_ERR_WAIT_TIMEOUT);
        break;
      }
      uint8_t* st = const_cast<uint8_t*>(smem_gen) + s * kStageBytes;
      uint4 v[4 * MT];
#pragma unroll
      for (int j = 0; j < 4 * MT; ++j) {
        const int m = 2 * j + half;
        v[j] = m < p.M ? __ldcg(reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + grp * kUnitK) + cc) : make_uint4(0u, 0u, 0u, 0u);
      }
      uint4 nw = make_uint4(0u, 0u, 0u, 0u);
      if (NORM) nw = __ldg(reinterpret_cast<const uint4*>(p.norm_weight + grp * kUnitK) + cc);
#pragma unroll
      for (int j = 0; j < 4 * MT; ++j) {
        const int m = 2 * j + half;
        if (NORM) {
          // 16-bit(16-bit(h * inv) * w), the roundings of the norm as a kernel of its own
          const uint32_t hw[4] = {v[j].x, v[j].y, v[j].z, v[j].w}, ww[4] = {nw.x, nw.y, nw.z, nw.w};
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a0 = raw16_to_float<BF16>(float_to_raw16<BF16>(raw16_to_float<BF16>((uint16_t)(hw[e] & 0xFFFF)) * inv_tok[j]));
            const float a1 = raw16_to_float<BF16>(float_to_raw16<BF16>(raw16_to_float<BF16>((uint16_t)(hw[e] >> 16)) * inv_tok[j]));
            o[e] = (uint32_t)float_to_raw16<BF16>(a0 * raw16_to_float<BF16>((uint16_t)(ww[e] & 0xFFFF))) |
                   ((uint32_t)float_to_raw16<BF16>(a1 * raw16_to_float<BF16>((uint16_t)(ww[e] >> 16))) << 16);
          }
          v[j] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        *reinterpret_cast<uint4*>(st + ((cc >> 3) ? kOffX1 : kOffX0) + m * 128 + (((cc & 7) ^ (m & 7)) << 4)) = v[j];
        const uint32_t wds[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        float a = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          a += raw16_to_float<BF16>((uint16_t)(wds[e] & 0xFFFF)) + raw16_to_float<BF16>((uint16_t)(wds[e] >> 16));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
        if (cc == 0) *reinterpret_cast<float*>(st + kOffXs + 4 * m) = a;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_xs[s]));
      if (++grp == G) grp = 0;
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  const int gq = lane >> 2, tig = lane & 3;
  const int w = warp;
  const int chunk = 2 * (w & 3) + (gq >> 2), inword = (gq & 3) * 4;
  const uint32_t w_off = (w >> 2) ? kOffW1 : kOffW0;
  // rows 16ks + 2tig + {0,1,8,9}: (row & 7) is 2tig or 2tig+1
  const uint32_t sw_even = ((uint32_t)(chunk ^ ((2 * tig) & 7)) << 4) + inword;
  const uint32_t sw_odd = ((uint32_t)(chunk ^ ((2 * tig + 1) & 7)) << 4) + inword;
  const uint32_t row0 = (uint32_t)(2 * tig) * 128;

  float total[MT][4][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) total[mt][b][i] = 0.f;

  int tile = (int)(u_begin / G), grp = (int)(u_begin % G);
  const int first_tile = tile;
  int seg_begin = grp;
  bool alive = true;

  for (int i = 0; i < nunits && alive; ++i) {
    const int s = i % kStages;
    if (!mbar_wait(smem_u32(&bar_full[s]), (i / kStages) & 1)) {
      atomicExch(p.counters + kStatusWord, NQB200_ERR_WAIT_TIMEOUT);
      alive = false;
      break;
    }
    if (!mbar_wait(smem_u32(&bar_xs[s]), (i / kStages) & 1)) {
      atomicExch(p.counters + kStatusWord, NQB200_ERR_WAIT_TIMEOUT);
      alive = false;
      break;
    }
    const uint8_t* st = smem_gen + s * kStageBytes;
    const uint8_t* wb = st + w_off + row0;

    float acc[MT][4][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[mt][b][q] = 0.f;
    }

#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint8_t* rb = wb + ks * 16 * 128;
      const uint32_t w0 = lds32(rb, sw_even), w1 = lds32(rb, 128 + sw_odd);
      const uint32_t w2 = lds32(rb, 8 * 128 + sw_even), w3 = lds32(rb, 9 * 128 + sw_odd);
      uint32_t xb0[MT], xb1[MT];
      const uint8_t* xbox = st + ((ks >> 2) ? kOffX1 : kOffX0);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint8_t* xr = xbox + (uint32_t)(8 * mt + gq) * 128 + tig * 4;
        xb0[mt] = lds32(xr, (uint32_t)((2 * (ks & 3)) ^ gq) << 4);
        xb1[mt] = lds32(xr, (uint32_t)((2 * (ks & 3) + 1) ^ gq) << 4);
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t sel = (uint32_t)b | ((uint32_t)b << 4) | ((uint32_t)(4 + b) << 8) | ((uint32_t)(4 + b) << 12);
        const uint32_t p01 = __byte_perm(w0, w1, sel), p23 = __byte_perm(w2, w3, sel);
        uint32_t a0, a1, a2, a3;
        if (BF16) {
          a0 = (p01 & LO) | 0x43004300u; a1 = ((p01 >> 4) & LO) | 0x43004300u;
          a2 = (p23 & LO) | 0x43004300u; a3 = ((p23 >> 4) & LO) | 0x43004300u;
        } else {
          a0 = p01 & LO; a1 = p01 & HI; a2 = p23 & LO; a3 = p23 & HI;
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) mma16816s<BF16>(acc[mt][b], a0, a1, a2, a3, xb0[mt], xb1[mt]);
      }
    }

    // scale, power of two and zero-point, once per group
    {
      float xs[MT][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const float2 v = *reinterpret_cast<const float2*>(st + kOffXs + 4 * (8 * mt + 2 * tig));
        xs[mt][0] = v.x; xs[mt][1] = v.y;
      }
      const uint4 sv = lds128(st, kOffSc + (uint32_t)(64 * w + 8 * gq) * 2);
      const uint32_t zw = lds32(st, kOffZ + (uint32_t)(8 * w + gq) * 4);
      const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int b = j >> 1, r = j & 1;
        const int e = (j < 4) ? 2 * j : 2 * (j - 4) + 1;
        const float sc = raw16_to_float<BF16>((uint16_t)((sw[e >> 1] >> (16 * (e & 1))) & 0xFFFF));
        const float z = (float)((zw >> (4 * j)) & 0xF);
        const float A = sc * (r ? MULT_HI : MULT_LO), B = sc * (z + OFF);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int t = 0; t < 2; ++t) total[mt][b][2 * r + t] += A * acc[mt][b][2 * r + t] - B * xs[mt][t];
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bar_empty[s]));

    const bool tile_done = grp == G - 1;
    if (tile_done || i == nunits - 1) {
      const int n0 = tile * kUnitN + 64 * w + 8 * gq;
      const bool n_ok = n0 < p.N;
      if (seg_begin == 0 && tile_done) {
        // this CTA saw the tile's whole K: write the output directly
        if (n_ok) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int m = 8 * mt + 2 * tig + t;
              if (m < p.M) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                  float v0 = NQ_TOTAL_AT(total[mt], e, t), v1 = NQ_TOTAL_AT(total[mt], e + 1, t);
                  if (p.bias) { v0 += bias_to_float(p.bias, p.bias_dtype, n0 + e); v1 += bias_to_float(p.bias, p.bias_dtype, n0 + e + 1); }
                  o[e >> 1] = (uint32_t)float_to_raw16<BF16>(v0) | ((uint32_t)float_to_raw16<BF16>(v1) << 16);
                }
                *reinterpret_cast<uint4*>(p.out + (size_t)m * p.N + n0) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
        }
      } else {
        // rows beyond M are never read
        float* slot = p.slots + ((size_t)blockIdx.x * 2 + (tile == first_tile ? 0 : 1)) * kSlotFloats;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const int m = 8 * mt + 2 * tig + t;
            if (m < p.M) {
              float* dst = slot + m * kUnitN + 64 * w + 8 * gq;
              __stcg(reinterpret_cast<float4*>(dst), make_float4(NQ_TOTAL_AT(total[mt], 0, t), NQ_TOTAL_AT(total[mt], 1, t),
                                                                 NQ_TOTAL_AT(total[mt], 2, t), NQ_TOTAL_AT(total[mt], 3, t)));
              __stcg(reinterpret_cast<float4*>(dst + 4), make_float4(NQ_TOTAL_AT(total[mt], 4, t), NQ_TOTAL_AT(total[mt], 5, t),
                                                                     NQ_TOTAL_AT(total[mt], 6, t), NQ_TOTAL_AT(total[mt], 7, t)));
            }
          }
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int q = 0; q < 4; ++q) total[mt][b][q] = 0.f;
      seg_begin = 0;
    }
    if (++grp == G) { grp = 0; ++tile; }
  }

}

// Sum over the contributors j, j+W, j+2W, ... of one tile's partial segments for token m, columns
// col..col+3: all of a thread's loads (up to eight) are in flight together.  Returns the number of
// contributors of the tile.
template <int kReduceWays>
__device__ __forceinline__ int reduce_tile_partials(const StreamParams& p, int C, int slot_floats, int tile, int m, int col, int j,
                                                    float4& v) {
  const int G = p.G;
  const uint32_t U = p.U;
  const int first_cta = cta_of_unit((uint32_t)tile * G, U, (uint32_t)C);
  const int nc = cta_of_unit((uint32_t)tile * G + G - 1, U, (uint32_t)C) - first_cta + 1;
  // the first contributor's segment is its last one unless its range starts with this tile
  const int first_slot = 2 * first_cta + ((int)(cta_begin(first_cta, U, (uint32_t)C) / G) == tile ? 0 : 1);
  const float* base = p.slots + (size_t)m * kUnitN + col;
  v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (nc == 1) return 1;
  for (int c0 = j; c0 < nc; c0 += 8 * kReduceWays) {
    float4 q[8];
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      const int c = c0 + kReduceWays * d < nc ? c0 + kReduceWays * d : 0;  // beyond the last: a valid address, value unused
      const float* src = base + (size_t)(c == 0 ? first_slot : 2 * (first_cta + c)) * slot_floats;
      asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(q[d].x), "=f"(q[d].y), "=f"(q[d].z), "=f"(q[d].w) : "l"(src));
    }
#pragma unroll
    for (int d = 0; d < 8; ++d)
      if (c0 + kReduceWays * d < nc) { v.x += q[d].x; v.y += q[d].y; v.z += q[d].z; v.w += q[d].w; }
  }
  return nc;
}

// Last step of the reducing kernels, called by every thread of the CTA: the owner threads (one per
// four columns) hold the finished fp32 values `a`.  Without a residual they are rounded and stored to
// out.  With one, out gets the new residual stream 16-bit(16-bit(a) + residual_in) and the CTA adds
// the squares of what it stored into ssq_out[token][tile] (shuffles, then the four owner warps in
// order), for the RMSNorm prologue of the next linear.
template <bool BF16>
__device__ __forceinline__ void store_reduced(const StreamParams& p, int tile, int m, int n, bool owner, const float (&a)[4],
                                              float* s_red) {
  const size_t elem = (size_t)m * p.N + n;
  if (!p.residual_in) {
    if (owner)
      *reinterpret_cast<uint2*>(p.out + elem) =
          make_uint2((uint32_t)float_to_raw16<BF16>(a[0]) | ((uint32_t)float_to_raw16<BF16>(a[1]) << 16),
                     (uint32_t)float_to_raw16<BF16>(a[2]) | ((uint32_t)float_to_raw16<BF16>(a[3]) << 16));
    return;
  }
  float ss = 0.f;
  if (owner) {
    const uint2 r = __ldcg(reinterpret_cast<const uint2*>(p.residual_in + elem));
    const uint32_t rw[2] = {r.x, r.y};
    uint16_t h[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float y = raw16_to_float<BF16>(float_to_raw16<BF16>(a[k]));
      h[k] = float_to_raw16<BF16>(y + raw16_to_float<BF16>((uint16_t)((rw[k >> 1] >> (16 * (k & 1))) & 0xFFFF)));
      const float hf = raw16_to_float<BF16>(h[k]);
      ss += hf * hf;
    }
    *reinterpret_cast<uint2*>(p.out + elem) = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
  }
  const int lin = (int)(threadIdx.y * blockDim.x + threadIdx.x);  // owners are threads 0..127: warps 0..3
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if (lin < 128 && (lin & 31) == 0) s_red[lin >> 5] = ss;
  __syncthreads();
  if (lin == 0) p.ssq_out[(size_t)m * p.ntiles + tile] = ((s_red[0] + s_red[1]) + s_red[2]) + s_red[3];
}

// Adds the partial segments of one tile (blockIdx.x) and token (blockIdx.y).  Thread (t, j) owns
// columns 4t..4t+3 and the contributors j, j+W, j+2W, ... (W = 1 when a tile has at most eight
// contributors, else 4); the W partial sums of a column meet in shared memory, always in the same
// order, so the result does not depend on timing.  Tiles that one CTA of the main kernel covered
// alone were written there.
//
// SILU: the matrix is a merged gate|up projection (N = 2 I).  The CTA adds tile blockIdx.x of the
// gate half and the same tile of the up half and writes silu(gate) * up to out[M, I], with the
// roundings of the separate steps (each half to 16 bits, silu to 16 bits, the product to 16 bits:
// models/qwen3_quantized.py:150 of the reference).  The host takes this path only when every tile
// has more than one contributor.
template <bool BF16, int kReduceWays, bool SILU>
__global__ void __launch_bounds__(kUnitN / 4 * kReduceWays) stream_reduce_kernel(const StreamParams p, const int C, const int slot_floats) {
  __shared__ float4 part[SILU ? 2 : 1][kReduceWays][kUnitN / 4];
  grid_launch_dependents();
  grid_dependency_wait();
  const int tile = (int)blockIdx.x, m = (int)blockIdx.y;
  const int t = (int)threadIdx.x, j = (int)threadIdx.y;
  const int col = 4 * t, n = tile * kUnitN + col;
  float4 v, u = make_float4(0.f, 0.f, 0.f, 0.f);
  const int nc = reduce_tile_partials<kReduceWays>(p, C, slot_floats, tile, m, col, j, v);
  if (!SILU && nc == 1) return;
  const int half_n = p.N / 2;
  if (SILU) reduce_tile_partials<kReduceWays>(p, C, slot_floats, tile + p.ntiles / 2, m, col, j, u);
  part[0][j][t] = v;
  if (SILU) part[SILU ? 1 : 0][j][t] = u;
  __syncthreads();
  const bool owner = j == 0 && n < (SILU ? half_n : p.N);
  if (owner) {
#pragma unroll
    for (int k = 1; k < kReduceWays; ++k) {
      const float4 o = part[0][k][t];
      v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
      if (SILU) { const float4 o2 = part[SILU ? 1 : 0][k][t]; u.x += o2.x; u.y += o2.y; u.z += o2.z; u.w += o2.w; }
    }
    if (p.bias) {
      v.x += bias_to_float(p.bias, p.bias_dtype, n); v.y += bias_to_float(p.bias, p.bias_dtype, n + 1);
      v.z += bias_to_float(p.bias, p.bias_dtype, n + 2); v.w += bias_to_float(p.bias, p.bias_dtype, n + 3);
      if (SILU) {
        u.x += bias_to_float(p.bias, p.bias_dtype, half_n + n); u.y += bias_to_float(p.bias, p.bias_dtype, half_n + n + 1);
        u.z += bias_to_float(p.bias, p.bias_dtype, half_n + n + 2); u.w += bias_to_float(p.bias, p.bias_dtype, half_n + n + 3);
      }
    }
  }
  if (SILU) {
    if (!owner) return;
    auto act = [](float g, float up) {
      g = raw16_to_float<BF16>(float_to_raw16<BF16>(g));
      up = raw16_to_float<BF16>(float_to_raw16<BF16>(up));
      const float sl = raw16_to_float<BF16>(float_to_raw16<BF16>(g / (1.f + expf(-g))));
      return sl * up;
    };
    v.x = act(v.x, u.x); v.y = act(v.y, u.y); v.z = act(v.z, u.z); v.w = act(v.w, u.w);
    const uint32_t o0 = (uint32_t)float_to_raw16<BF16>(v.x) | ((uint32_t)float_to_raw16<BF16>(v.y) << 16);
    const uint32_t o1 = (uint32_t)float_to_raw16<BF16>(v.z) | ((uint32_t)float_to_raw16<BF16>(v.w) << 16);
    *reinterpret_cast<uint2*>(p.out + (size_t)m * half_n + n) = make_uint2(o0, o1);
    return;
  }
  __shared__ float s_red[4];
  const float a[4] = {v.x, v.y, v.z, v.w};
  store_reduced<BF16>(p, tile, m, n, owner, a, s_red);
}

// The reducing kernel of a row-parallel linear under tensor parallelism, with the all-reduce over
// the ranks in the same launch.  Each CTA adds the split-K partial sums of its tile and token as
// above, rounds them to the 16-bit type (what the GEMM alone would output) and stores them straight
// into the slot of every rank's peer-mapped buffer (area `source rank` of the slot), then raises its
// flag on every rank, waits for every rank's flag on its own, adds the ranks' areas of its own slot
// in rank order (identical bits on all ranks), adds the bias once and writes the output.  One NVLink
// crossing per value and no launch of its own for the collective.  Flags only grow: each flag set
// (one per CTA of the grid) counts its own calls in device memory, so the launch can be replayed
// from a CUDA graph; slots are used round-robin by the caller, so an area is rewritten only after
// every rank has passed the flags of a later call.  Waits are bounded (about a second) and record
// NQB200_ERR_WAIT_TIMEOUT in the buffer's status word.  Plain peer stores and loads only.
template <bool BF16, int kReduceWays>
__global__ void __launch_bounds__(kUnitN / 4 * kReduceWays)
stream_reduce_allreduce_kernel(const StreamParams p, const int C, const int slot_floats, const __grid_constant__ PeerEpilogue pe) {
  __shared__ float4 part[kReduceWays][kUnitN / 4];
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  grid_launch_dependents();
  grid_dependency_wait();
  const int tile = (int)blockIdx.x, m = (int)blockIdx.y;
  const int t = (int)threadIdx.x, j = (int)threadIdx.y;
  const int col = 4 * t, n = tile * kUnitN + col;
  float4 v;
  reduce_tile_partials<kReduceWays>(p, C, slot_floats, tile, m, col, j, v);
  part[j][t] = v;
  const int set = (int)(blockIdx.y * gridDim.x + blockIdx.x);
  uint8_t* mine = pe.peers[pe.rank];
  if (t == 0 && j == 0) {
    uint32_t* ep = reinterpret_cast<uint32_t*>(mine + kArOffEpoch2) + set;
    s_epoch = *ep + 1;
    *ep = s_epoch;
    s_ok = 1;
  }
  __syncthreads();
  const bool owner = j == 0 && n < p.N;
  const size_t mn = (size_t)p.M * p.N, elem = (size_t)m * p.N + n;
  if (owner) {
#pragma unroll
    for (int k = 1; k < kReduceWays; ++k) { const float4 o = part[k][t]; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
    const uint2 w = make_uint2((uint32_t)float_to_raw16<BF16>(v.x) | ((uint32_t)float_to_raw16<BF16>(v.y) << 16),
                               (uint32_t)float_to_raw16<BF16>(v.z) | ((uint32_t)float_to_raw16<BF16>(v.w) << 16));
    for (int r = 0; r < pe.world; ++r)
      *reinterpret_cast<uint2*>(pe.peers[r] + kArOffData + pe.slot_off + ((size_t)pe.rank * mn + elem) * 2) = w;
  }
  __syncthreads();  // every store of this CTA is ordered before the flags raised below
  const uint32_t e = s_epoch;
  const int lin = j * (int)blockDim.x + t;
  if (lin < pe.world) {
    st_flag(reinterpret_cast<uint32_t*>(pe.peers[lin] + kArOffFlags2) + (size_t)set * kMaxRanks + pe.rank, e);
    const uint32_t* ours = reinterpret_cast<const uint32_t*>(mine + kArOffFlags2) + (size_t)set * kMaxRanks + lin;
    const unsigned long long t0 = global_timer_ns(), limit = peer_wait_limit_ns(mine);
    uint32_t it = 0;
    while ((int32_t)(ld_flag(ours) - e) < 0) {  // a rank already one call ahead shows e + 1
      if ((++it & 255u) == 0 && global_timer_ns() - t0 > limit) {
        atomicExch(reinterpret_cast<int*>(mine), NQB200_ERR_WAIT_TIMEOUT);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (owner) {
    for (int r = 0; r < pe.world; ++r) {
      uint32_t w0, w1;
      asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(w0), "=r"(w1)
                   : "l"(mine + kArOffData + pe.slot_off + ((size_t)r * mn + elem) * 2) : "memory");
      acc[0] += raw16_to_float<BF16>((uint16_t)(w0 & 0xFFFF)); acc[1] += raw16_to_float<BF16>((uint16_t)(w0 >> 16));
      acc[2] += raw16_to_float<BF16>((uint16_t)(w1 & 0xFFFF)); acc[3] += raw16_to_float<BF16>((uint16_t)(w1 >> 16));
    }
    if (p.bias) {
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] += bias_to_float(p.bias, p.bias_dtype, n + k);
    }
  }
  __shared__ float s_red[4];
  store_reduced<BF16>(p, tile, m, n, owner, acc, s_red);
}

// CTAs of this kernel that one SM holds at a time (0 on error): the persistent grid is sized so
// that all of it is resident at once.
template <int MT, bool BF16>
static int stream_ctas_per_sm() {
  // measured once per device (the attributes set here belong to the device that is current)
  static std::mutex mu;
  static int occ[kMaxDevices];
  static bool known[kMaxDevices] = {false};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return 0; }
  std::lock_guard<std::mutex> lock(mu);
  if (!known[dev]) {
    constexpr int kStreamSmem = StreamCfg<MT>::kSmem;
    int n = 0;
    int n2 = 0;
    if (cudaFuncSetAttribute(stream_kernel<MT, BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem) != cudaSuccess ||
        cudaFuncSetAttribute(stream_kernel<MT, BF16, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, stream_kernel<MT, BF16, false>, kStreamThreads, kStreamSmem) != cudaSuccess ||
        cudaFuncSetAttribute(stream_kernel<MT, BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem) != cudaSuccess ||
        cudaFuncSetAttribute(stream_kernel<MT, BF16, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n2, stream_kernel<MT, BF16, true>, kStreamThreads, kStreamSmem) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    if (n2 < n) n = n2;
    occ[dev] = n < StreamCfg<MT>::kCtasPerSm ? n : StreamCfg<MT>::kCtasPerSm;
    known[dev] = true;
  }
  return occ[dev];
}

template <int MT, bool BF16>
static int launch_stream_t(const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tz, const StreamParams& sp,
                           int max_contributors, bool silu, const PeerEpilogue* peer, cudaStream_t st) {
  // the attributes were set when the occupancy was measured
  const int rc = sp.norm_ssq ? launch_overlapped(stream_kernel<MT, BF16, true>, dim3(sp.nctas), dim3(kStreamThreads), StreamCfg<MT>::kSmem, st, tw, ts, tz, sp)
                             : launch_overlapped(stream_kernel<MT, BF16, false>, dim3(sp.nctas), dim3(kStreamThreads), StreamCfg<MT>::kSmem, st, tw, ts, tz, sp);
  if (rc != NQB200_OK || max_contributors <= 1) return rc;
  const int sf = (int)StreamCfg<MT>::kSlotFloats;
  if (peer)
    return max_contributors <= 8
               ? launch_overlapped(stream_reduce_allreduce_kernel<BF16, 1>, dim3(sp.ntiles, sp.M), dim3(kUnitN / 4, 1), 0, st, sp, sp.nctas, sf, *peer)
               : launch_overlapped(stream_reduce_allreduce_kernel<BF16, 4>, dim3(sp.ntiles, sp.M), dim3(kUnitN / 4, 4), 0, st, sp, sp.nctas, sf, *peer);
  const dim3 grid(silu ? sp.ntiles / 2 : sp.ntiles, sp.M);
  if (max_contributors <= 8)
    return silu ? launch_overlapped(stream_reduce_kernel<BF16, 1, true>, grid, dim3(kUnitN / 4, 1), 0, st, sp, sp.nctas, sf)
                : launch_overlapped(stream_reduce_kernel<BF16, 1, false>, grid, dim3(kUnitN / 4, 1), 0, st, sp, sp.nctas, sf);
  return silu ? launch_overlapped(stream_reduce_kernel<BF16, 4, true>, grid, dim3(kUnitN / 4, 4), 0, st, sp, sp.nctas, sf)
              : launch_overlapped(stream_reduce_kernel<BF16, 4, false>, grid, dim3(kUnitN / 4, 4), 0, st, sp, sp.nctas, sf);
}

// the most contributors any tile has (same arithmetic as the kernels)
static int stream_max_contributors(int ntiles, int G, int C, int* fewest = nullptr) {
  const unsigned long long U = (unsigned long long)ntiles * G;
  int most = 1, least = 1 << 30;
  for (int t = 0; t < ntiles; ++t) {
    const unsigned long long u0 = (unsigned long long)t * G, u1 = u0 + G - 1;
    const int nc = (int)(((u1 + 1) * C - 1) / U - ((u0 + 1) * C - 1) / U) + 1;
    if (nc > most) most = nc;
    if (nc < least) least = nc;
  }
  if (fewest) *fewest = least;
  return most;
}

// The merged gate|up epilogue needs both halves tile-aligned and every tile reduced by the second
// kernel (a tile that one CTA covers alone is written by the main kernel, before the activation).
// Assumes the full occupancy the kernel is built for; launch_stream checks again with the real one.
bool stream_silu_supported(int64_t M, int64_t N, int64_t K, int64_t g) {
  if (!stream_supports(M, N, K, g) || N % (2 * kUnitN) != 0) return false;
  const int G = (int)(K / 128), ntiles = (int)(N / kUnitN);
  const long long U = (long long)ntiles * G, cap = (long long)kNumSMs * (M > 8 ? 1 : 2);
  int fewest = 0;
  stream_max_contributors(ntiles, G, (int)(U < cap ? U : cap), &fewest);
  return fewest >= 2;
}

// The all-reduce epilogue needs every tile reduced by the second kernel and a flag set per CTA of it.
bool stream_allreduce_supported(int64_t M, int64_t N, int64_t K, int64_t g) {
  if (!stream_supports(M, N, K, g)) return false;
  const int G = (int)(K / 128), ntiles = (int)((N + kUnitN - 1) / kUnitN);
  const long long U = (long long)ntiles * G, cap = (long long)kNumSMs * (M > 8 ? 1 : 2);
  int fewest = 0;
  stream_max_contributors(ntiles, G, (int)(U < cap ? U : cap), &fewest);
  return fewest >= 2 && (long long)ntiles * M <= kEpilogueSets;
}

// 2 when some tile needs the reducing kernel.  Assumes the full occupancy the kernel is built for.
int stream_launches(int64_t M, int64_t N, int64_t K) {
  const int G = (int)(K / 128), ntiles = (int)((N + kUnitN - 1) / kUnitN);
  const long long U = (long long)ntiles * G, cap = (long long)kNumSMs * (M > 8 ? 1 : 2);
  return stream_max_contributors(ntiles, G, (int)(U < cap ? U : cap)) > 1 ? 2 : 1;
}

int launch_stream(const GemmArgs& a) {
  const int G = a.K / 128;
  const int ntiles = (a.N + kUnitN - 1) / kUnitN;
  const long long U = (long long)ntiles * G;
  if (U * 2 * kNumSMs >= (1ll << 31)) return NQB200_ERR_TOO_LARGE;
  const int mt = a.M > 8 ? 2 : 1;
  const bool bf = a.dtype == NQB200_BF16;
  const int per_sm = mt == 1 ? (bf ? stream_ctas_per_sm<1, true>() : stream_ctas_per_sm<1, false>())
                             : (bf ? stream_ctas_per_sm<2, true>() : stream_ctas_per_sm<2, false>());
  if (per_sm <= 0) return NQB200_ERR_LAUNCH;
  const long long cap = (long long)kNumSMs * per_sm;
  const int C = (int)(U < cap ? U : cap);
  if (!a.ws || a.ws_bytes < stream_workspace_bytes(a.M, a.N, a.K)) return NQB200_ERR_WORKSPACE;
  if (!aligned16(a.ws)) return NQB200_ERR_MISALIGNED;
  alignas(64) CUtensorMap tw, ts, tz;
  bool ok = encode_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qw, a.K, a.N / 8, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && encode_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.sc, G, a.N / 2, 1, 256, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tz, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qz, G, a.N / 8, 1, 64, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (!ok) return NQB200_ERR_LAUNCH;
  StreamParams sp;
  sp.bias = a.bias; sp.bias_dtype = a.bias_dtype; sp.out = (uint16_t*)a.out;
  sp.x = (const uint16_t*)a.x;
  sp.M = a.M; sp.N = a.N; sp.K = a.K; sp.G = G; sp.ntiles = ntiles; sp.nctas = C; sp.U = (uint32_t)U;
  sp.counters = (int*)a.ws; sp.slots = (float*)((char*)a.ws + kCounterBytes);
  sp.norm_ssq = a.norm_ssq; sp.norm_tiles = a.norm_tiles; sp.norm_weight = (const uint16_t*)a.norm_weight; sp.norm_eps = a.norm_eps;
  sp.residual_in = (const uint16_t*)a.residual_in; sp.ssq_out = a.ssq_out;
  int fewest = 0;
  const int reduce = stream_max_contributors(ntiles, G, C, &fewest);
  const bool silu = a.epilogue == 1;
  if (silu && (a.N % (2 * kUnitN) != 0 || fewest < 2)) return NQB200_ERR_BAD_SHAPE;
  const PeerEpilogue* peer = a.peer;
  if (peer && (silu || fewest < 2 || (long long)ntiles * a.M > kEpilogueSets)) return NQB200_ERR_BAD_SHAPE;
  if (a.residual_in && (silu || fewest < 2 || !a.ssq_out)) return NQB200_ERR_BAD_SHAPE;
  if (a.norm_ssq && (!a.norm_weight || a.norm_tiles <= 0)) return NQB200_ERR_BAD_SHAPE;
  if (mt == 1) return bf ? launch_stream_t<1, true>(tw, ts, tz, sp, reduce, silu, peer, a.stream) : launch_stream_t<1, false>(tw, ts, tz, sp, reduce, silu, peer, a.stream);
  return bf ? launch_stream_t<2, true>(tw, ts, tz, sp, reduce, silu, peer, a.stream) : launch_stream_t<2, false>(tw, ts, tz, sp, reduce, silu, peer, a.stream);
}

}  // namespace nqb200

// ---------------------------------------------------------------------------
// Decode GEMM for callers that may not allocate device memory.
//
// Some hosts of this library own every byte of device memory themselves: a
// serving engine that has already handed all free HBM to its KV-cache pool, or
// a plugin interface that gives the plugin no allocator and treats a cudaMalloc
// from inside it as an error.  Such a caller cannot create the scratch buffer
// that nqb200_gemm expects.  For them the scratch of the streaming decode kernel
// lives in the fixed array below, which every GPU that loads this library
// holds from load until exit (kNoAllocScratchBytes, about 9.4 MiB).
//
// The name `g_noalloc_scratch` is only a host-side handle here, not a device
// address; the device address is fetched once per device with
// cudaGetSymbolAddress (with that device current) and passed to the kernel.
// ---------------------------------------------------------------------------
namespace nqb200 {
// counters + two slots for each of the 296 CTAs of the 8-token configuration (the 16-token
// configuration needs the same: 148 CTAs with slots twice the size)
constexpr size_t kNoAllocScratchBytes = (size_t)kCounterBytes + (size_t)2 * kNumSMs * 2 * 8 * kUnitN * sizeof(float);
}  // namespace nqb200

static __device__ __align__(256) unsigned char g_noalloc_scratch[nqb200::kNoAllocScratchBytes];

static void* noalloc_scratch_for_current_device(int* status) {
  static std::mutex mu;
  static void* ptrs[nqb200::kMaxDevices] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= nqb200::kMaxDevices) {
    cudaGetLastError();
    *status = NQB200_ERR_UNSUPPORTED_DEVICE;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) {
      cudaGetLastError();
      *status = NQB200_ERR_LAUNCH;
      return nullptr;
    }
    ptrs[dev] = ptr;
  }
  return ptrs[dev];
}

extern "C" int nqb200_gemm_decode_noalloc(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                                          const void* bias, int bias_dtype, void* out, int64_t M, int64_t N, int64_t K,
                                          int64_t group_size, int dtype, void* stream) {
  using namespace nqb200;
  if (M < 0 || N <= 0 || K <= 0 || group_size <= 0 || K % group_size != 0 || N % 8 != 0) return NQB200_ERR_BAD_SHAPE;
  if (dtype != NQB200_F16 && dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  if (M == 0) return NQB200_OK;
  // beyond what the fixed scratch was sized for: more than 16 tokens, or a shape the streaming
  // kernel does not take (it needs group size 128 and N a multiple of 32)
  if (M > 16 || !stream_supports(M, N, K, group_size) || stream_workspace_bytes(M, N, K) > kNoAllocScratchBytes)
    return NQB200_ERR_TOO_LARGE;
  if (!x || !qweight || !qscales || !qzeros || !out) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(qscales) || !aligned16(qzeros) || !aligned16(out) ||
      (bias && !aligned16(bias)))
    return NQB200_ERR_MISALIGNED;
  if (bias && bias_dtype != NQB200_F16 && bias_dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  int st = NQB200_OK;
  void* scratch = noalloc_scratch_for_current_device(&st);
  if (!scratch) return st;
  // The array keeps whatever the previous call left.  The streaming kernels read a slot only after
  // this call's own kernel has written it, so only the status word of bounded waits must start at
  // zero: four bytes on the caller's stream, no allocation.
  if (cudaMemsetAsync(reinterpret_cast<int*>(scratch) + kStatusWord, 0, sizeof(int), (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return NQB200_ERR_LAUNCH;
  }
  GemmArgs a;
  a.x = x; a.qw = (const uint32_t*)qweight; a.sc = qscales; a.qz = (const uint32_t*)qzeros;
  a.bias = bias; a.bias_dtype = bias_dtype; a.out = out;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.g = (int)group_size; a.dtype = dtype;
  a.ws = scratch; a.ws_bytes = kNoAllocScratchBytes; a.stream = (cudaStream_t)stream;
  return launch_stream(a);
}
