// Decode kernel on the 5th-generation tensor cores: W4A16 skinny GEMM for up to
// 16 tokens, group size 128, bound by HBM bandwidth.
//
// The legacy mma.sync path tops out near 256 FMA/clk/SM on this part, below what
// streaming int4 weights at full HBM rate needs, so the contraction runs as
// tcgen05.mma with the weights as the 128-row A operand held in tensor memory
// and the tokens as a 16-column B operand read from shared memory:
//
//   D[n, tok] (TMEM, fp32) = sum_k A[n, k] (TMEM, fp16) * x[tok, k] (smem)
//
// One persistent CTA per SM; units of 128 rows (one group) x 256 columns are
// dealt to CTAs as equal contiguous ranges of u = tile * G + group.
//
//   warp 0      TMA producer: packed weights (128 x 128 B, 128-byte swizzle) into an
//               8-stage ring that the dequantisers release; activations (two
//               16 x 64 boxes, 128-byte swizzle), scales and zero-points into a
//               16-stage ring that lives until the group's epilogue.
//   warps 2-9   dequantisers.  A packed word holds 8 columns of one k; PRMT
//               interleaves byte b of rows k and k+1 and two ANDs leave the
//               nibbles as fp16 subnormals (q * 2^-24, q * 2^-20), two adjacent
//               k per register.  These four registers are exactly what one
//               tcgen05.st.16x128b.x2 wants: lanes g and g+8, columns t and t+4.
//               Byte b of the word goes to lanes 16*(b&1).. of the warp's lane
//               quarter in A block b>>1, so 4 warps x 8 words fill two 128-lane
//               blocks (256 columns of the matrix, in a permuted lane order that
//               the epilogue undoes).  No subtract, no multiply, no smem write.
//   warp 1      issues the MMAs: per 16-row k-step one for each A block.  An MMA
//               that accumulates onto the previous one waits for it (about 120
//               cycles at this tiny N), so the 8 k-steps of a group alternate over
//               2 accumulators per block and the epilogue adds the two.
//   warps 10-13 epilogue, once per group: sum_k x[tok, k] from the activation
//               tile in shared memory, read D, then in fp32
//               total += s * 2^(24|20) * D - s * z * sum(x).
//               At the end of a column tile the totals go to the output (if
//               this CTA saw the tile's whole K) or to a per-CTA slot; the last
//               contributor of a tile adds the slots in CTA order.
//
// Every wait is bounded; on expiry the kernel records NQB200_ERR_WAIT_TIMEOUT in
// the workspace status word, all roles drain, and tensor memory is released.
#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"

namespace nqb200 {
namespace dec {

constexpr int kUnitN = 256, kUnitK = 128;
constexpr int kWStages = 8, kXStages = 16, kAStages = 3, kAcc = 2;
constexpr int kDequantWarps = 8, kEpiWarps = 4;
constexpr int kThreads = (2 + kDequantWarps + kEpiWarps) * 32;
// two rings: the packed weights (released by the dequantisers as soon as they are in tensor memory)
// and the small per-group data -- activations, scales, zero-points -- that the MMAs and the
// epilogue still need much later
constexpr int kWStageBytes = 16384;
constexpr int kOffX0 = 0, kOffX1 = 2048, kOffSc = 4096, kOffZ = 4608, kXStageBytes = 5120;
constexpr int kXRingBase = kWStages * kWStageBytes;
constexpr int kSmem = kXRingBase + kXStages * kXStageBytes + 1024;
constexpr uint32_t kWTx = 16384, kXTx = 4096 + 512 + 128;
constexpr int kColA = 0, kColD = 384, kDBuf = 2 * kAcc * 16, kTmemCols = 512;  // A: 3 x 128 columns, D: 2 x 64
constexpr int kSlotFloats = 16 * kUnitN;
constexpr int kStatusWord = kCounterBytes / 4 - 1;

struct Params {
  const void* bias; int bias_dtype; uint16_t* out;
  int M, N, G, nctas;
  uint32_t U;
  int* counters; float* slots;
};

__device__ __forceinline__ uint32_t cta_begin(uint32_t c, uint32_t U, uint32_t C) { return (c * U) / C; }
__device__ __forceinline__ int cta_of_unit(uint32_t u, uint32_t U, uint32_t C) { return (int)(((u + 1) * C - 1) / U); }

// Bounded wait that also gives up as soon as another role has given up.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  const uint32_t b = smem_u32(bar);
  if (mbar_try_wait(b, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(b, parity)) return true;
    if ((i & 63u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        atomicExch(status, NQB200_ERR_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}

template <int MC, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
umma_decode_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_sc,
                   const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_x, const Params p) {
  constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u;
  constexpr float MULT_LO = BF16 ? 1.f : 16777216.f, MULT_HI = BF16 ? 1.f : 1048576.f, OFF = BF16 ? 128.f : 0.f;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_wfull[kWStages], bar_wempty[kWStages], bar_xfull[kXStages], bar_xempty[kXStages],
      bar_afull[kAStages], bar_aempty[kAStages],
      bar_dfull[2], bar_dempty[2], bar_seg, bar_drain;
  __shared__ uint32_t s_tmem;
  __shared__ int s_last, s_abort_i;
  __shared__ int s_slot[kNumSMs];

  volatile int* s_abort = &s_abort_i;
  int* status = p.counters + kStatusWord;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t U = p.U, C = (uint32_t)p.nctas;
  const uint32_t u_begin = cta_begin(blockIdx.x, U, C), u_end = cta_begin(blockIdx.x + 1, U, C);
  const int nunits = (int)(u_end - u_begin);
  const int G = p.G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWStages; ++s) { mbar_init(smem_u32(&bar_wfull[s]), 1); mbar_init(smem_u32(&bar_wempty[s]), kDequantWarps); }
    for (int s = 0; s < kXStages; ++s) { mbar_init(smem_u32(&bar_xfull[s]), 1); mbar_init(smem_u32(&bar_xempty[s]), 1 + kEpiWarps); }
    for (int s = 0; s < kAStages; ++s) { mbar_init(smem_u32(&bar_afull[s]), kDequantWarps); mbar_init(smem_u32(&bar_aempty[s]), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&bar_dfull[s]), 1); mbar_init(smem_u32(&bar_dempty[s]), kEpiWarps); }
    mbar_init(smem_u32(&bar_seg), kEpiWarps);
    mbar_init(smem_u32(&bar_drain), 1);
    s_abort_i = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(&s_tmem), kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  grid_launch_dependents();
  if (warp != 0) grid_dependency_wait();  // nothing for these warps to do before the activations exist

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tm_w); prefetch_tmap(&tm_sc); prefetch_tmap(&tm_z); prefetch_tmap(&tm_x);
      int tile = (int)(u_begin / G), grp = (int)(u_begin % G);
      int issued = 0;
      // The packed weights are read-only: the first ring of them is requested before the kernel
      // ahead of this one on the stream has finished, everything else after it has.
      const int nfirst = nunits < kWStages ? nunits : kWStages;
      {
        int t2 = tile, g2 = grp;
        for (int i = 0; i < nfirst; ++i) {
          const uint32_t wbar = smem_u32(&bar_wfull[i]);
          mbar_expect_tx(wbar, kWTx);
          tma_load_2d(smem_base + i * kWStageBytes, &tm_w, t2 * 32, g2 * kUnitK, wbar);
          if (++g2 == G) { g2 = 0; ++t2; }
        }
      }
      grid_dependency_wait();
      for (int i = 0; i < nunits; ++i) {
        const int ws = i % kWStages, xs = i % kXStages;
        if (i >= kWStages && !wait_bar(&bar_wempty[ws], ((i / kWStages) - 1) & 1, s_abort, status)) break;
        if (i >= kXStages && !wait_bar(&bar_xempty[xs], ((i / kXStages) - 1) & 1, s_abort, status)) break;
        const uint32_t wst = smem_base + ws * kWStageBytes, xst = smem_base + kXRingBase + xs * kXStageBytes;
        const uint32_t wbar = smem_u32(&bar_wfull[ws]), xbar = smem_u32(&bar_xfull[xs]);
        if (i >= kWStages) {
          mbar_expect_tx(wbar, kWTx);
          tma_load_2d(wst, &tm_w, tile * 32, grp * kUnitK, wbar);
        }
        mbar_expect_tx(xbar, kXTx);
        tma_load_2d(xst + kOffX0, &tm_x, grp * kUnitK, 0, xbar);
        tma_load_2d(xst + kOffX1, &tm_x, grp * kUnitK + 64, 0, xbar);
        tma_load_2d(xst + kOffSc, &tm_sc, tile * 128, grp, xbar);
        tma_load_2d(xst + kOffZ, &tm_z, tile * 32, grp, xbar);
        ++issued;
        if (++grp == G) { grp = 0; ++tile; }
      }
      // do not leave while a copy of ours may still be landing in this CTA's shared memory
      for (int i = issued > kWStages ? issued - kWStages : 0; i < issued; ++i)
        mbar_wait(smem_u32(&bar_wfull[i % kWStages]), (i / kWStages) & 1);
      for (int i = issued > kXStages ? issued - kXStages : 0; i < issued; ++i)
        mbar_wait(smem_u32(&bar_xfull[i % kXStages]), (i / kXStages) & 1);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BF16 ? 1 : 0, 128, 16);
      for (int i = 0; i < nunits; ++i) {
        const int xs = i % kXStages, sa = i % kAStages, sd = i & 1;
        if (!wait_bar(&bar_xfull[xs], (i / kXStages) & 1, s_abort, status)) break;
        if (!wait_bar(&bar_afull[sa], (i / kAStages) & 1, s_abort, status)) break;
        if (i >= 2 && !wait_bar(&bar_dempty[sd], ((i >> 1) - 1) & 1, s_abort, status)) break;
        tc_fence_after();
        const uint32_t xaddr = smem_base + kXRingBase + xs * kXStageBytes + kOffX0;
        const uint32_t a0 = tmem + kColA + sa * 128, a1 = a0 + 64, d = tmem + kColD + sd * kDBuf;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t bdesc = umma_smem_desc_sw128(xaddr + (ks >> 2) * 2048 + (ks & 3) * 32);
          umma_ts(d + 16 * (ks % kAcc), a0 + ks * 8, bdesc, idesc, ks >= kAcc);
          umma_ts(d + 16 * kAcc + 16 * (ks % kAcc), a1 + ks * 8, bdesc, idesc, ks >= kAcc);
        }
        umma_commit(smem_u32(&bar_aempty[sa]));
        umma_commit(smem_u32(&bar_dfull[sd]));
        umma_commit(smem_u32(&bar_xempty[xs]));
      }
      // everything issued has completed before tensor memory may be released
      umma_commit(smem_u32(&bar_drain));
      mbar_wait(smem_u32(&bar_drain), 0);
    }
  } else if (warp < 2 + kDequantWarps) {
    // -------------------------------------------------------------- dequantisers
    const int q = warp & 3, h = (warp - 2) >> 2;
    const int gq = lane >> 2, tig = lane & 3;
    const int chunk = 2 * q + (gq >> 2), inword = (gq & 3) * 4;
    const uint32_t sw_even = ((uint32_t)(chunk ^ ((2 * tig) & 7)) << 4) + inword;
    const uint32_t sw_odd = ((uint32_t)(chunk ^ ((2 * tig + 1) & 7)) << 4) + inword;
    const uint32_t row0 = (uint32_t)(2 * tig) * 128;
    const uint32_t lane_base = tmem + ((uint32_t)(32 * q) << 16);
    for (int i = 0; i < nunits; ++i) {
      const int ws = i % kWStages, sa = i % kAStages;
      if (!wait_bar(&bar_wfull[ws], (i / kWStages) & 1, s_abort, status)) break;
      if (i >= kAStages && !wait_bar(&bar_aempty[sa], ((i / kAStages) - 1) & 1, s_abort, status)) break;
      tc_fence_after();
      const uint8_t* wb = smem_gen + ws * kWStageBytes + row0;
      const uint32_t acol = lane_base + kColA + sa * 128;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int ks = 4 * h + kk;
        const uint8_t* rb = wb + ks * 16 * 128;
        const uint32_t w0 = lds32(rb, sw_even), w1 = lds32(rb, 128 + sw_odd);
        const uint32_t w2 = lds32(rb, 8 * 128 + sw_even), w3 = lds32(rb, 9 * 128 + sw_odd);
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
          tmem_st_16x128b_x2(acol + ((uint32_t)(16 * (b & 1)) << 16) + 64 * (b >> 1) + 8 * ks, a0, a1, a2, a3);
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(smem_u32(&bar_afull[sa])); mbar_arrive(smem_u32(&bar_wempty[ws])); }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int et = threadIdx.x - (2 + kDequantWarps) * 32;  // 0..127 among the epilogue threads
    const uint32_t lane_base = tmem + ((uint32_t)(32 * q) << 16);
    // lane t of the quarter holds, in A block blk, column 64q + 8g + e of the tile
    const int g = lane & 7, r = (lane >> 3) & 1, bb = lane >> 4;
    int nloc[2], jn[2];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const int j = 2 * (2 * blk + bb) + r;
      jn[blk] = j;
      nloc[blk] = 64 * q + 8 * g + ((j < 4) ? 2 * j : 2 * (j - 4) + 1);
    }
    const float mult = r ? MULT_HI : MULT_LO;
    float total[2][MC];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk)
#pragma unroll
      for (int m = 0; m < MC; ++m) total[blk][m] = 0.f;

    int tile = (int)(u_begin / G), grp = (int)(u_begin % G);
    const int first_tile = tile;
    int seg_begin = grp;
    uint32_t seg_phase = 0;

    for (int i = 0; i < nunits; ++i) {
      const int xq = i % kXStages, sd = i & 1;
      if (!wait_bar(&bar_xfull[xq], (i / kXStages) & 1, s_abort, status)) break;  // activations, scales, zero-points
      const uint8_t* st = smem_gen + kXRingBase + xq * kXStageBytes;
      // sum over the group's 128 k of each token: lane l adds k = 4l..4l+3, then a butterfly
      float xs[MC];
      {
        const uint8_t* xb = st + ((lane >> 4) ? kOffX1 : kOffX0) + 8 * (lane & 1);
        const uint32_t ch = (uint32_t)(lane & 15) >> 1;
#pragma unroll
        for (int m = 0; m < MC; ++m) {
          const uint2 v = *reinterpret_cast<const uint2*>(xb + m * 128 + ((ch ^ (uint32_t)(m & 7)) << 4));
          float a = raw16_to_float<BF16>((uint16_t)(v.x & 0xFFFF)) + raw16_to_float<BF16>((uint16_t)(v.x >> 16)) +
                    raw16_to_float<BF16>((uint16_t)(v.y & 0xFFFF)) + raw16_to_float<BF16>((uint16_t)(v.y >> 16));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
          xs[m] = a;
        }
      }
      const uint32_t zw = lds32(st, kOffZ + (uint32_t)(8 * q + g) * 4);
      float cA[2], cB[2];
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        const float sc = raw16_to_float<BF16>(*reinterpret_cast<const uint16_t*>(st + kOffSc + 2 * nloc[blk]));
        const float z = (float)((zw >> (4 * jn[blk])) & 0xF);
        cA[blk] = sc * mult; cB[blk] = sc * (z + OFF);
      }
      if (!wait_bar(&bar_dfull[sd], (i >> 1) & 1, s_abort, status)) break;
      tc_fence_after();
      const uint32_t dcol = lane_base + kColD + sd * kDBuf;
      float dsum[2][MC];
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        uint32_t da[kAcc][MC];
#pragma unroll
        for (int a = 0; a < kAcc; ++a) tmem_ld_cols<MC>(dcol + 16 * kAcc * blk + 16 * a, da[a]);
        tc_wait_ld();
#pragma unroll
        for (int m = 0; m < MC; ++m)
          dsum[blk][m] = __uint_as_float(da[0][m]) + __uint_as_float(da[1][m]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_dempty[sd]));
#pragma unroll
      for (int blk = 0; blk < 2; ++blk)
#pragma unroll
        for (int m = 0; m < MC; ++m) total[blk][m] += cA[blk] * dsum[blk][m] - cB[blk] * xs[m];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_xempty[xq]));

      const bool tile_done = grp == G - 1;
      if (tile_done || i == nunits - 1) {
        const int tn0 = tile * kUnitN;
        if (seg_begin == 0 && tile_done) {
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            const int n = tn0 + nloc[blk];
            if (n < p.N) {
              const float bv = p.bias ? bias_to_float(p.bias, p.bias_dtype, n) : 0.f;
#pragma unroll
              for (int m = 0; m < MC; ++m)
                if (m < p.M) p.out[(size_t)m * p.N + n] = float_to_raw16<BF16>(total[blk][m] + bv);
            }
          }
        } else {
          float* slot = p.slots + ((size_t)blockIdx.x * 2 + (tile == first_tile ? 0 : 1)) * kSlotFloats;
#pragma unroll
          for (int blk = 0; blk < 2; ++blk)
#pragma unroll
            for (int m = 0; m < MC; ++m)
              if (m < p.M) __stcg(slot + m * kUnitN + nloc[blk], total[blk][m]);
          __threadfence();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_seg));
          if (!wait_bar(&bar_seg, seg_phase, s_abort, status)) break;
          seg_phase ^= 1;
          const int first_cta = cta_of_unit((uint32_t)tile * G, U, C);
          const int last_cta = cta_of_unit((uint32_t)tile * G + G - 1, U, C);
          if (et == 0) s_last = (atomicAdd(p.counters + tile, 1) == last_cta - first_cta);
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_seg));
          if (!wait_bar(&bar_seg, seg_phase, s_abort, status)) break;
          seg_phase ^= 1;
          const bool last = s_last != 0;
          if (last) {
            __threadfence();
            for (int c = first_cta + et; c <= last_cta; c += kEpiWarps * 32)
              s_slot[c - first_cta] = 2 * c + ((int)(cta_begin(c, U, C) / G) == tile ? 0 : 1);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_seg));
          if (!wait_bar(&bar_seg, seg_phase, s_abort, status)) break;
          seg_phase ^= 1;
          if (last) {
            const int ncontrib = last_cta - first_cta + 1;
            for (int idx = et; idx < p.M * (kUnitN / 4); idx += kEpiWarps * 32) {
              const int m = idx / (kUnitN / 4), c4 = (idx % (kUnitN / 4)) * 4;
              if (tn0 + c4 < p.N) {
                const float* src = p.slots + m * kUnitN + c4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                // loads of eight contributors are in flight together; the additions stay in CTA order
                for (int c0 = 0; c0 < ncontrib; c0 += 8) {
                  float4 qv[8];
#pragma unroll
                  for (int dd = 0; dd < 8; ++dd)
                    qv[dd] = c0 + dd < ncontrib ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)s_slot[c0 + dd] * kSlotFloats))
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                  for (int dd = 0; dd < 8; ++dd) { v.x += qv[dd].x; v.y += qv[dd].y; v.z += qv[dd].z; v.w += qv[dd].w; }
                }
                if (p.bias) {
                  v.x += bias_to_float(p.bias, p.bias_dtype, tn0 + c4); v.y += bias_to_float(p.bias, p.bias_dtype, tn0 + c4 + 1);
                  v.z += bias_to_float(p.bias, p.bias_dtype, tn0 + c4 + 2); v.w += bias_to_float(p.bias, p.bias_dtype, tn0 + c4 + 3);
                }
                const uint32_t o0 = (uint32_t)float_to_raw16<BF16>(v.x) | ((uint32_t)float_to_raw16<BF16>(v.y) << 16);
                const uint32_t o1 = (uint32_t)float_to_raw16<BF16>(v.z) | ((uint32_t)float_to_raw16<BF16>(v.w) << 16);
                *reinterpret_cast<uint2*>(p.out + (size_t)m * p.N + tn0 + c4) = make_uint2(o0, o1);
              }
            }
            if (et == 0) p.counters[tile] = 0;  // leave the workspace as it was found
          }
          // s_last and s_slot are next written only after another barrier round, which no warp
          // passes before every warp is done with them here
        }
#pragma unroll
        for (int blk = 0; blk < 2; ++blk)
#pragma unroll
          for (int m = 0; m < MC; ++m) total[blk][m] = 0.f;
        seg_begin = 0;
      }
      if (++grp == G) { grp = 0; ++tile; }
    }
  }

  // all roles meet here, also after a give-up, so that tensor memory is always released
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, kTmemCols); }
}

template <int MC, bool BF16>
static int launch_t(const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tz, const CUtensorMap& tx,
                    const Params& sp, cudaStream_t st) {
  static bool configured = false;  // idempotent attribute; a repeated set from two threads is harmless
  if (!configured) {
    if (cudaFuncSetAttribute(umma_decode_kernel<MC, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) {
      cudaGetLastError();
      return NQB200_ERR_LAUNCH;
    }
    configured = true;
  }
  return launch_overlapped(umma_decode_kernel<MC, BF16>, dim3(sp.nctas), dim3(kThreads), kSmem, st, tw, ts, tz, tx, sp);
}

}  // namespace dec

bool umma_decode_supports(int64_t M, int64_t N, int64_t K, int64_t g) {
  const int64_t ntiles = (N + dec::kUnitN - 1) / dec::kUnitN;
  return M >= 1 && M <= 16 && g == 128 && K % 128 == 0 && N % 32 == 0 && ntiles < dec::kStatusWord &&
         ntiles * (K / 128) * kNumSMs < (1ll << 31);
}

size_t umma_decode_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  (void)M;
  const long long U = ((N + dec::kUnitN - 1) / dec::kUnitN) * (K / 128);
  const long long C = U < kNumSMs ? U : kNumSMs;
  return (size_t)kCounterBytes + (size_t)C * 2 * dec::kSlotFloats * sizeof(float);
}

int launch_umma_decode(const GemmArgs& a) {
  using namespace dec;
  const int G = a.K / 128;
  const int ntiles = (a.N + kUnitN - 1) / kUnitN;
  const long long U = (long long)ntiles * G;
  const int C = (int)(U < kNumSMs ? U : kNumSMs);
  if (!a.ws || a.ws_bytes < umma_decode_workspace_bytes(a.M, a.N, a.K)) return NQB200_ERR_WORKSPACE;
  if (!aligned16(a.ws)) return NQB200_ERR_MISALIGNED;
  alignas(64) CUtensorMap tw, ts, tz, tx;
  const CUtensorMapDataType xdt = a.dtype == NQB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  bool ok = encode_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qw, a.K, a.N / 8, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && encode_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.sc, G, a.N / 2, 1, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tz, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qz, G, a.N / 8, 1, 32, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tx, xdt, 2, a.x, a.M, a.K, 16, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return NQB200_ERR_LAUNCH;
  Params sp;
  sp.bias = a.bias; sp.bias_dtype = a.bias_dtype; sp.out = (uint16_t*)a.out;
  sp.M = a.M; sp.N = a.N; sp.G = G; sp.nctas = C; sp.U = (uint32_t)U;
  sp.counters = (int*)a.ws; sp.slots = (float*)((char*)a.ws + kCounterBytes);
  const bool bf = a.dtype == NQB200_BF16;
  if (a.M <= 4) return bf ? launch_t<4, true>(tw, ts, tz, tx, sp, a.stream) : launch_t<4, false>(tw, ts, tz, tx, sp, a.stream);
  if (a.M <= 8) return bf ? launch_t<8, true>(tw, ts, tz, tx, sp, a.stream) : launch_t<8, false>(tw, ts, tz, tx, sp, a.stream);
  return bf ? launch_t<16, true>(tw, ts, tz, tx, sp, a.stream) : launch_t<16, false>(tw, ts, tz, tx, sp, a.stream);
}

}  // namespace nqb200
