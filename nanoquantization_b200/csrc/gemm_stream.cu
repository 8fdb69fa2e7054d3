// Streaming decode kernel: W4A16 skinny GEMM for up to 16 tokens, group size 128.
//
// One persistent CTA per SM.  The packed matrix is cut into units of 128 rows
// (one quantisation group) by 512 columns; unit u = tile * G + group, so that a
// contiguous range of units walks down K inside a column tile.  The CTA holds
// two consumer groups of 8 warps; each group is a worker of its own with its own
// contiguous range of units (296 workers, ranges differ by at most one unit).
// One ring of shared-memory stages serves both: the stages are filled in the
// order worker 0's unit, worker 1's unit, worker 0's next unit, ..., which keeps
// the two groups in step whatever the warp scheduler prefers.
//
//   producer warp : for each unit, four TMA tensor loads into the ring (two
//                   128x128-byte boxes of packed weights with the 128-byte
//                   swizzle, the group's scales and zero-points), completion on
//                   an mbarrier.  About 165 KB per SM is in flight from the first
//                   cycle.  It reads nothing another kernel writes, so under
//                   programmatic stream serialisation it starts before the
//                   kernel ahead of it has finished.
//   activation warp : the group's 128 k of every token by plain loads, stored so
//                   that the four k a consumer thread feeds to one mma
//                   (2t, 2t+1, 2t+8, 2t+9 of a 16-k step) are one 8-byte word,
//                   rows 288 bytes apart (conflict-free), and their sum per token.
//   coefficient warp : per output column of the unit, the two fp32 factors of the
//                   once-per-group correction, scale * 2^p and scale * zero-point,
//                   in the order the consumer threads read them, so that four
//                   lanes do not each convert the same scales and zero-points.
//   2 x 8 consumer warps : warp w owns columns 64w..64w+63 of the tile for the
//                   whole group.  One ldmatrix.x4.trans per 16-k step gives a
//                   thread, per register, four nibbles of row k and the same four
//                   of row k+1: the k pairs that the tensor-core operand wants,
//                   with no byte permutes.  Two masks (and one shift) per
//                   register make four operand registers; the raw nibbles go
//                   into mma.sync m16n8k16 as fp16 subnormals q * 2^-24 and
//                   q * 2^-20 (bf16: 128 + q), and scale, power of two and
//                   zero-point are applied once per group in fp32:
//                   y = sum_g s * (sum_k x q - z sum_k x).
//
// A worker whose range covers a tile's whole K writes the output itself.  Other
// segments go to a per-worker slot (fp32) in the workspace, and a second, small
// kernel adds a tile's slots in worker order (so the result does not depend on
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
#ifndef NQ_EXP
#define NQ_EXP 0
#endif

namespace nqb200 {

constexpr int kUnitN = 512, kUnitK = 128;
constexpr int kGroupWarps = 8, kGroups = 2;                // two workers per CTA
constexpr int kConsumerWarps = kGroupWarps * kGroups;
constexpr int kProducerWarp = kConsumerWarps, kXWarp = kConsumerWarps + 1, kCoefWarp = kConsumerWarps + 2;
constexpr int kStreamThreads = (kConsumerWarps + 3) * 32;
constexpr int kXRow = 288;                                 // bytes between the tokens' rows of a stage's activations
constexpr int kOffW0 = 0, kOffW1 = 16384, kOffX = 32768;

// MT = 1: up to 8 tokens, MT = 2: up to 16.
template <int MT> struct StreamCfg {
  static constexpr int kStages = 5;
  static constexpr int kOffSc = kOffX + 8 * MT * kXRow;
  static constexpr int kOffZ = kOffSc + 1024;
  static constexpr int kOffXs = kOffZ + 256;                  // sum over the group's k of each token, fp32
  static constexpr int kOffCoef = kOffXs + 64;                // [warp][g][A cs0 | A cs1 | B cs0 | B cs1], 16 bytes each
  static constexpr int kStageBytes = (kOffCoef + 4096 + 1023) / 1024 * 1024;
  static constexpr int kSmem = kStages * kStageBytes + 1024;
  static constexpr int kSlotFloats = 8 * MT * kUnitN;         // one segment's slot
  static constexpr uint32_t kStageTx = 2 * 16384 + 1024 + 256;  // what TMA brings: weights, scales, zero-points
};
constexpr int kStatusWord = kCounterBytes / 4 - 1;  // last word of the counter region
constexpr int kMaxWorkers = kNumSMs * kGroups;

struct StreamParams {
  const void* bias; int bias_dtype; uint16_t* out;
  const uint16_t* x;
  int M, N, K, G, ntiles, nctas;  // nctas: workers (consumer groups), two per CTA
  uint32_t U;
  int* counters; float* slots;
  // Optional prologue: x is a residual stream h and the GEMM input is RMSNorm(h) * norm_weight, with
  // mean(h^2) given as sums of squares per (token, 512-column tile of h): norm_ssq[M][norm_tiles].
  const float* norm_ssq; int norm_tiles; const uint16_t* norm_weight; float norm_eps;
  // Optional epilogue of the reducing kernel: out = 16-bit(16-bit(y) + residual_in) (the new residual
  // stream) and its sums of squares per (token, tile) into ssq_out[M][ntiles].
  const uint16_t* residual_in; float* ssq_out;
};

bool stream_supports(int64_t M, int64_t N, int64_t K, int64_t g) {
  return M >= 1 && M <= 16 && g == 128 && K % 128 == 0 && N % 32 == 0 && (N + kUnitN - 1) / kUnitN < kStatusWord;
}

size_t stream_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const long long U = ((N + kUnitN - 1) / kUnitN) * (K / 128);
  const long long C = U < kMaxWorkers ? U : kMaxWorkers;
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

// Four 8x8 matrices of 16-bit elements, transposed: lanes 8i..8i+7 give the addresses of the rows of
// matrix i; register i of thread (g = lane / 4, t = lane % 4) holds elements [2t][g] (low half) and
// [2t+1][g] (high half) of matrix i.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}

// unit ranges in 32-bit arithmetic (the host checks U * C < 2^31): 64-bit division is a long
// dependent instruction sequence on the GPU and these run on the critical path of the tail
__device__ __forceinline__ uint32_t cta_begin(uint32_t c, uint32_t U, uint32_t C) { return c >= C ? U : (c * U) / C; }
__device__ __forceinline__ int cta_of_unit(uint32_t u, uint32_t U, uint32_t C) { return (int)(((u + 1) * C - 1) / U); }

// The ring is filled alternately for the CTA's two workers while both have units left, then for the
// one that has more.  Position in that order of worker `grp`'s j-th unit (n0, n1: the workers' unit counts).
__device__ __forceinline__ int ring_index(int grp, int j, int n0, int n1) {
  const int m = n0 < n1 ? n0 : n1;
  return j < m ? 2 * j + grp : 2 * m + (j - m);
}
// ... and the inverse: worker and j of ring position idx.
__device__ __forceinline__ void ring_owner(int idx, int n0, int n1, int& grp, int& j) {
  const int m = n0 < n1 ? n0 : n1;
  if (idx < 2 * m) { grp = idx & 1; j = idx >> 1; }
  else { grp = n0 > n1 ? 0 : 1; j = m + (idx - 2 * m); }
}

template <int MT, bool BF16, bool NORM>
__global__ void __launch_bounds__(kStreamThreads, 1)
stream_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_sc,
              const __grid_constant__ CUtensorMap tm_z, const StreamParams p) {
  constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u, MAGIC = 0x43004300u;
  constexpr float MULT_LO = BF16 ? 1.f : 16777216.f, MULT_HI = BF16 ? 1.f : 1048576.f, OFF = BF16 ? 128.f : 0.f;
  using Cfg = StreamCfg<MT>;
  constexpr int kStages = Cfg::kStages, kStageBytes = Cfg::kStageBytes, kOffSc = Cfg::kOffSc,
                kOffZ = Cfg::kOffZ, kOffXs = Cfg::kOffXs, kOffCoef = Cfg::kOffCoef, kSlotFloats = Cfg::kSlotFloats;
  constexpr uint32_t kStageTx = Cfg::kStageTx;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages], bar_empty[kStages], bar_x[kStages], bar_coef[kStages];

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));  // same place, generic pointer
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t U = p.U, C = (uint32_t)p.nctas;
  const int G = p.G;
  // the CTA's two workers
  const uint32_t w0 = 2 * blockIdx.x, w1 = w0 + 1;
  const uint32_t begin0 = cta_begin(w0, U, C), begin1 = cta_begin(w1, U, C), end1 = cta_begin(w1 + 1, U, C);
  const int n0 = (int)(begin1 - begin0), n1 = (int)(end1 - begin1);
  const int ntotal = n0 + n1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), kGroupWarps);
      mbar_init(smem_u32(&bar_x[s]), 1); mbar_init(smem_u32(&bar_coef[s]), 1);
    }
    mbar_fence_init();
  }
  __syncthreads();

  grid_launch_dependents();
  if (warp != kProducerWarp && warp != kCoefWarp) grid_dependency_wait();  // these two read only weights, scales and zero-points

  if (warp == kProducerWarp) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      prefetch_tmap(&tm_w); prefetch_tmap(&tm_sc); prefetch_tmap(&tm_z);
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < ntotal; ++i) {
        int grp, j;
        ring_owner(i, n0, n1, grp, j);
        const uint32_t u = (grp ? begin1 : begin0) + (uint32_t)j;
        const int tile = (int)(u / (uint32_t)G), gk = (int)(u % (uint32_t)G);
        const int s = i % kStages;
        if (i >= kStages && !mbar_wait(smem_u32(&bar_empty[s]), ((i / kStages) - 1) & 1)) { ok = false; break; }
        const uint32_t st = smem_base + s * kStageBytes, bar = smem_u32(&bar_full[s]);
#ifdef NQ_GEOM
        mbar_expect_tx(bar, 32768);
        for (int b = 0; b < 128 / NQ_GEOM * 2; ++b)
          tma_load_2d(st + b * (NQ_GEOM * 128), &tm_w, tile * (64 * 128 / NQ_GEOM) + 32 * b, gk * NQ_GEOM, bar);
#else
        mbar_expect_tx(bar, kStageTx);
        tma_load_2d(st + kOffW0, &tm_w, tile * 64, gk * kUnitK, bar);
        tma_load_2d(st + kOffW1, &tm_w, tile * 64 + 32, gk * kUnitK, bar);
        tma_load_2d(st + kOffSc, &tm_sc, tile * 256, gk, bar);
        tma_load_2d(st + kOffZ, &tm_z, tile * 64, gk, bar);
#endif
        ++issued;
      }
      if (!ok) { grid_dependency_wait(); atomicExch(p.counters + kStatusWord, NQB200_ERR_WAIT_TIMEOUT); }
      // do not leave while a copy of ours may still be landing in this CTA's shared memory
      for (int i = issued > kStages ? issued - kStages : 0; i < issued; ++i)
        mbar_wait(smem_u32(&bar_full[i % kStages]), (i / kStages) & 1);
    }
    return;
  }
  if (warp == kXWarp) {
    // --------------------------------------------------------- activation warp
    // Brings the group's 128 k of every token from global memory with plain loads (they are small,
    // L2-resident and must not queue behind the weight boxes).  Lanes 0-15 hold one token's 256 bytes
    // (lane c: k = 8c..8c+7), lanes 16-31 the next token's.  A 16-k step's halves go to
    // [step][t][k = 2t, 2t+1, 2t+8, 2t+9], 32 bytes per step: lane c writes its four k pairs to
    // step c/2, t = 0..3, at byte 4 * (c % 2) of t's 8 bytes.
    const int cc = lane & 15, half = lane >> 4;
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
    for (int i = 0; i < ntotal; ++i) {
      int grp, jj;
      ring_owner(i, n0, n1, grp, jj);
      const int gk = (int)(((grp ? begin1 : begin0) + (uint32_t)jj) % (uint32_t)G);
      const int s = i % kStages;
      if (i >= kStages && !mbar_wait(smem_u32(&bar_empty[s]), ((i / kStages) - 1) & 1)) {
        atomicExch(p.counters + kStatusWord, NQB200_ERR_WAIT_TIMEOUT);
        break;
      }
      uint8_t* st = smem_gen + s * kStageBytes;
#if NQ_EXP == 2 || NQ_EXP == 3 || defined(NQ_GEOM)
      if (p.M > 0) { if (lane == 0) mbar_arrive(smem_u32(&bar_x[s])); continue; }
#endif
      uint4 v[4 * MT];
#pragma unroll
      for (int j = 0; j < 4 * MT; ++j) {
        const int m = 2 * j + half;
        v[j] = m < p.M ? __ldcg(reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + gk * kUnitK) + cc) : make_uint4(0u, 0u, 0u, 0u);
      }
      uint4 nw = make_uint4(0u, 0u, 0u, 0u);
      if (NORM) nw = __ldg(reinterpret_cast<const uint4*>(p.norm_weight + gk * kUnitK) + cc);
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
        uint32_t* row = reinterpret_cast<uint32_t*>(st + kOffX + m * kXRow + (cc >> 1) * 32 + (cc & 1) * 4);
        row[0] = v[j].x; row[2] = v[j].y; row[4] = v[j].z; row[6] = v[j].w;
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
      if (lane == 0) mbar_arrive(smem_u32(&bar_x[s]));
    }
    return;
  }
  if (warp == kCoefWarp) {
    // ------------------------------------------------------- coefficient warp
    // Lane l converts words l and l + 32 of the unit's 64 packed words of zero-points (8 columns each)
    // and their 8 scales.  Word W = 32 box + 4 chunk + wd belongs to consumer warp 4 box + chunk / 2,
    // chunk half cs = chunk % 2; its even columns are read by the threads with g = 2 wd, its odd columns
    // by g = 2 wd + 1, column 2 i + parity as the i-th of the thread's four.
    for (int i = 0; i < ntotal; ++i) {
      const int s = i % kStages;
      if (!mbar_wait(smem_u32(&bar_full[s]), (i / kStages) & 1)) {
        grid_dependency_wait();
        atomicExch(p.counters + kStatusWord, NQB200_ERR_WAIT_TIMEOUT);
        break;
      }
      uint8_t* st = smem_gen + s * kStageBytes;
#if NQ_EXP == 2 || NQ_EXP == 4 || defined(NQ_GEOM)
      if (p.M > 0) { if (lane == 0) mbar_arrive(smem_u32(&bar_coef[s])); continue; }
#endif
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int Wd = lane + 32 * h;
        const uint4 sv = lds128(st, kOffSc + (uint32_t)Wd * 16);
        const uint32_t zw = lds32(st, kOffZ + (uint32_t)Wd * 4);
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
        float A[8], B[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float sc = raw16_to_float<BF16>((uint16_t)((sw[e >> 1] >> (16 * (e & 1))) & 0xFFFF));
          const float z = (float)((zw >> (4 * (e >> 1) + 16 * (e & 1))) & 0xF);
          A[e] = sc * (((e >> 1) & 1) ? MULT_HI : MULT_LO);
          B[e] = sc * (z + OFF);
        }
        const int wcons = 4 * (Wd >> 5) + (((Wd >> 2) & 7) >> 1), cs = (Wd >> 2) & 1, wd = Wd & 3;
        uint8_t* even = st + kOffCoef + (wcons * 8 + 2 * wd) * 64 + 16 * cs;
        *reinterpret_cast<float4*>(even) = make_float4(A[0], A[2], A[4], A[6]);
        *reinterpret_cast<float4*>(even + 32) = make_float4(B[0], B[2], B[4], B[6]);
        *reinterpret_cast<float4*>(even + 64) = make_float4(A[1], A[3], A[5], A[7]);
        *reinterpret_cast<float4*>(even + 96) = make_float4(B[1], B[3], B[5], B[7]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_coef[s]));
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  const int grp = warp >> 3, w = warp & 7;
  const int g = lane >> 2, t = lane & 3;
  const int nunits = grp ? n1 : n0;
  const uint32_t u_begin = grp ? begin1 : begin0;
  const int worker = (int)(grp ? w1 : w0);
  // ldmatrix: lanes 8i..8i+7 address matrix i = (chunk half i / 2, k half i % 2), row lane % 8
  const uint32_t ld_off = (uint32_t)(w >> 2) * 16384u + (uint32_t)(8 * ((lane >> 3) & 1) + (lane & 7)) * 128u +
                          ((uint32_t)((2 * (w & 3) + (lane >> 4)) ^ (lane & 7)) << 4);
  const uint32_t x_off = (uint32_t)kOffX + (uint32_t)g * kXRow + (uint32_t)t * 8;
  const uint32_t coef_off = (uint32_t)kOffCoef + (uint32_t)(w * 8 + g) * 64;

  float total[MT][4][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int d = 0; d < 4; ++d)
#pragma unroll
      for (int i = 0; i < 4; ++i) total[mt][d][i] = 0.f;

  int tile = (int)(u_begin / (uint32_t)G), gk = (int)(u_begin % (uint32_t)G);
  const int first_tile = tile;
  int seg_begin = gk;

  for (int j = 0; j < nunits; ++j) {
    const int idx = ring_index(grp, j, n0, n1);
    const int s = idx % kStages;
    const uint32_t par = (uint32_t)(idx / kStages) & 1u;
    if (!mbar_wait(smem_u32(&bar_coef[s]), par) || !mbar_wait(smem_u32(&bar_full[s]), par) ||
        !mbar_wait(smem_u32(&bar_x[s]), par)) {
      atomicExch(p.counters + kStatusWord, NQB200_ERR_WAIT_TIMEOUT);
      break;
    }
    const uint8_t* st = smem_gen + s * kStageBytes;
    const uint32_t st_s = smem_base + s * kStageBytes;

    float acc[MT][4][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int d = 0; d < 4; ++d)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[mt][d][q] = 0.f;

#if NQ_EXP == 1 || defined(NQ_GEOM)
    if (p.M < 0)
#endif
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t R[4];
      ldmatrix_x4_trans(R, st_s + ld_off + ks * 2048);
      uint2 xb[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) xb[mt] = *reinterpret_cast<const uint2*>(st + x_off + mt * 8 * kXRow + ks * 32);
#pragma unroll
      for (int cs = 0; cs < 2; ++cs) {
#pragma unroll
        for (int ph = 0; ph < 2; ++ph) {
          uint32_t a0, a1, a2, a3;
          if (BF16) {
            a0 = ((R[2 * cs] >> (8 * ph)) & LO) | MAGIC; a1 = ((R[2 * cs] >> (8 * ph + 4)) & LO) | MAGIC;
            a2 = ((R[2 * cs + 1] >> (8 * ph)) & LO) | MAGIC; a3 = ((R[2 * cs + 1] >> (8 * ph + 4)) & LO) | MAGIC;
          } else {
            const uint32_t l = R[2 * cs] >> (8 * ph), h = R[2 * cs + 1] >> (8 * ph);
            a0 = l & LO; a1 = l & HI; a2 = h & LO; a3 = h & HI;
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma16816s<BF16>(acc[mt][2 * cs + ph], a0, a1, a2, a3, xb[mt].x, xb[mt].y);
        }
      }
    }

    // scale, power of two and zero-point, once per group
    {
      const float4 A0 = *reinterpret_cast<const float4*>(st + coef_off), A1 = *reinterpret_cast<const float4*>(st + coef_off + 16);
      const float4 B0 = *reinterpret_cast<const float4*>(st + coef_off + 32), B1 = *reinterpret_cast<const float4*>(st + coef_off + 48);
      const float cA[2][4] = {{A0.x, A0.y, A0.z, A0.w}, {A1.x, A1.y, A1.z, A1.w}};
      const float cB[2][4] = {{B0.x, B0.y, B0.z, B0.w}, {B1.x, B1.y, B1.z, B1.w}};
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const float2 xs = *reinterpret_cast<const float2*>(st + kOffXs + 4 * (8 * mt + 2 * t));
#pragma unroll
        for (int cs = 0; cs < 2; ++cs)
#pragma unroll
          for (int ph = 0; ph < 2; ++ph)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const float a = cA[cs][2 * ph + r], b = cB[cs][2 * ph + r];
              float* tt = total[mt][2 * cs + ph];
              const float* ac = acc[mt][2 * cs + ph];
              tt[2 * r] = fmaf(a, ac[2 * r], fmaf(-b, xs.x, tt[2 * r]));
              tt[2 * r + 1] = fmaf(a, ac[2 * r + 1], fmaf(-b, xs.y, tt[2 * r + 1]));
            }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bar_empty[s]));

    const bool tile_done = gk == G - 1;
    if (tile_done || j == nunits - 1) {
      // Thread (g, t) holds, per token pair and chunk half cs, columns nb + 2i + g % 2 (i = 2 ph + r) of
      // nb = 32 (2 (w % 4) + cs) + 8 (g / 2) in its 256-column box; lane ^ 4 holds the other parity.  After
      // one exchange the even-g lane has columns nb..nb+3 and the odd-g lane nb+4..nb+7, contiguous.
      const bool direct = seg_begin == 0 && tile_done;  // this worker saw the tile's whole K: write the output itself
      float* slot = p.slots + ((size_t)worker * 2 + (tile == first_tile ? 0 : 1)) * kSlotFloats;
      const int odd = g & 1;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int tk = 0; tk < 2; ++tk) {
          const int m = 8 * mt + 2 * t + tk;
#pragma unroll
          for (int cs = 0; cs < 2; ++cs) {
            const float v0 = total[mt][2 * cs][tk], v1 = total[mt][2 * cs][2 + tk];
            const float v2 = total[mt][2 * cs + 1][tk], v3 = total[mt][2 * cs + 1][2 + tk];
            const float r0 = __shfl_xor_sync(0xFFFFFFFFu, odd ? v0 : v2, 4);
            const float r1 = __shfl_xor_sync(0xFFFFFFFFu, odd ? v1 : v3, 4);
            float o0, o1, o2, o3;
            if (odd) { o0 = r0; o1 = v2; o2 = r1; o3 = v3; } else { o0 = v0; o1 = r0; o2 = v1; o3 = r1; }
            const int ncol = 256 * (w >> 2) + 32 * (2 * (w & 3) + cs) + 8 * (g >> 1) + 4 * odd;  // within the tile
            const int n = tile * kUnitN + ncol;
            if (m < p.M && n < p.N) {
              if (direct) {
                if (p.bias) {
                  o0 += bias_to_float(p.bias, p.bias_dtype, n); o1 += bias_to_float(p.bias, p.bias_dtype, n + 1);
                  o2 += bias_to_float(p.bias, p.bias_dtype, n + 2); o3 += bias_to_float(p.bias, p.bias_dtype, n + 3);
                }
                *reinterpret_cast<uint2*>(p.out + (size_t)m * p.N + n) =
                    make_uint2((uint32_t)float_to_raw16<BF16>(o0) | ((uint32_t)float_to_raw16<BF16>(o1) << 16),
                               (uint32_t)float_to_raw16<BF16>(o2) | ((uint32_t)float_to_raw16<BF16>(o3) << 16));
              } else {
                __stcg(reinterpret_cast<float4*>(slot + m * kUnitN + ncol), make_float4(o0, o1, o2, o3));  // rows beyond M are never read
              }
            }
          }
        }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int d = 0; d < 4; ++d)
#pragma unroll
          for (int q = 0; q < 4; ++q) total[mt][d][q] = 0.f;
      seg_begin = 0;
    }
    if (++gk == G) { gk = 0; ++tile; }
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

// Sets the kernel's attributes on the current device (once per device) and checks that a CTA fits an SM;
// the persistent grid (one CTA per SM) must be resident all at once.
template <int MT, bool BF16>
static bool stream_configure() {
  static std::mutex mu;
  static int state[kMaxDevices] = {0};  // 0 unknown, 1 ok, -1 failed
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return false; }
  std::lock_guard<std::mutex> lock(mu);
  if (state[dev] == 0) {
    constexpr int kStreamSmem = StreamCfg<MT>::kSmem;
    int n = 0, n2 = 0;
    const bool ok =
        cudaFuncSetAttribute(stream_kernel<MT, BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem) == cudaSuccess &&
        cudaFuncSetAttribute(stream_kernel<MT, BF16, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, stream_kernel<MT, BF16, false>, kStreamThreads, kStreamSmem) == cudaSuccess &&
        cudaFuncSetAttribute(stream_kernel<MT, BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem) == cudaSuccess &&
        cudaFuncSetAttribute(stream_kernel<MT, BF16, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n2, stream_kernel<MT, BF16, true>, kStreamThreads, kStreamSmem) == cudaSuccess;
    if (!ok) cudaGetLastError();
    state[dev] = ok && n >= 1 && n2 >= 1 ? 1 : -1;
  }
  return state[dev] == 1;
}

template <int MT, bool BF16>
static int launch_stream_t(const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tz, const StreamParams& sp,
                           int max_contributors, bool silu, const PeerEpilogue* peer, cudaStream_t st) {
  if (!stream_configure<MT, BF16>()) return NQB200_ERR_LAUNCH;
  const dim3 main_grid((sp.nctas + kGroups - 1) / kGroups);
  const int rc = sp.norm_ssq ? launch_overlapped(stream_kernel<MT, BF16, true>, main_grid, dim3(kStreamThreads), StreamCfg<MT>::kSmem, st, tw, ts, tz, sp)
                             : launch_overlapped(stream_kernel<MT, BF16, false>, main_grid, dim3(kStreamThreads), StreamCfg<MT>::kSmem, st, tw, ts, tz, sp);
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
  const long long U = (long long)ntiles * G, cap = (long long)kMaxWorkers;
  int fewest = 0;
  stream_max_contributors(ntiles, G, (int)(U < cap ? U : cap), &fewest);
  return fewest >= 2;
}

// The all-reduce epilogue needs every tile reduced by the second kernel and a flag set per CTA of it.
bool stream_allreduce_supported(int64_t M, int64_t N, int64_t K, int64_t g) {
  if (!stream_supports(M, N, K, g)) return false;
  const int G = (int)(K / 128), ntiles = (int)((N + kUnitN - 1) / kUnitN);
  const long long U = (long long)ntiles * G, cap = (long long)kMaxWorkers;
  int fewest = 0;
  stream_max_contributors(ntiles, G, (int)(U < cap ? U : cap), &fewest);
  return fewest >= 2 && (long long)ntiles * M <= kEpilogueSets;
}

// 2 when some tile needs the reducing kernel.  Assumes the full occupancy the kernel is built for.
int stream_launches(int64_t M, int64_t N, int64_t K) {
  const int G = (int)(K / 128), ntiles = (int)((N + kUnitN - 1) / kUnitN);
  const long long U = (long long)ntiles * G, cap = (long long)kMaxWorkers;
  return stream_max_contributors(ntiles, G, (int)(U < cap ? U : cap)) > 1 ? 2 : 1;
}

int launch_stream(const GemmArgs& a) {
#ifdef NQ_GEOM
  const int G = a.K / NQ_GEOM;
  const int ntiles = (a.N + kUnitN * (128 / NQ_GEOM) - 1) / (kUnitN * (128 / NQ_GEOM));
#else
  const int G = a.K / 128;
  const int ntiles = (a.N + kUnitN - 1) / kUnitN;
#endif
  const long long U = (long long)ntiles * G;
  if ((U + 1) * kMaxWorkers >= (1ll << 31)) return NQB200_ERR_TOO_LARGE;
  const int mt = a.M > 8 ? 2 : 1;
  const bool bf = a.dtype == NQB200_BF16;
  const long long cap = (long long)kMaxWorkers;
  const int C = (int)(U < cap ? U : cap);
  if (!a.ws || a.ws_bytes < stream_workspace_bytes(a.M, a.N, a.K)) return NQB200_ERR_WORKSPACE;
  if (!aligned16(a.ws)) return NQB200_ERR_MISALIGNED;
  alignas(64) CUtensorMap tw, ts, tz;
#ifdef NQ_GEOM
  bool ok = encode_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qw, a.K, a.N / 8, NQ_GEOM, 32, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && encode_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.sc, a.K / 128, a.N / 2, 1, 256, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tz, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qz, a.K / 128, a.N / 8, 1, 64, CU_TENSOR_MAP_SWIZZLE_NONE);
#else
  bool ok = encode_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qw, a.K, a.N / 8, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && encode_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.sc, G, a.N / 2, 1, 256, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tz, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qz, G, a.N / 8, 1, 64, CU_TENSOR_MAP_SWIZZLE_NONE);
#endif
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
// holds from load until exit (kNoAllocScratchBytes, about 18.6 MiB).
//
// The name `g_noalloc_scratch` is only a host-side handle here, not a device
// address; the device address is fetched once per device with
// cudaGetSymbolAddress (with that device current) and passed to the kernel.
// ---------------------------------------------------------------------------
namespace nqb200 {
// counters + two slots of 16 tokens x 512 columns (fp32) for each of the 296 workers
constexpr size_t kNoAllocScratchBytes = (size_t)kCounterBytes + (size_t)kMaxWorkers * 2 * 16 * kUnitN * sizeof(float);
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
