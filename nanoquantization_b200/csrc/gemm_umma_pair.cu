// Prefill kernel for many tokens on the 5th-generation tensor cores: W4A16 GEMM, group size 128, two SMs per
// tile (tcgen05.mma.cta_group::2).  Replaces what the reference does from 256 tokens on -- a Triton kernel that
// writes the dense 16-bit weight to HBM, then torch.matmul (nanoquantization/layers/gemm.py:10-123, 552-567) --
// with one kernel that never materialises the dense weight.
//
//   D[n, tok] (TMEM, fp32) = sum_k W[k, n] (TMEM, 16-bit) * x[tok, k] (smem)
//
// The weights are the A operand, dequantised to their true 16-bit values (q - z) * s -- the integer difference
// first, then one multiply, which is the reference's rounding -- straight from registers into tensor memory; the
// tokens are the N dimension of the MMA, read from shared memory as a K-major operand that TMA wrote with the
// 128-byte swizzle.  A dequantised value never touches shared memory.
//
// A dequantised weight should feed as many tokens as possible, and the activations should be fetched as rarely as
// possible.  The two CTAs of a cluster (the two SMs of a TPC) work as one: M = 256 weight columns (128 from each
// CTA's tensor memory: one A block of 64 columns per 128-k slot, four slots) by N = up to 256 tokens, of which each
// CTA loads only its half.  Per CTA and 128-k unit: 8.5 KB of packed weights, scales and zero-points, at most
// 32 KB of activations, and 8 MMAs of about 141 cycles.  Tensor memory is full: 256 columns of A ring and 256 of
// accumulator, so the accumulator is single and the tensor pipe idles while the epilogue reads it (about 2 us per
// tile); the epilogue therefore only moves the tile into shared memory, 16-bit, and one TMA store writes it out.
//
// Work: a unit is one 128-k group of one output tile; cluster c takes a contiguous range of units, token tiles
// fastest so that neighbours share packed weights in L2.  Either ranges end on tile boundaries (whole tiles), or
// they are equal (stream-K) and a tile that a boundary cuts leaves as fp32 segments, which a second kernel adds in
// cluster order (results do not depend on timing) together with the bias.  The host picks whichever its cost model
// says ends first (make_plan).
//
//   warp 0        TMA producer of the activations: two boxes per unit into a ring of four stages.
//   warp 30       TMA producer of the packed weights (64-byte swizzle), scales and zero-points: a ring of three
//                 stages, freed as soon as the dequantisers have read them.
//   warp 1        MMA issuer (the leader CTA's): 8 tcgen05.mma per unit, software-pipelined (see there).
//   warps 2-17    dequantisers, two sets of 8 taking alternate units.  Warp (lane quarter q, k half h) takes the
//                 32 columns of chunk q for k-steps 4h..4h+3: ldmatrix.x2.trans gives a thread four nibbles of
//                 row k and of row k+1 per register (the k pairs of the operand layout); masks make 1024+q
//                 (1024+16q for the odd nibbles, 128+q in bf16), a subtract (or fma by 1/16) removes offset and
//                 zero-point exactly, a multiply applies the scale; tcgen05.st.16x128b.x2 puts them into 16 lanes
//                 of the A slot.
//   warps 18-29   epilogue: accumulator -> registers -> (+ bias, 16-bit) shared memory -> TMA store, or the fp32
//                 segment of a cut tile.
//
// Every wait is bounded; on expiry the kernel records NQB200_ERR_WAIT_TIMEOUT in the workspace status word, all
// roles drain, both CTAs meet at the closing cluster barrier, and tensor memory is released.  A wait on a phase
// parity is only right for a waiter that has seen the phase before it: see kWBars.
#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"
#include <mutex>

namespace nqb200 {
// One arrival on the barrier at this shared-memory offset in every CTA of `mask` (bit r: CTA r of the pair) when
// every MMA issued so far by this thread has completed.  `bar` is the executing CTA's own address.
__device__ __forceinline__ void umma_commit_pair_both(uint32_t bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}
namespace pair {

constexpr int kCols = 128, kUnitK = 128;
// Two rings of shared memory and one of tensor memory.  The packed weights of a unit (with scales and
// zero-points: 8.5 KB) are done with as soon as the dequantisers have read them, so they get a ring of
// their own (three stages: what the 64 KB staging tile of the epilogue leaves).  The unit's activations (up to 32 KB) must stay until its MMAs have
// completed, exactly as long as its slot of the A operand in tensor memory: those two rings have the same depth
// and one completion report frees both.  A unit's data is therefore requested while four units of tensor-core
// work are still queued, and the fetch of the weights, their dequantisation and the fetch of the activations
// overlap instead of following one another.
constexpr int kXStages = 4, kWStages = 3;
// A parity wait is only right if the waiter has seen the phase before: the two sets of dequantisers take
// alternate units, so with an odd number of weight stages a stage alternates between the sets.  The "landed"
// barriers are therefore counted per unit modulo twice the ring: each is then always waited on by the same set,
// phase after phase.
constexpr int kWBars = 2 * kWStages;
constexpr int kDequantWarps = 16, kEpiWarps = 12;
constexpr int kWProducerWarp = 2 + kDequantWarps + kEpiWarps;
constexpr int kThreads = (kWProducerWarp + 1) * 32;
constexpr int kXStageBytes = 32768, kWStageBytes = 8704, kOffSc = 8192, kOffZ = kOffSc + 256;
constexpr int kOffWRing = kXStages * kXStageBytes;
constexpr int kOffOut = kOffWRing + kWStages * kWStageBytes;   // the 16-bit output tile, [token][128 columns]
constexpr int kOutBytes = 256 * kCols * 2;
constexpr int kSmem = kOffOut + kOutBytes + 1024;
constexpr uint32_t kWStageTx = 8192 + 256 + 64;
constexpr int kColA = 0, kColD = 256, kTmemCols = 512;
constexpr int kFixThreads = 256;
constexpr int kSlotRows = 256;     // token rows of an fp32 slot (whatever the tile's token count), 256 columns each

struct Params {
  const void* bias; int bias_dtype; uint16_t* out;
  int M, N, G;
  int ntn, ntt;        // output tiles: column tiles of 128 x CTAs, token tiles of NT
  int NT, TH;          // tokens per tile (the MMA's N) and per CTA (NT / CTAs)
  int nclusters, quantum;   // quantum: 1 (stream-K) or G (a cluster takes whole tiles)
  uint32_t U;          // units: ntn * ntt * G
  float* slots; int slot_floats;  // [2 * nclusters][kSlotRows tokens][CTAs * 128 columns] fp32
  int* status;         // may be null
};

// A wait suspends in hardware for up to kSuspendNs at a time (woken at once when the phase completes), so the
// 31 warps that wait most of the time hardly issue; the limit is checked against the clock after each suspension.
constexpr uint32_t kSuspendNs = 20000;
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  const uint32_t b = smem_u32(bar);
  if (mbar_test_wait(b, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
    if (mbar_try_wait_suspend(b, parity, kSuspendNs)) return true;
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > kWaitLimitNs) {
      *abort_flag = 1;
      if (status) atomicExch(status, NQB200_ERR_WAIT_TIMEOUT);
      return false;
    }
  }
}

template <bool BF16> __device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
  uint32_t r;
  if (BF16) asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <bool BF16> __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  uint32_t r;
  if (BF16) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t fma2_f16(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// cluster c's units: [range_begin(c), range_begin(c + 1)), boundaries on multiples of q units (q = 1: stream-K;
// q = a tile's units: whole tiles only); 32-bit arithmetic (the host checks U * C < 2^31)
__host__ __device__ __forceinline__ uint32_t range_begin(uint32_t c, uint32_t U, uint32_t C, uint32_t q) {
  return c >= C ? U : ((c * (U / q)) / C) * q;
}
__host__ __device__ __forceinline__ int cluster_of_unit(uint32_t u, uint32_t U, uint32_t C) { return (int)(((u + 1) * C - 1) / U); }

// The column of the CTA's 128 that lane `l` of tensor memory holds (the order the dequantisers' stores give).
__device__ __forceinline__ int column_of_lane(int l) {
  const int q = l >> 5, ph = (l >> 4) & 1, r = (l >> 3) & 1, g = l & 7;
  return 32 * q + 8 * (g >> 1) + 4 * ph + 2 * r + (g & 1);
}

template <bool BF16, int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
umma_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_sc,
                    const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_x,
                    const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_slot, const Params p) {
  constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u;
  constexpr uint32_t MAGIC = BF16 ? 0x43004300u : 0x64006400u;  // 128.0 / 1024.0 in both halves
  constexpr uint32_t SIXTEENTH = 0x2C002C00u;                   // 1/16 in both halves (fp16)

  extern __shared__ uint8_t smem_raw[];
  // wfull / wfree: the weight ring (TMA landed / the set's 8 dequantiser warps have read it).
  // xfull: the activations landed.  afull: the A slot is filled and the CTA's activations have landed (of a
  // pair only the leader's is waited on: it collects both CTAs' arrivals, like "D empty").  done: the unit's
  // MMAs have completed: its activation stage and its A slot are free.
  __shared__ __align__(8) uint64_t bar_wfull[kWBars], bar_wfree[kWStages], bar_xfull[kXStages], bar_afull[kXStages],
      bar_done[kXStages], bar_dfull, bar_dempty, bar_drain, bar_ofull, bar_ofree;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort_i;

  volatile int* s_abort = &s_abort_i;
  int* status = p.status;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0u;
  const uint32_t cluster_id = blockIdx.x / CTAS;
  const int G = p.G;
  const uint32_t u_begin = range_begin(cluster_id, p.U, (uint32_t)p.nclusters, (uint32_t)p.quantum);
  const uint32_t u_end = range_begin(cluster_id + 1, p.U, (uint32_t)p.nclusters, (uint32_t)p.quantum);
  const int nunits = (int)(u_end - u_begin);

  grid_launch_dependents();
  grid_dependency_wait();  // the activations come from the kernel ahead on the stream

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWBars; ++s) mbar_init(smem_u32(&bar_wfull[s]), 1);
    for (int s = 0; s < kWStages; ++s) mbar_init(smem_u32(&bar_wfree[s]), kDequantWarps / 2);
    for (int s = 0; s < kXStages; ++s) {
      mbar_init(smem_u32(&bar_xfull[s]), 1); mbar_init(smem_u32(&bar_afull[s]), CTAS * kDequantWarps / 2); mbar_init(smem_u32(&bar_done[s]), 1);
    }
    mbar_init(smem_u32(&bar_dfull), 1);
    mbar_init(smem_u32(&bar_dempty), CTAS * kEpiWarps);
    mbar_init(smem_u32(&bar_drain), 1);
    mbar_init(smem_u32(&bar_ofull), kEpiWarps);
    mbar_init(smem_u32(&bar_ofree), 1);
    s_abort_i = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    if (CTAS == 2) { tmem_alloc_pair(smem_u32(&s_tmem), kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(&s_tmem), kTmemCols); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them from the other side
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  if (warp == 0) {
    // ------------------------------------------------- producer of the activations
    if (lane == 0) {
      prefetch_tmap(&tm_x);
      const uint32_t tx_bytes = 2u * (uint32_t)p.TH * 128u;
      int issued = 0;
      for (int i = 0; i < nunits; ++i) {
        const uint32_t u = u_begin + (uint32_t)i;
        const int item = (int)(u / (uint32_t)G), gk = (int)(u % (uint32_t)G);
        const int tok_row = (item % p.ntt) * p.NT + (int)rank * p.TH;   // this CTA's part of the token tile
        const int s = i % kXStages;
        if (i >= kXStages && !wait_bar(&bar_done[s], ((i / kXStages) - 1) & 1, s_abort, status)) break;
        const uint32_t st = smem_base + s * kXStageBytes, bar = smem_u32(&bar_xfull[s]);
        mbar_expect_tx(bar, tx_bytes);
        tma_load_2d(st, &tm_x, gk * kUnitK, tok_row, bar);
        tma_load_2d(st + p.TH * 128, &tm_x, gk * kUnitK + 64, tok_row, bar);
        ++issued;
      }
      // do not leave while a copy of ours may still be landing in this CTA's shared memory
      for (int j = issued > kXStages ? issued - kXStages : 0; j < issued; ++j)
        mbar_wait(smem_u32(&bar_xfull[j % kXStages]), (j / kXStages) & 1);
    }
  } else if (warp == kWProducerWarp) {
    // ----------------------------------- producer of the packed weights, scales and zero-points
    if (lane == 0) {
      prefetch_tmap(&tm_w); prefetch_tmap(&tm_sc); prefetch_tmap(&tm_z);
      int issued = 0;
      for (int i = 0; i < nunits; ++i) {
        const uint32_t u = u_begin + (uint32_t)i;
        const int item = (int)(u / (uint32_t)G), gk = (int)(u % (uint32_t)G);
        const int col_tile = (item / p.ntt) * CTAS + (int)rank;          // this CTA's 128 columns
        const int s = i % kWStages;
        if (i >= kWStages && !wait_bar(&bar_wfree[s], ((i / kWStages) - 1) & 1, s_abort, status)) break;
        const uint32_t st = smem_base + kOffWRing + s * kWStageBytes, bar = smem_u32(&bar_wfull[i % kWBars]);
        mbar_expect_tx(bar, kWStageTx);
        tma_load_2d(st, &tm_w, col_tile * 16, gk * kUnitK, bar);
        tma_load_2d(st + kOffSc, &tm_sc, col_tile * 64, gk, bar);
        tma_load_2d(st + kOffZ, &tm_z, col_tile * 16, gk, bar);
        ++issued;
      }
      for (int j = issued > kWStages ? issued - kWStages : 0; j < issued; ++j)
        mbar_wait(smem_u32(&bar_wfull[j % kWBars]), (j / kWBars) & 1);
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (of a pair: the leader's)
    // One thread, so every instruction here is on the critical path at several cycles each: counters instead
    // of divisions, the descriptor as a base plus precomputed offsets, one completion report per unit.
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(BF16 ? 1 : 0, 128 * CTAS, p.NT);
      const uint64_t desc0 = umma_smem_desc_sw128(smem_base);
      const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
      const uint32_t x1 = ((uint32_t)p.TH * 128u) >> 4;          // second activation box, in the descriptor's 16-byte units
      // The MMA queue is short (the tensor pipe ran dry during the 300 ns that this thread spent between two
      // units on waits, the completion report and loop bookkeeping), so the loop is software-pipelined: the
      // next unit's barrier is polled and the previous unit's completion is reported between MMAs of the
      // current unit, while MMAs are queued.  A report therefore also covers the next unit's first two
      // MMAs and frees its stage about 160 ns later than it could, which four stages absorb.
      uint32_t s = 0, phase = 0;
      int gk = (int)(u_begin % (uint32_t)G), li = 0, pending = -1;
      bool first = true;
      bool ok = nunits > 0 && wait_bar(&bar_afull[0], 0, s_abort, status);   // (both CTAs') A slot filled, activations landed
      const uint32_t d = tmem + kColD;
      auto mma = [&](uint32_t lo, uint32_t a, int ks, uint32_t acc) {
        const uint32_t dlo = lo + (ks >> 2) * x1 + (ks & 3) * 2;
        if (CTAS == 2) umma_ts_pair_lohi(d, a + ks * 8, dlo, desc_hi, idesc, acc);
        else umma_ts_lohi(d, a + ks * 8, dlo, desc_hi, idesc, acc);
      };
      auto report = [&](uint64_t* bar) {
        if (CTAS == 2) umma_commit_pair_both(smem_u32(bar), 3); else umma_commit(smem_u32(bar));
      };
      for (uint32_t u = u_begin; ok && u < u_end; ++u) {
        const bool last = gk == G - 1 || u == u_end - 1, more = u + 1 < u_end;
        tc_fence_after();
        const uint32_t lo = desc_lo0 + s * (uint32_t)(kXStageBytes >> 4);
        const uint32_t a = tmem + kColA + s * 64;
        mma(lo, a, 0, first ? 0u : 1u);
        mma(lo, a, 1, 1u);
        if (pending >= 0) { report(&bar_done[pending]); pending = -1; }
#pragma unroll
        for (int ks = 2; ks < 6; ++ks) mma(lo, a, ks, 1u);
        const uint32_t sn = s + 1 == kXStages ? 0u : s + 1, phn = s + 1 == kXStages ? phase ^ 1u : phase;
        const bool ready = more && !last && mbar_test_wait(smem_u32(&bar_afull[sn]), phn);
        mma(lo, a, 6, 1u);
        mma(lo, a, 7, 1u);
        if (last) {
          report(&bar_done[s]);
          report(&bar_dfull);
          ++li;
          if (more) ok = wait_bar(&bar_dempty, (li - 1) & 1, s_abort, status);   // the epilogues drained D
        } else {
          pending = (int)s;
        }
        if (more && !ready && ok) ok = wait_bar(&bar_afull[sn], phn, s_abort, status);
        first = last;
        if (++gk == G) gk = 0;
        s = sn; phase = phn;
      }
      if (pending >= 0) report(&bar_done[pending]);
      // everything issued has completed before tensor memory may be released
      if (CTAS == 2) umma_commit_pair(map_to_cta(smem_u32(&bar_drain), 0)); else umma_commit(smem_u32(&bar_drain));
      mbar_wait(smem_u32(&bar_drain), 0);
    }
  } else if (warp < 2 + kDequantWarps) {
    // -------------------------------------------------------------- dequantisers
    const int dw = warp - 2;
    const int q = warp & 3, h = (dw >> 2) & 1, set = dw >> 3;  // set: which units (even / odd) this warp serves
    const int g = lane >> 2, odd = g & 1;
    const uint32_t lane_base = tmem + ((uint32_t)(32 * q) << 16);
    const uint32_t afull_addr = CTAS == 2 ? map_to_cta(smem_u32(&bar_afull[0]), 0) : smem_u32(&bar_afull[0]);
    // ldmatrix: lanes 0-7 address rows k = 0..7 of a k-step, lanes 8-15 rows 8..15 (the others repeat them);
    // rows are 64 bytes, 16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3)
    const int lr = lane & 15;
    const uint32_t ld_row = (uint32_t)lr * 64u, ld_x = (uint32_t)((lr >> 1) & 3);
    for (int i = set; i < nunits; i += 2) {
      const int sw = i % kWStages, sa = i % kXStages;
      if (!wait_bar(&bar_wfull[i % kWBars], (i / kWBars) & 1, s_abort, status)) break;
      const uint32_t st = smem_base + kOffWRing + sw * kWStageBytes;
      // per column of this thread's four (2 pp + odd of word 4q + g/2): the scale, and what to remove, in both halves
      uint32_t sc2[4], zm2[4];
      {
        uint32_t swd[4], zw;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(swd[0]), "=r"(swd[1]), "=r"(swd[2]), "=r"(swd[3])
                     : "r"(st + kOffSc + (uint32_t)(4 * q + (g >> 1)) * 16u));
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zw) : "r"(st + kOffZ + (uint32_t)(4 * q + (g >> 1)) * 4u));
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          sc2[pp] = odd ? __byte_perm(swd[pp], 0, 0x3232) : __byte_perm(swd[pp], 0, 0x1010);
          const uint32_t z = (zw >> (4 * pp + 16 * odd)) & 0xFu;
          if (!BF16 && (pp & 1)) {
            // odd nibbles arrive as 1024 + 16 q: fma by 1/16 with -(64 + z) gives q - z exactly.
            // -(64 + z) in fp16: 0xD400 is -64, and integers 64..79 are steps of 1/16 of its binade: low mantissa bits z << 4
            const uint32_t hneg = 0xD400u | (z << 4);
            zm2[pp] = hneg | (hneg << 16);
          } else {
            zm2[pp] = (z | (z << 16)) | MAGIC;  // 1024 + z (128 + z): integers in the magic's binade are its low mantissa bits
          }
        }
      }
      // the A slot is free once the MMAs of the unit four before this one have completed
      if (i >= kXStages && !wait_bar(&bar_done[sa], ((i / kXStages) - 1) & 1, s_abort, status)) break;
      tc_fence_after();
      const uint32_t acol = lane_base + kColA + sa * 64;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int ks = 4 * h + kk;
        uint32_t R0, R1;
        // ((16 ks + lr) >> 1) & 3 == (lr >> 1) & 3
        ldmatrix_x2_trans(R0, R1, st + (uint32_t)ks * 1024u + ld_row + (((uint32_t)q ^ ld_x) << 4));
#pragma unroll
        for (int ph = 0; ph < 2; ++ph) {
          uint32_t a0, a1, a2, a3;
          if (BF16) {
            a0 = ((R0 >> (8 * ph)) & LO) | MAGIC; a1 = ((R0 >> (8 * ph + 4)) & LO) | MAGIC;
            a2 = ((R1 >> (8 * ph)) & LO) | MAGIC; a3 = ((R1 >> (8 * ph + 4)) & LO) | MAGIC;
            a0 = mul2<true>(sub2<true>(a0, zm2[2 * ph]), sc2[2 * ph]);
            a2 = mul2<true>(sub2<true>(a2, zm2[2 * ph]), sc2[2 * ph]);
            a1 = mul2<true>(sub2<true>(a1, zm2[2 * ph + 1]), sc2[2 * ph + 1]);
            a3 = mul2<true>(sub2<true>(a3, zm2[2 * ph + 1]), sc2[2 * ph + 1]);
          } else {
            const uint32_t l = R0 >> (8 * ph), hh = R1 >> (8 * ph);
            a0 = (l & LO) | MAGIC; a1 = (l & HI) | MAGIC; a2 = (hh & LO) | MAGIC; a3 = (hh & HI) | MAGIC;
            a0 = mul2<false>(sub2<false>(a0, zm2[2 * ph]), sc2[2 * ph]);
            a2 = mul2<false>(sub2<false>(a2, zm2[2 * ph]), sc2[2 * ph]);
            a1 = mul2<false>(fma2_f16(a1, SIXTEENTH, zm2[2 * ph + 1]), sc2[2 * ph + 1]);
            a3 = mul2<false>(fma2_f16(a3, SIXTEENTH, zm2[2 * ph + 1]), sc2[2 * ph + 1]);
          }
          tmem_st_16x128b_x2(acol + ((uint32_t)(16 * ph) << 16) + 8 * ks, a0, a1, a2, a3);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_wfree[sw]));   // this warp has read what it needs of the packed tile
      tc_wait_st();
      tc_fence_before();
      // this CTA's half of the activations must have landed too before the (leader's) issuer may go
      if (!wait_bar(&bar_xfull[sa], (i / kXStages) & 1, s_abort, status)) break;
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2) mbar_arrive_cluster(afull_addr + (uint32_t)sa * 8u);  // the leader's barrier, from either CTA
        else mbar_arrive(afull_addr + (uint32_t)sa * 8u);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3, sub = (warp - 2 - kDequantWarps) >> 2;
    const uint32_t lane_base = tmem + ((uint32_t)(32 * q) << 16);
    const int n_local = column_of_lane(32 * q + lane);
    const uint32_t dempty_addr = CTAS == 2 ? map_to_cta(smem_u32(&bar_dempty), 0) : smem_u32(&bar_dempty);
    int li = 0, ow = 0;                    // tiles read from D; tiles that went out through the staging area
    const int first_item = (int)(u_begin / (uint32_t)G);
    uint32_t u = u_begin;
    while (u < u_end) {
      // the segment of this item that the cluster covers: groups [g0, g1)
      const int item = (int)(u / (uint32_t)G), g0 = (int)(u % (uint32_t)G);
      const uint32_t item_end = (uint32_t)(item + 1) * (uint32_t)G;
      const uint32_t seg_end = item_end < u_end ? item_end : u_end;
      const int g1 = g0 + (int)(seg_end - u);
      u = seg_end;
      const int tn = item / p.ntt, tt = item % p.ntt;
      if (!wait_bar(&bar_dfull, li & 1, s_abort, status)) break;
      tc_fence_after();
      const bool whole = g0 == 0 && g1 == G;
      const int n = (tn * CTAS + (int)rank) * kCols + n_local;
      const bool n_ok = n < p.N;
      const int tok0 = tt * p.NT;
      const float bv = (whole && p.bias && n_ok) ? bias_to_float(p.bias, p.bias_dtype, n) : 0.f;
      if (whole) {
        // The tile leaves through shared memory: [token][column] in 16 bits, written by one TMA store that clips
        // at M and N.  The accumulator is handed back as soon as it has been read.
        if (ow > 0 && !wait_bar(&bar_ofree, (ow - 1) & 1, s_abort, status)) break;   // the previous store has read the staging area
        uint8_t* stage = smem_raw + (smem_base - smem_u32(smem_raw)) + kOffOut + n_local * 2;
        // The accumulator is handed back right after the last read, before the last values are converted:
        // the tensor pipe idles from the tile's last MMA until then.
        constexpr int kStep = 16 * (kEpiWarps / 4);
        bool handed_back = false;
        for (int c0 = 16 * sub; c0 < p.NT; c0 += kStep) {
          uint32_t d[16];
          tmem_ld_32x32b_x16(lane_base + kColD + c0, d);
          tc_wait_ld();
          if (c0 + kStep >= p.NT) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (CTAS == 2) mbar_arrive_cluster(dempty_addr); else mbar_arrive(dempty_addr);
            }
            handed_back = true;
          }
#pragma unroll
          for (int c = 0; c < 16; ++c)
            *reinterpret_cast<uint16_t*>(stage + (c0 + c) * (kCols * 2)) = float_to_raw16<BF16>(__uint_as_float(d[c]) + bv);
        }
        if (!handed_back) {   // (a tile of so few tokens that this warp had none)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CTAS == 2) mbar_arrive_cluster(dempty_addr); else mbar_arrive(dempty_addr);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the writes, before the TMA engine reads them
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_ofull));
        if (warp == 2 + kDequantWarps && lane == 0) {
          if (!wait_bar(&bar_ofull, ow & 1, s_abort, status)) break;
          const int col0 = (tn * CTAS + (int)rank) * kCols;
          if (col0 < p.N) {   // (the second CTA's columns may all lie beyond N)
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                         ::"l"(&tm_out), "r"(col0), "r"(tok0), "r"(smem_base + kOffOut) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          mbar_arrive(smem_u32(&bar_ofree));
        }
        __syncwarp();
        ++ow;
      } else {
        // A segment of a tile that another cluster shares: fp32 to this cluster's slot, [token][column], in two
        // halves of 128 tokens through the same staging area (64 KB hold 128 x 128 fp32), one TMA store each.
        constexpr int kStep = 16 * (kEpiWarps / 4);
        const int slot_row = ((int)cluster_id * 2 + (item == first_item ? 0 : 1)) * kSlotRows;
        uint8_t* stage = smem_raw + (smem_base - smem_u32(smem_raw)) + kOffOut + n_local * 4;
        bool handed_back = false, gave_up = false;
        for (int h = 0; 128 * h < p.NT && !gave_up; ++h) {
          if (ow > 0 && !wait_bar(&bar_ofree, (ow - 1) & 1, s_abort, status)) { gave_up = true; break; }
          const int t_lo = 128 * h, t_hi = min(t_lo + 128, p.NT);
          for (int c0 = 16 * sub; c0 < t_hi; c0 += kStep) {
            if (c0 < t_lo) continue;
            uint32_t d[16];
            tmem_ld_32x32b_x16(lane_base + kColD + c0, d);
            tc_wait_ld();
            if (c0 + kStep >= p.NT) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                if (CTAS == 2) mbar_arrive_cluster(dempty_addr); else mbar_arrive(dempty_addr);
              }
              handed_back = true;
            }
#pragma unroll
            for (int c = 0; c < 16; ++c) *reinterpret_cast<uint32_t*>(stage + (c0 - t_lo + c) * (kCols * 4)) = d[c];
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_ofull));
          if (warp == 2 + kDequantWarps && lane == 0) {
            if (wait_bar(&bar_ofull, ow & 1, s_abort, status)) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&tm_slot), "r"((int)rank * kCols), "r"(slot_row + t_lo), "r"(smem_base + kOffOut) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
              mbar_arrive(smem_u32(&bar_ofree));
            }
          }
          __syncwarp();
          ++ow;
        }
        if (gave_up) break;
        if (!handed_back) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CTAS == 2) mbar_arrive_cluster(dempty_addr); else mbar_arrive(dempty_addr);
          }
        }
      }
      ++li;
    }
  }

  // All roles (of both CTAs) meet here, also after a give-up: neither CTA may leave while the other can
  // still read its shared or tensor memory or arrive on its barriers; then tensor memory is released.
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (CTAS == 2) tmem_dealloc_pair(tmem, kTmemCols); else tmem_dealloc(tmem, kTmemCols);
  }
}

// Adds, for every output tile that more than one cluster worked on, the clusters' fp32 segments in
// cluster order, adds the bias and writes out[tok, n].  A tile is shared exactly where a boundary between
// two clusters' ranges falls inside it, so blockIdx.x runs over the boundaries (cluster c = blockIdx.x + 1
// against c - 1) and the first boundary inside a tile owns it; blockIdx.y runs over the tile's blocks of
// 32 tokens x 32 columns.  Slots and output are both [token][column]: a warp reads and writes rows of 32.
template <bool BF16>
__global__ void __launch_bounds__(kFixThreads) pair_fixup_kernel(const Params p, const int ctas) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int G = p.G;
  const uint32_t U = p.U, C = (uint32_t)p.nclusters;
  const uint32_t c = blockIdx.x + 1, b = range_begin(c, U, C, 1u);
  if (b % (uint32_t)G == 0) return;                       // the boundary falls between two tiles
  const int item = (int)(b / (uint32_t)G);
  const int first_c = cluster_of_unit((uint32_t)item * G, U, C);
  if (first_c != (int)c - 1) return;                       // an earlier boundary inside this tile owns it
  const int nc = cluster_of_unit((uint32_t)item * G + G - 1, U, C) - first_c + 1;
  const int first_slot = 2 * first_c + ((int)(range_begin(first_c, U, C, 1u) / (uint32_t)G) == item ? 0 : 1);
  const int tn = item / p.ntt, tt = item % p.ntt;
  const int cols = kCols * ctas;
  const int tblocks = (p.NT + 31) / 32;
  const int n0 = 32 * ((int)blockIdx.y / tblocks), t0 = 32 * ((int)blockIdx.y % tblocks);
  const int tx = (int)threadIdx.x & 31, ty = (int)threadIdx.x >> 5;  // 8 rows of 32 threads
  const int n = tn * cols + n0 + tx;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < nc; ++k) {
    const float* src = p.slots + (size_t)(k == 0 ? first_slot : 2 * (first_c + k)) * p.slot_floats + n0 + tx;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = t0 + ty + 8 * j;
      if (row < p.NT) v[j] += __ldcg(src + (size_t)row * cols);
    }
  }
  const float bv = (p.bias && n < p.N) ? bias_to_float(p.bias, p.bias_dtype, n) : 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int row = t0 + ty + 8 * j, tok = tt * p.NT + row;
    if (row < p.NT && tok < p.M && n < p.N) p.out[(size_t)tok * p.N + n] = float_to_raw16<BF16>(v[j] + bv);
  }
}

// The shape of the work for a problem: CTAs per cluster, tokens per tile, clusters, units.
struct Plan { int ctas, NT, TH, ntn, ntt, nclusters, quantum; long long U; double est_us; bool fixup; size_t slot_floats; };
static Plan make_plan(int64_t M, int64_t N, int64_t K) {
  Plan pl;
  pl.ctas = 2;
  const int64_t cap = 128 * pl.ctas, unit = 16 * pl.ctas;   // each CTA's share is a multiple of 16 tokens
  pl.NT = (int)(M >= cap ? cap : (M + unit - 1) / unit * unit);
  pl.TH = pl.NT / pl.ctas;
  pl.ntn = (int)((N + kCols * pl.ctas - 1) / (kCols * pl.ctas));
  pl.ntt = (int)((M + pl.NT - 1) / pl.NT);
  const int G = (int)(K / 128);
  pl.U = (long long)pl.ntn * pl.ntt * G;
  const long long maxc = kNumSMs / pl.ctas, items = (long long)pl.ntn * pl.ntt;
  // Stream-K keeps every cluster busy to the end, but the tiles that a range boundary cuts go through fp32 slots
  // and a second kernel, and the clusters drift apart in k, so that the activations (which all column tiles of a
  // token tile share) are fetched from L2 at scattered times: measured 0.95 us per unit + 10 us.  Whole tiles keep
  // the clusters in step (0.78 us per unit in a full wave) and lose only the last wave's idle clusters, which
  // itself runs faster the emptier it is (0.6 to 0.8 us per unit).  Fitted on M in 192..4096 x the sweep's five
  // shapes, where it picks the faster dealing every time.  Whichever ends first:
  const long long full = items / maxc, rem = items % maxc;
  const double t_whole = G * (0.78 * (double)full + (rem ? 0.6 + 0.2 * (double)rem / (double)maxc : 0.0));
  const double t_stream = 0.95 * (double)((pl.U + maxc - 1) / maxc) + 10.0;
  const bool whole = t_whole <= t_stream;
  pl.quantum = whole ? G : 1;
  pl.est_us = whole ? t_whole : t_stream;
  const long long parts = whole ? items : pl.U;
  pl.nclusters = (int)(parts < maxc ? parts : maxc);
  // some tile is shared between clusters unless every range boundary falls on a tile boundary
  pl.fixup = false;
  if (!whole && (pl.U + 1) * pl.nclusters < (1ll << 31))
    for (int c = 1; c < pl.nclusters && !pl.fixup; ++c)
      if (range_begin((uint32_t)c, (uint32_t)pl.U, (uint32_t)pl.nclusters, 1u) % (uint32_t)G != 0) pl.fixup = true;
  pl.slot_floats = (size_t)kCols * pl.ctas * kSlotRows;
  return pl;
}

template <typename Kern>
static int launch_main(Kern kern, int ctas_per_cluster, int grid, cudaStream_t st, const CUtensorMap& tw, const CUtensorMap& ts,
                       const CUtensorMap& tz, const CUtensorMap& tx, const CUtensorMap& to, const CUtensorMap& tsl, const Params& sp) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmem; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = ctas_per_cluster; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, kern, tw, ts, tz, tx, to, tsl, sp) != cudaSuccess) { cudaGetLastError(); return NQB200_ERR_LAUNCH; }
  return NQB200_OK;
}

template <bool BF16>
static int launch_t(const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tz, const CUtensorMap& tx, const CUtensorMap& to,
                    const CUtensorMap& tsl, const Params& sp, const Plan& pl, cudaStream_t st) {
  // The shared-memory attribute belongs to the device that is current when it is set: one flag per device.
  static std::mutex mu;
  static bool configured[kMaxDevices] = {false};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return NQB200_ERR_UNSUPPORTED_DEVICE; }
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!configured[dev]) {
      if (cudaFuncSetAttribute(umma_pair_kernel<BF16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) {
        cudaGetLastError();
        return NQB200_ERR_LAUNCH;
      }
      configured[dev] = true;
    }
  }
  const int grid = pl.nclusters * pl.ctas;
  const int rc = launch_main(umma_pair_kernel<BF16, 2>, 2, grid, st, tw, ts, tz, tx, to, tsl, sp);
  if (rc != NQB200_OK || !pl.fixup) return rc;
  const int blocks_per_tile = (kCols * pl.ctas / 32) * ((pl.NT + 31) / 32);
  return launch_overlapped(pair_fixup_kernel<BF16>, dim3(pl.nclusters - 1, blocks_per_tile), dim3(kFixThreads), 0, st, sp, pl.ctas);
}

}  // namespace pair

bool umma_pair_supports(int64_t M, int64_t N, int64_t K, int64_t g) {
  if (!(M > 128 && g == 128 && K % 128 == 0 && N % 32 == 0)) return false;
  // Against the single-CTA kernel: its own cost model's estimate for the shape, less the 10 us by which this
  // kernel's fixed cost (cluster launch, tensor-memory allocation for a pair, a deeper pipeline to fill) exceeds
  // that kernel's.  Over M in 192..4096 x the sweep's five shapes this rule picks the faster kernel every time.
  const pair::Plan pl = pair::make_plan(M, N, K);
  if ((pl.U + 1) * pl.nclusters >= (1ll << 31)) return false;   // the kernel's 32-bit unit arithmetic
  return pl.est_us <= umma_prefill_estimate_us(M, N, K) - 10.0;
}

int umma_pair_launches(int64_t M, int64_t N, int64_t K) { return pair::make_plan(M, N, K).fixup ? 2 : 1; }

size_t umma_pair_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const pair::Plan pl = pair::make_plan(M, N, K);
  return (size_t)kCounterBytes + (pl.fixup ? (size_t)2 * pl.nclusters * pl.slot_floats * sizeof(float) : 0);
}

int launch_umma_pair(const GemmArgs& a) {
  using namespace pair;
  const int G = a.K / 128;
  const Plan pl = make_plan(a.M, a.N, a.K);
  if ((pl.U + 1) * pl.nclusters >= (1ll << 31)) return NQB200_ERR_TOO_LARGE;
  Params sp;
  sp.bias = a.bias; sp.bias_dtype = a.bias_dtype; sp.out = (uint16_t*)a.out;
  sp.M = a.M; sp.N = a.N; sp.G = G;
  sp.ntn = pl.ntn; sp.ntt = pl.ntt; sp.NT = pl.NT; sp.TH = pl.TH;
  sp.nclusters = pl.nclusters; sp.quantum = pl.quantum; sp.U = (uint32_t)pl.U;
  sp.status = (a.ws && a.ws_bytes >= (size_t)kCounterBytes) ? (int*)a.ws + (kCounterBytes / 4 - 1) : nullptr;
  sp.slots = nullptr; sp.slot_floats = (int)pl.slot_floats;
  if (pl.fixup) {
    if (!a.ws || a.ws_bytes < umma_pair_workspace_bytes(a.M, a.N, a.K)) return NQB200_ERR_WORKSPACE;
    if (!aligned16(a.ws)) return NQB200_ERR_MISALIGNED;
    sp.slots = (float*)((char*)a.ws + kCounterBytes);
  }
  alignas(64) CUtensorMap tw, ts, tz, tx, to, tsl;
  const CUtensorMapDataType xdt = a.dtype == NQB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  bool ok = encode_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qw, a.K, a.N / 8, 128, 16, CU_TENSOR_MAP_SWIZZLE_64B);
  ok = ok && encode_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.sc, G, a.N / 2, 1, 64, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tz, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qz, G, a.N / 8, 1, 16, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tx, xdt, 2, a.x, a.M, a.K, (uint32_t)pl.TH, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && encode_2d(&to, xdt, 2, a.out, a.M, a.N, (uint32_t)pl.NT, kCols, CU_TENSOR_MAP_SWIZZLE_NONE);
  // the fp32 slots as one matrix of [2 * clusters * kSlotRows][256]; without stream-K segments the map is never used
  if (pl.fixup) ok = ok && encode_2d(&tsl, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, sp.slots, (uint64_t)2 * pl.nclusters * kSlotRows,
                                     kCols * pl.ctas, 128, kCols, CU_TENSOR_MAP_SWIZZLE_NONE);
  else tsl = to;
  if (!ok) return NQB200_ERR_LAUNCH;
  return a.dtype == NQB200_BF16 ? launch_t<true>(tw, ts, tz, tx, to, tsl, sp, pl, a.stream)
                                : launch_t<false>(tw, ts, tz, tx, to, tsl, sp, pl, a.stream);
}

}  // namespace nqb200
