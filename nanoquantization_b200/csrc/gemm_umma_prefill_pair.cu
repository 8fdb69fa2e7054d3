// Prefill kernel for large token counts on CTA pairs (tcgen05 cta_group::2).
//
// The single-CTA prefill kernel is bound by L2 -> shared-memory traffic: for
// every 256-column weight tile it re-reads a 128-token activation tile (32 KB
// per group of 128 k against 16 KB of packed weights).  Here two CTAs of a
// cluster, on the two SMs of a TPC, work as one: each dequantises its own 256
// weight columns into its own tensor memory, each loads only half of the
// activation tile (64 tokens) into its own shared memory, and one
// tcgen05.mma.cta_group::2 (M = 256: 128 rows from each CTA; N = 128 tokens, 64
// rows of B from each CTA) feeds both.  Per CTA and group that is 16 KB of
// weights plus 16 KB of activations instead of 16 + 32.
//
// Roles per CTA are those of the single-CTA kernel (TMA producer, 16
// dequantiser warps in two sets, epilogue warps); the MMAs of the pair are
// issued by the leader (cluster rank 0).  Hand-offs that cross the pair:
//   * the dequantisers of both CTAs arrive on the leader's "A full" barrier (the
//     follower's through its shared::cluster address) -- having waited for their
//     own TMA stage first, so the arrival also covers the activation half;
//   * the leader commits every completion to the barrier of each CTA in turn
//     (plain tcgen05.commit on a shared::cluster address; no multicast form);
//   * the epilogue warps of both CTAs arrive on the leader's "D empty" barrier.
// Every wait is bounded; the cluster barrier at the end is reached by every
// thread also after a give-up, and tensor memory is released after it.
#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"

namespace nqb200 {
namespace pre2 {

constexpr int kTileN = 256, kTileT = 128, kUnitK = 128;
constexpr int kStages = 6, kAStages = 2;
constexpr int kDequantWarps = 16, kEpiWarps = 12;  // three epilogue warps per lane quarter share a tile's token columns
constexpr int kThreads = (2 + kDequantWarps + kEpiWarps) * 32;
constexpr int kOffW = 0, kOffX0 = 16384, kOffX1 = 24576, kOffSc = 32768, kOffZ = 33280, kStageBytes = 33792;
constexpr int kSmem = kStages * kStageBytes + 1024;
constexpr uint32_t kStageTx = 16384 + 2 * 8192 + 512 + 128;
constexpr int kColA = 0, kColD = 256, kTmemCols = 512;

struct Params {
  const void* bias; int bias_dtype; uint16_t* out;
  int M, N, G, npairs_n, ntiles_t;  // npairs_n: pairs of adjacent 256-column tiles
  int* status;                       // may be null
};

// `sleep_ns` > 0: back off between polls (roles that wait long should not take issue slots).
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                         unsigned sleep_ns = 0) {
  const uint32_t b = smem_u32(bar);
  if (mbar_try_wait(b, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(b, parity)) return true;
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((i & 63u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (status) atomicExch(status, NQB200_ERR_WAIT_TIMEOUT);
        return false;
      }
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

template <bool BF16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
umma_prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_sc,
                         const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_x, const Params p) {
  constexpr uint32_t LO = 0x000F000Fu;
  constexpr uint32_t MAGIC = BF16 ? 0x43004300u : 0x64006400u;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages], bar_empty[kStages], bar_afull[kAStages], bar_aempty[kAStages],
      bar_dfull, bar_dempty, bar_drain;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort_i;

  volatile int* s_abort = &s_abort_i;
  int* status = p.status;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
  const int G = p.G;
  const int nitems = p.npairs_n * p.ntiles_t;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), kDequantWarps / 2 + 1); }
    // only the leader's copies of these two are waited on: they collect arrivals from both CTAs
    for (int s = 0; s < kAStages; ++s) { mbar_init(smem_u32(&bar_afull[s]), kDequantWarps); mbar_init(smem_u32(&bar_aempty[s]), 1); }
    mbar_init(smem_u32(&bar_dfull), 1);
    mbar_init(smem_u32(&bar_dempty), 2 * kEpiWarps);
    mbar_init(smem_u32(&bar_drain), 1);
    s_abort_i = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc_pair(smem_u32(&s_tmem), kTmemCols); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them from the other side
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  int my_items = 0;
  for (int w = cluster_id; w < nitems; w += nclusters) ++my_items;
  const int nunits = my_items * G;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tm_w); prefetch_tmap(&tm_sc); prefetch_tmap(&tm_z); prefetch_tmap(&tm_x);
      int issued = 0, i = 0;
      bool ok = true;
      for (int w = cluster_id; w < nitems && ok; w += nclusters) {
        const int tile_n = 2 * (w / p.ntiles_t) + (int)rank, tile_t = w % p.ntiles_t;
        const int tok_row = tile_t * kTileT + 64 * (int)rank;  // this CTA's half of the token tile
        for (int grp = 0; grp < G; ++grp, ++i) {
          const int s = i % kStages;
          if (i >= kStages && !wait_bar(&bar_empty[s], ((i / kStages) - 1) & 1, s_abort, status)) { ok = false; break; }
          const uint32_t st = smem_base + s * kStageBytes, bar = smem_u32(&bar_full[s]);
          mbar_expect_tx(bar, kStageTx);
          tma_load_2d(st + kOffW, &tm_w, tile_n * 32, grp * kUnitK, bar);
          tma_load_2d(st + kOffX0, &tm_x, grp * kUnitK, tok_row, bar);
          tma_load_2d(st + kOffX1, &tm_x, grp * kUnitK + 64, tok_row, bar);
          tma_load_2d(st + kOffSc, &tm_sc, tile_n * 128, grp, bar);
          tma_load_2d(st + kOffZ, &tm_z, tile_n * 32, grp, bar);
          ++issued;
        }
      }
      for (int j = issued > kStages ? issued - kStages : 0; j < issued; ++j)
        mbar_wait(smem_u32(&bar_full[j % kStages]), (j / kStages) & 1);
    }
  } else if (warp == 1) {
    // ------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(BF16 ? 1 : 0, 256, kTileT);
      for (int i = 0; i < nunits; ++i) {
        const int s = i % kStages, sa = i % kAStages;
        const int grp = i % G, lt = i / G;
        if (grp == 0 && lt > 0 && !wait_bar(&bar_dempty, (lt - 1) & 1, s_abort, status)) break;  // both epilogues drained D
        if (!wait_bar(&bar_full[s], (i / kStages) & 1, s_abort, status)) break;
        if (!wait_bar(&bar_afull[sa], (i / kAStages) & 1, s_abort, status)) break;              // both CTAs' A and activations
        tc_fence_after();
        const uint32_t xaddr = smem_base + s * kStageBytes + kOffX0;
        const uint32_t a0 = tmem + kColA + sa * 128, a1 = a0 + 64, d = tmem + kColD;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t bdesc = umma_smem_desc_sw128(xaddr + (ks >> 2) * 8192 + (ks & 3) * 32);
          const uint32_t acc = (grp > 0 || ks > 0) ? 1u : 0u;
          umma_ts_pair(d, a0 + ks * 8, bdesc, idesc, acc);
          umma_ts_pair(d + 128, a1 + ks * 8, bdesc, idesc, acc);
        }
        // completion is reported to each CTA's own barrier
#pragma unroll
        for (uint32_t r = 0; r < 2; ++r) {
          umma_commit_pair(map_to_cta(smem_u32(&bar_aempty[sa]), r));
          umma_commit_pair(map_to_cta(smem_u32(&bar_empty[s]), r));
          if (grp == G - 1) umma_commit_pair(map_to_cta(smem_u32(&bar_dfull), r));
        }
      }
      umma_commit_pair(map_to_cta(smem_u32(&bar_drain), 0));
      mbar_wait(smem_u32(&bar_drain), 0);
    }
  } else if (warp < 2 + kDequantWarps) {
    // -------------------------------------------------------------- dequantisers
    const int dw = warp - 2;
    const int q = warp & 3, h = (dw >> 2) & 1, set = dw >> 3;
    const int gq = lane >> 2, tig = lane & 3;
    const int chunk = 2 * q + (gq >> 2), inword = (gq & 3) * 4;
    const uint32_t sw_even = ((uint32_t)(chunk ^ ((2 * tig) & 7)) << 4) + inword;
    const uint32_t sw_odd = ((uint32_t)(chunk ^ ((2 * tig + 1) & 7)) << 4) + inword;
    const uint32_t row0 = (uint32_t)(2 * tig) * 128;
    const uint32_t lane_base = tmem + ((uint32_t)(32 * q) << 16);
    for (int i = set; i < nunits; i += 2) {
      const int s = i % kStages, sa = i % kAStages;
      if (!wait_bar(&bar_full[s], (i / kStages) & 1, s_abort, status)) break;
      const uint8_t* st = smem_gen + s * kStageBytes;
      uint32_t sc2[8], zm2[8];
      {
        const uint4 sv = lds128(st, kOffSc + (uint32_t)(64 * q + 8 * gq) * 2);
        const uint32_t zw = lds32(st, kOffZ + (uint32_t)(8 * q + gq) * 4);
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int e = (j < 4) ? 2 * j : 2 * (j - 4) + 1;
          sc2[j] = (e & 1) ? __byte_perm(sw[e >> 1], 0, 0x3232) : __byte_perm(sw[e >> 1], 0, 0x1010);
          const uint32_t z = (zw >> (4 * j)) & 0xFu;
          zm2[j] = (z | (z << 16)) | MAGIC;
        }
      }
      // the leader's commit frees the slot in both CTAs; each CTA waits on its own copy
      if (i >= kAStages && !wait_bar(&bar_aempty[sa], ((i / kAStages) - 1) & 1, s_abort, status)) break;
      tc_fence_after();
      const uint8_t* wb = st + kOffW + row0;
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
          uint32_t a0 = (p01 & LO) | MAGIC, a1 = ((p01 >> 4) & LO) | MAGIC;
          uint32_t a2 = (p23 & LO) | MAGIC, a3 = ((p23 >> 4) & LO) | MAGIC;
          a0 = mul2<BF16>(sub2<BF16>(a0, zm2[2 * b]), sc2[2 * b]);
          a2 = mul2<BF16>(sub2<BF16>(a2, zm2[2 * b]), sc2[2 * b]);
          a1 = mul2<BF16>(sub2<BF16>(a1, zm2[2 * b + 1]), sc2[2 * b + 1]);
          a3 = mul2<BF16>(sub2<BF16>(a3, zm2[2 * b + 1]), sc2[2 * b + 1]);
          tmem_st_16x128b_x2(acol + ((uint32_t)(16 * (b & 1)) << 16) + 64 * (b >> 1) + 8 * ks, a0, a1, a2, a3);
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(map_to_cta(smem_u32(&bar_afull[sa]), 0));  // the leader's barrier, from either CTA
        mbar_arrive(smem_u32(&bar_empty[s]));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3, sub = (warp - 2 - kDequantWarps) >> 2;
    const uint32_t lane_base = tmem + ((uint32_t)(32 * q) << 16);
    const int g = lane & 7, r = (lane >> 3) & 1, bb = lane >> 4;
    int nloc[2];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const int j = 2 * (2 * blk + bb) + r;
      nloc[blk] = 64 * q + 8 * g + ((j < 4) ? 2 * j : 2 * (j - 4) + 1);
    }
    int lt = 0;
    for (int w = cluster_id; w < nitems; w += nclusters, ++lt) {
      const int tile_n = 2 * (w / p.ntiles_t) + (int)rank, tile_t = w % p.ntiles_t;
      if (!wait_bar(&bar_dfull, lt & 1, s_abort, status, 200)) break;
      tc_fence_after();
      const int tok0 = tile_t * kTileT;
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        const int n = tile_n * kTileN + nloc[blk];
        const bool n_ok = n < p.N;
        const float bv = (p.bias && n_ok) ? bias_to_float(p.bias, p.bias_dtype, n) : 0.f;
        for (int c0 = 16 * sub; c0 < kTileT; c0 += 16 * (kEpiWarps / 4)) {
          uint32_t d[16];
          tmem_ld_32x32b_x16(lane_base + kColD + 128 * blk + c0, d);
          tc_wait_ld();
          if (!n_ok) continue;
          const int tok = tok0 + c0;
          const int ntok = min(16, p.M - tok);
          uint16_t* dst = p.out + (size_t)tok * p.N + n;
#pragma unroll
          for (int c = 0; c < 16; ++c)
            if (c < ntok) dst[(size_t)c * p.N] = float_to_raw16<BF16>(__uint_as_float(d[c]) + bv);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_dempty), 0));
    }
  }

  // Every thread of both CTAs meets here, also after a give-up: neither CTA may leave while the
  // other can still read its shared or tensor memory or arrive on its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc_pair(tmem, kTmemCols); }
}

template <bool BF16>
static int launch_t(const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tz, const CUtensorMap& tx,
                    const Params& sp, int ctas, cudaStream_t st) {
  static bool configured = false;  // idempotent attribute; a repeated set from two threads is harmless
  if (!configured) {
    if (cudaFuncSetAttribute(umma_prefill_pair_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) {
      cudaGetLastError();
      return NQB200_ERR_LAUNCH;
    }
    configured = true;
  }
  umma_prefill_pair_kernel<BF16><<<ctas, kThreads, kSmem, st>>>(tw, ts, tz, tx, sp);
  return check_launch();
}

}  // namespace pre2

// Worth it once there are enough (512 columns x 128 tokens) items to keep every CTA pair busy.
bool umma_prefill_pair_supports(int64_t M, int64_t N, int64_t K, int64_t g) {
  if (!(M >= 128 && g == 128 && K % 128 == 0 && N % 32 == 0)) return false;
  const long long items = ((N + 511) / 512) * ((M + 127) / 128);
  return items >= kNumSMs / 2;
}

int launch_umma_prefill_pair(const GemmArgs& a) {
  using namespace pre2;
  const int G = a.K / 128;
  Params sp;
  sp.bias = a.bias; sp.bias_dtype = a.bias_dtype; sp.out = (uint16_t*)a.out;
  sp.M = a.M; sp.N = a.N; sp.G = G;
  sp.npairs_n = (a.N + 2 * kTileN - 1) / (2 * kTileN);
  sp.ntiles_t = (a.M + kTileT - 1) / kTileT;
  sp.status = (a.ws && a.ws_bytes >= (size_t)kCounterBytes) ? (int*)a.ws + (kCounterBytes / 4 - 1) : nullptr;
  const long long items = (long long)sp.npairs_n * sp.ntiles_t;
  const int clusters = (int)(items < kNumSMs / 2 ? items : kNumSMs / 2);
  alignas(64) CUtensorMap tw, ts, tz, tx;
  const CUtensorMapDataType xdt = a.dtype == NQB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  bool ok = encode_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qw, a.K, a.N / 8, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && encode_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.sc, G, a.N / 2, 1, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tz, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qz, G, a.N / 8, 1, 32, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tx, xdt, 2, a.x, a.M, a.K, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return NQB200_ERR_LAUNCH;
  return a.dtype == NQB200_BF16 ? launch_t<true>(tw, ts, tz, tx, sp, 2 * clusters, a.stream)
                                : launch_t<false>(tw, ts, tz, tx, sp, 2 * clusters, a.stream);
}

}  // namespace nqb200
