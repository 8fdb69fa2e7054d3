// Prefill kernel on the 5th-generation tensor cores: W4A16 GEMM for more than
// 16 tokens, group size 128, bound by the tensor pipe (and, below a few hundred
// tokens, by HBM).
//
//   D[n, tok] (TMEM, fp32) = sum_k W[k, n] (TMEM, 16-bit) * x[tok, k] (smem)
//
// The weights are the 128-row A operand, dequantised to their true 16-bit
// values (q - z) * s -- the integer difference first, then one multiply, which
// is the reference's rounding -- straight from registers into tensor memory;
// the tokens are the N dimension (up to 128 per tile), read from shared memory
// as a K-major operand that TMA wrote with the 128-byte swizzle.  A packed word
// never touches shared memory again after the TMA load, and a dequantised
// value never touches shared memory at all.
//
// Persistent CTAs, one per SM, walk output tiles of 256 weight columns x 128
// tokens (token tiles of one column tile go to neighbouring CTAs so that they
// share the packed weights in L2).  Per tile, for each group of 128 k:
//
//   warp 0        TMA producer: 128 x 128 B of packed weights, two 128 x 64
//                 boxes of activations, the group's scales and zero-points.
//   warps 2-17    dequantisers, two sets of 8 taking alternate groups.  Warp
//                 (quarter q, half h) turns words 8q..8q+7 of k-steps 4h..4h+3
//                 into operand registers: PRMT pairs byte b of rows k and k+1,
//                 LOP3 makes 1024+q (fp16) or 128+q (bf16), HSUB2 removes
//                 1024+z, HMUL2 applies the scale; tcgen05.st.16x128b.x2 puts
//                 byte b into lanes 16*(b&1).. of its lane quarter of A block
//                 b>>1.
//   warps 1, 30   MMA issuers, one per A block: per k-step one tcgen05.mma (M=128,
//                 N=tokens, K=16), accumulating over all of K in tensor memory.
//                 Issuing costs the thread about 100 cycles per MMA whatever its
//                 size (measured with in-kernel timestamps), so a single issuer
//                 caps the tensor pipe near 60 % at N=128; two issuers on
//                 disjoint accumulators lift that.
//   warps 18-21   epilogue at the end of a tile: D -> registers -> bias ->
//                 16-bit -> out[tok, n].
//
// Every wait is bounded; on expiry the kernel records NQB200_ERR_WAIT_TIMEOUT in
// the workspace status word (when a workspace is given), all roles drain, and
// tensor memory is released.
#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"
#include <mutex>

namespace nqb200 {
namespace pre {

constexpr int kTileN = 256, kTileT = 128, kUnitK = 128;
constexpr int kStages = 4, kAStages = 2;
constexpr int kDequantWarps = 16, kEpiWarps = 12;  // three epilogue warps per lane quarter share a tile's token columns
constexpr int kThreads = (2 + kDequantWarps + kEpiWarps + 1) * 32;  // + a second MMA issuer
constexpr int kMmaWarpB = 2 + kDequantWarps + kEpiWarps;
constexpr int kOffW = 0, kOffX0 = 16384, kOffX1 = 32768, kOffSc = 49152, kOffZ = 49664, kStageBytes = 50176;
constexpr int kSmem = kStages * kStageBytes + 1024;
constexpr uint32_t kStageTx = 16384 + 2 * 16384 + 512 + 128;
constexpr int kColA = 0, kColD = 256, kTmemCols = 512;

struct Params {
  const void* bias; int bias_dtype; uint16_t* out;
  int M, N, G, ntiles_n, ntiles_t, nt;  // nt: MMA N (tokens per tile rounded up to 16)
  int ksplit;                           // CTAs along K per output tile (1: results go straight to `out`)
  float* partials;                      // [ksplit][M][N] fp32 when ksplit > 1
  int* status;                          // may be null
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

// Work item w = (output tile, K split): token tile fastest, then K split, then column tile.
struct Item { int tile_n, tile_t, ks, g0, g1; };
__device__ __forceinline__ Item decode_item(int w, const Params& p) {
  Item it;
  it.tile_t = w % p.ntiles_t;
  const int r = w / p.ntiles_t;
  it.ks = r % p.ksplit;
  it.tile_n = r / p.ksplit;
  it.g0 = (it.ks * p.G) / p.ksplit;
  it.g1 = ((it.ks + 1) * p.G) / p.ksplit;
  return it;
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
umma_prefill_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_sc,
                    const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_x, const Params p) {
  constexpr uint32_t LO = 0x000F000Fu;
  constexpr uint32_t MAGIC = BF16 ? 0x43004300u : 0x64006400u;  // 128.0 / 1024.0 in both halves

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages], bar_empty[kStages], bar_afull[kAStages], bar_aempty[kAStages],
      bar_dfull, bar_dempty, bar_drain[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort_i;

  volatile int* s_abort = &s_abort_i;
  int* status = p.status;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nitems = p.ntiles_n * p.ntiles_t * p.ksplit;

  grid_launch_dependents();
  grid_dependency_wait();  // the activations come from the kernel ahead on the stream

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), kDequantWarps / 2 + 2); }
    for (int s = 0; s < kAStages; ++s) { mbar_init(smem_u32(&bar_afull[s]), kDequantWarps / 2); mbar_init(smem_u32(&bar_aempty[s]), 2); }
    mbar_init(smem_u32(&bar_dfull), 2);
    mbar_init(smem_u32(&bar_dempty), kEpiWarps);
    mbar_init(smem_u32(&bar_drain[0]), 1);
    mbar_init(smem_u32(&bar_drain[1]), 1);
    s_abort_i = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(&s_tmem), kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  // Units (one group of one work item) are numbered consecutively over this CTA's items.
  int nunits = 0;
  for (int w = blockIdx.x; w < nitems; w += gridDim.x) { const Item it = decode_item(w, p); nunits += it.g1 - it.g0; }

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tm_w); prefetch_tmap(&tm_sc); prefetch_tmap(&tm_z); prefetch_tmap(&tm_x);
      int issued = 0, i = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
        const Item it = decode_item(w, p);
        const int tile_n = it.tile_n, tile_t = it.tile_t;
        for (int grp = it.g0; grp < it.g1; ++grp, ++i) {
          const int s = i % kStages;
          if (i >= kStages && !wait_bar(&bar_empty[s], ((i / kStages) - 1) & 1, s_abort, status)) { ok = false; break; }
          const uint32_t st = smem_base + s * kStageBytes, bar = smem_u32(&bar_full[s]);
          mbar_expect_tx(bar, kStageTx);
          tma_load_2d(st + kOffW, &tm_w, tile_n * 32, grp * kUnitK, bar);
          tma_load_2d(st + kOffX0, &tm_x, grp * kUnitK, tile_t * kTileT, bar);
          tma_load_2d(st + kOffX1, &tm_x, grp * kUnitK + 64, tile_t * kTileT, bar);
          tma_load_2d(st + kOffSc, &tm_sc, tile_n * 128, grp, bar);
          tma_load_2d(st + kOffZ, &tm_z, tile_n * 32, grp, bar);
          ++issued;
        }
      }
      // do not leave while a copy of ours may still be landing in this CTA's shared memory
      for (int j = issued > kStages ? issued - kStages : 0; j < issued; ++j)
        mbar_wait(smem_u32(&bar_full[j % kStages]), (j / kStages) & 1);
    }
  } else if (warp == 1 || warp == kMmaWarpB) {
    // --------------------------------------------------- MMA issuers (one per A block)
    if (lane == 0) {
      const int blk = warp == 1 ? 0 : 1;
      const uint32_t idesc = umma_idesc(BF16 ? 1 : 0, 128, p.nt);
      int i = 0, li = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x, ++li) {
        const Item it = decode_item(w, p);
        for (int grp = it.g0; grp < it.g1; ++grp, ++i) {
          const int s = i % kStages, sa = i % kAStages;
          if (grp == it.g0 && li > 0 && !wait_bar(&bar_dempty, (li - 1) & 1, s_abort, status)) { ok = false; break; }  // epilogue drained D
          if (!wait_bar(&bar_full[s], (i / kStages) & 1, s_abort, status)) { ok = false; break; }
          if (!wait_bar(&bar_afull[sa], (i / kAStages) & 1, s_abort, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t xaddr = smem_base + s * kStageBytes + kOffX0;
          const uint32_t a = tmem + kColA + sa * 128 + 64 * blk, d = tmem + kColD + 128 * blk;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t bdesc = umma_smem_desc_sw128(xaddr + (ks >> 2) * 16384 + (ks & 3) * 32);
            const uint32_t acc = (grp > it.g0 || ks > 0) ? 1u : 0u;
            umma_ts(d, a + ks * 8, bdesc, idesc, acc);
          }
          umma_commit(smem_u32(&bar_aempty[sa]));
          umma_commit(smem_u32(&bar_empty[s]));
          if (grp == it.g1 - 1) umma_commit(smem_u32(&bar_dfull));
        }
      }
      // everything issued has completed before tensor memory may be released
      umma_commit(smem_u32(&bar_drain[blk]));
      mbar_wait(smem_u32(&bar_drain[blk]), 0);
    }
  } else if (warp < 2 + kDequantWarps) {
    // -------------------------------------------------------------- dequantisers
    const int dw = warp - 2;
    const int q = warp & 3, h = (dw >> 2) & 1, set = dw >> 3;  // set: which units (even / odd) this warp serves
    const int gq = lane >> 2, tig = lane & 3;
    const int chunk = 2 * q + (gq >> 2), inword = (gq & 3) * 4;
    const uint32_t sw_even = ((uint32_t)(chunk ^ ((2 * tig) & 7)) << 4) + inword;
    const uint32_t sw_odd = ((uint32_t)(chunk ^ ((2 * tig + 1) & 7)) << 4) + inword;
    const uint32_t row0 = (uint32_t)(2 * tig) * 128;
    const uint32_t lane_base = tmem + ((uint32_t)(32 * q) << 16);
    for (int i = set; i < nunits; i += 2) {
      const int s = i % kStages, sa = i % kAStages;  // kAStages == 2: sa == set
      if (!wait_bar(&bar_full[s], (i / kStages) & 1, s_abort, status)) break;
      const uint8_t* st = smem_gen + s * kStageBytes;
      // per column of this thread's word: the scale and 1024+z (128+z), each in both halves
      uint32_t sc2[8], zm2[8];
      {
        const uint4 sv = lds128(st, kOffSc + (uint32_t)(64 * q + 8 * gq) * 2);
        const uint32_t zw = lds32(st, kOffZ + (uint32_t)(8 * q + gq) * 4);
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int e = (j < 4) ? 2 * j : 2 * (j - 4) + 1;  // column held by nibble j
          sc2[j] = (e & 1) ? __byte_perm(sw[e >> 1], 0, 0x3232) : __byte_perm(sw[e >> 1], 0, 0x1010);
          const uint32_t z = (zw >> (4 * j)) & 0xFu;
          zm2[j] = (z | (z << 16)) | MAGIC;
        }
      }
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
          // nibble 2b (low) and 2b+1 (high) of rows (k0,k1) and (k2,k3)
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
      if (lane == 0) { mbar_arrive(smem_u32(&bar_afull[sa])); mbar_arrive(smem_u32(&bar_empty[s])); }
    }
  } else if (warp < kMmaWarpB) {
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
    for (int w = blockIdx.x; w < nitems; w += gridDim.x, ++lt) {
      const Item it = decode_item(w, p);
      const int tile_n = it.tile_n, tile_t = it.tile_t;
      if (!wait_bar(&bar_dfull, lt & 1, s_abort, status, 200)) break;
      tc_fence_after();
      const int tok0 = tile_t * kTileT;
      float* part = p.ksplit > 1 ? p.partials + (size_t)it.ks * p.M * p.N : nullptr;
      // A lane holds, per token, two neighbouring columns: an even one in the first A block's accumulator and
      // the odd one after it in the second's (nloc[1] == nloc[0] + 1), and the lanes of a warp hold 32 such
      // pairs side by side: read both accumulators and store the pairs, 128 contiguous bytes per token and
      // warp (256 for an fp32 partial) instead of 32 separate sectors.
      {
        const int n = tile_n * kTileN + nloc[0];
        const bool n_ok = n < p.N;
        const float bv0 = (p.bias && n_ok && !part) ? bias_to_float(p.bias, p.bias_dtype, n) : 0.f;
        const float bv1 = (p.bias && n_ok && !part) ? bias_to_float(p.bias, p.bias_dtype, n + 1) : 0.f;
        for (int c0 = 8 * sub; c0 < p.nt; c0 += 8 * (kEpiWarps / 4)) {
          uint32_t d0[8], d1[8];
          tmem_ld_32x32b_x8(lane_base + kColD + c0, d0);
          tmem_ld_32x32b_x8(lane_base + kColD + 128 + c0, d1);
          tc_wait_ld();
          if (!n_ok) continue;
          const int tok = tok0 + c0;
          const int ntok = min(8, p.M - tok);  // <= 0 when the whole batch of columns is beyond M
          if (part) {
            float* dst = part + (size_t)tok * p.N + n;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              if (c < ntok) __stcg(reinterpret_cast<float2*>(dst + (size_t)c * p.N), make_float2(__uint_as_float(d0[c]), __uint_as_float(d1[c])));
          } else {
            uint16_t* dst = p.out + (size_t)tok * p.N + n;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              if (c < ntok)
                *reinterpret_cast<uint32_t*>(dst + (size_t)c * p.N) =
                    (uint32_t)float_to_raw16<BF16>(__uint_as_float(d0[c]) + bv0) | ((uint32_t)float_to_raw16<BF16>(__uint_as_float(d1[c]) + bv1) << 16);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_dempty));
    }
  }

  // all roles meet here, also after a give-up, so that tensor memory is always released
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, kTmemCols); }
}

// out[m, n] = 16-bit( sum over the K splits, in split order, + bias ): 4 columns per thread.
template <bool BF16>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partials, const void* bias, int bias_dtype,
                                                            uint16_t* __restrict__ out, int M, int N, int ksplit) {
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t total4 = (size_t)M * N / 4;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int ks = 0; ks < ksplit; ++ks) {
      const float4 q = __ldcg(reinterpret_cast<const float4*>(partials + (size_t)ks * M * N) + i);
      v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
    }
    if (bias) {
      const int n = (int)((i * 4) % N);
      v.x += bias_to_float(bias, bias_dtype, n); v.y += bias_to_float(bias, bias_dtype, n + 1);
      v.z += bias_to_float(bias, bias_dtype, n + 2); v.w += bias_to_float(bias, bias_dtype, n + 3);
    }
    const uint32_t o0 = (uint32_t)float_to_raw16<BF16>(v.x) | ((uint32_t)float_to_raw16<BF16>(v.y) << 16);
    const uint32_t o1 = (uint32_t)float_to_raw16<BF16>(v.z) | ((uint32_t)float_to_raw16<BF16>(v.w) << 16);
    reinterpret_cast<uint2*>(out)[i] = make_uint2(o0, o1);
  }
}

template <bool BF16>
static int launch_t(const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tz, const CUtensorMap& tx,
                    const Params& sp, int ctas, cudaStream_t st) {
  // The shared-memory attribute belongs to the device that is current when it is set: one flag per device.
  static std::mutex mu;
  static bool configured[kMaxDevices] = {false};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return NQB200_ERR_UNSUPPORTED_DEVICE; }
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!configured[dev]) {
      if (cudaFuncSetAttribute(umma_prefill_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) {
        cudaGetLastError();
        return NQB200_ERR_LAUNCH;
      }
      configured[dev] = true;
    }
  }
  const int rc = launch_overlapped(umma_prefill_kernel<BF16>, dim3(ctas), dim3(kThreads), kSmem, st, tw, ts, tz, tx, sp);
  if (rc != NQB200_OK || sp.ksplit <= 1) return rc;
  const size_t total4 = (size_t)sp.M * sp.N / 4;
  const int blocks = (int)((total4 + 255) / 256 < (size_t)kNumSMs * 8 ? (total4 + 255) / 256 : (size_t)kNumSMs * 8);
  return launch_overlapped(splitk_reduce_kernel<BF16>, dim3(blocks), dim3(256), 0, st, (const float*)sp.partials, sp.bias, sp.bias_dtype,
                           sp.out, sp.M, sp.N, sp.ksplit);
}

}  // namespace pre

bool umma_prefill_supports(int64_t M, int64_t N, int64_t K, int64_t g) {
  return M > 16 && g == 128 && K % 128 == 0 && N % 32 == 0;
}

// K is split across CTAs when whole tiles would fill the SMs badly (few tiles, or a last wave that
// is mostly empty).  The split is the one a small cost model of the kernel predicts to be fastest.
static int prefill_ksplit(int64_t M, int64_t N, int64_t K, double* est_us = nullptr) {
  const long long tiles = ((N + pre::kTileN - 1) / pre::kTileN) * ((M + pre::kTileT - 1) / pre::kTileT);
  const int G = (int)(K / 128);
  const int nt = M >= pre::kTileT ? pre::kTileT : (int)((M + 15) / 16) * 16;
  // measured: a CTA spends about 1.2 us on one 128-k group of a full 128-token tile (the tensor
  // pipe), never less than 0.7 us (the dequantisers), and about 1.5 us per work item outside its
  // group loop; a split adds a second launch and 8 bytes of fp32 traffic per output and split
  const double t_group = 1.2 * nt / 128.0 > 0.7 ? 1.2 * nt / 128.0 : 0.7;
  int best = 1;
  double best_us = 1e30, unsplit_us = 0.0;
  for (int ks = 1; ks <= 16 && ks <= G; ++ks) {
    const long long waves = (tiles * ks + kNumSMs - 1) / kNumSMs;
    double us = (double)waves * ((double)((G + ks - 1) / ks) * t_group + 1.5);
    if (ks > 1) us += 3.0 + (double)ks * (double)M * (double)N * 8.0 / 6.0e6;
    if (ks == 1) unsplit_us = us;
    if (us < best_us - 1e-9) { best_us = us; best = ks; }
  }
  const bool split = best_us < 0.92 * unsplit_us;  // the model is good to about 10 %
  if (est_us) *est_us = split ? best_us : unsplit_us;
  return split ? best : 1;
}

// What the model above expects this kernel to take (without its fixed launch cost), for the choice between
// this kernel and the two-SM one.
double umma_prefill_estimate_us(int64_t M, int64_t N, int64_t K) {
  double us = 0.0;
  prefill_ksplit(M, N, K, &us);
  return us;
}

int umma_prefill_launches(int64_t M, int64_t N, int64_t K) { return prefill_ksplit(M, N, K) > 1 ? 2 : 1; }

size_t umma_prefill_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const int ks = prefill_ksplit(M, N, K);
  return (size_t)kCounterBytes + (ks > 1 ? (size_t)ks * M * N * sizeof(float) : 0);
}

int launch_umma_prefill(const GemmArgs& a) {
  using namespace pre;
  const int G = a.K / 128;
  Params sp;
  sp.bias = a.bias; sp.bias_dtype = a.bias_dtype; sp.out = (uint16_t*)a.out;
  sp.M = a.M; sp.N = a.N; sp.G = G;
  sp.ntiles_n = (a.N + kTileN - 1) / kTileN;
  sp.ntiles_t = (a.M + kTileT - 1) / kTileT;
  sp.nt = a.M >= kTileT ? kTileT : ((a.M + 15) / 16) * 16;
  sp.status = (a.ws && a.ws_bytes >= (size_t)kCounterBytes) ? (int*)a.ws + (kCounterBytes / 4 - 1) : nullptr;
  sp.ksplit = prefill_ksplit(a.M, a.N, a.K);
  sp.partials = nullptr;
  if (sp.ksplit > 1) {
    if (!a.ws || a.ws_bytes < umma_prefill_workspace_bytes(a.M, a.N, a.K)) return NQB200_ERR_WORKSPACE;
    if (!aligned16(a.ws)) return NQB200_ERR_MISALIGNED;
    sp.partials = (float*)((char*)a.ws + kCounterBytes);
  }
  const long long tiles = (long long)sp.ntiles_n * sp.ntiles_t * sp.ksplit;
  const int ctas = (int)(tiles < kNumSMs ? tiles : kNumSMs);
  alignas(64) CUtensorMap tw, ts, tz, tx;
  const CUtensorMapDataType xdt = a.dtype == NQB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  bool ok = encode_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qw, a.K, a.N / 8, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && encode_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.sc, G, a.N / 2, 1, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tz, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a.qz, G, a.N / 8, 1, 32, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_2d(&tx, xdt, 2, a.x, a.M, a.K, kTileT, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return NQB200_ERR_LAUNCH;
  return a.dtype == NQB200_BF16 ? launch_t<true>(tw, ts, tz, tx, sp, ctas, a.stream)
                                : launch_t<false>(tw, ts, tz, tx, sp, ctas, a.stream);
}

}  // namespace nqb200
