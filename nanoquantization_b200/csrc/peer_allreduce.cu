// One-shot all-reduce over NVLink peer memory for the small messages of
// tensor-parallel decode (the [tokens, hidden] partial sums after a row-parallel
// linear: 8 KB to 512 KB).  NCCL's per-call latency is most of its cost at these
// sizes; here every rank's row-parallel GEMM writes its partial result straight
// into a slot of a buffer that all peers have mapped, and one kernel per rank
//   1. tells every peer "my slot holds call number e" and waits until every peer
//      has said the same (flags in peer memory, one set per CTA),
//   2. reads the same slot of every peer with plain loads and adds them in rank
//      order (so all ranks get identical bits), writing the sum to local memory.
// Slots are used round-robin, so a slot is rewritten only several calls later,
// by which time every peer has passed the barrier of a later call and therefore
// finished reading it; no closing barrier is needed.  The call number lives in
// device memory and is advanced by the kernel itself, so the kernel can be
// replayed from a CUDA graph.
//
// Waits are bounded (one second unless nqb200_comm_set_wait_limit says otherwise): on
// expiry the kernel records NQB200_ERR_WAIT_TIMEOUT in the rank's status word and returns
// without hanging and without writing `out`; the host must read the status
// (nqb200_comm_status) before it trusts the result.
// Only plain peer loads and stores are used: no multimem, no TMA.
#include "common.cuh"
#include "tma_utils.cuh"
#include "peer_layout.cuh"

namespace nqb200 {

constexpr int kArThreads = 256, kArThreadsLarge = 1024;  // per CTA; the larger for messages of 128 KB and more

struct ArParams {
  uint8_t* peers[kMaxRanks];   // every rank's comm buffer as mapped into this process (peers[rank] is our own)
  int rank, world;
  size_t slot_off;             // byte offset of the slot inside the data region
  void* out;
  const void* bias;            // optional, added once after the sum
  int bias_dtype;
  int64_t n;                   // elements (multiple of 8)
  int N;                       // row length, for the bias
};

__device__ __forceinline__ uint4 ld_peer(const uint4* p) {
  uint4 v; asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <bool BF16>
__global__ void __launch_bounds__(kArThreadsLarge) peer_allreduce_kernel(const ArParams p) {
  grid_launch_dependents();
  grid_dependency_wait();  // our slot was filled by the kernel ahead on the stream
  uint8_t* mine = p.peers[p.rank];
  uint32_t* my_epoch = reinterpret_cast<uint32_t*>(mine + kArOffEpoch) + blockIdx.x;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) { s_epoch = *my_epoch + 1; *my_epoch = s_epoch; s_ok = 1; }
  __syncthreads();
  const uint32_t e = s_epoch;
  if (threadIdx.x < p.world) {
    // announce: flag [block][my rank] in peer threadIdx.x's buffer
    uint32_t* theirs = reinterpret_cast<uint32_t*>(p.peers[threadIdx.x] + kArOffFlags) + blockIdx.x * kMaxRanks + p.rank;
    st_flag(theirs, e);
    // wait for peer threadIdx.x's announcement in our buffer
    const uint32_t* ours = reinterpret_cast<const uint32_t*>(mine + kArOffFlags) + blockIdx.x * kMaxRanks + threadIdx.x;
    const unsigned long long t0 = global_timer_ns(), limit = peer_wait_limit_ns(mine);
    uint32_t it = 0;
    // flags only grow; a peer that is already one call ahead shows e + 1
    while ((int32_t)(ld_flag(ours) - e) < 0) {
      if ((++it & 255u) == 0 && global_timer_ns() - t0 > limit) {
        atomicExch(reinterpret_cast<int*>(mine), NQB200_ERR_WAIT_TIMEOUT);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int64_t nvec = p.n >> 3;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    // every rank's 16 bytes are requested before any is used: one NVLink round trip per iteration, not one per rank
    uint4 v[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      v[r] = r < p.world ? ld_peer(reinterpret_cast<const uint4*>(p.peers[r] + kArOffData + p.slot_off) + i) : make_uint4(0u, 0u, 0u, 0u);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < p.world) {  // in rank order: the same bits on every rank
        const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += raw16_to_float<BF16>((uint16_t)(w[j] & 0xFFFF));
          acc[2 * j + 1] += raw16_to_float<BF16>((uint16_t)(w[j] >> 16));
        }
      }
    }
    if (p.bias) {
      const int n0 = (int)((i * 8) % p.N);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += bias_to_float(p.bias, p.bias_dtype, n0 + j);
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = (uint32_t)float_to_raw16<BF16>(acc[2 * j]) | ((uint32_t)float_to_raw16<BF16>(acc[2 * j + 1]) << 16);
    reinterpret_cast<uint4*>(p.out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- two-shot all-reduce for large messages (the [tokens, hidden] partial sums of a row-parallel linear
// in prefill: megabytes).  One-shot makes every rank read every rank's whole message (world x the bytes over
// NVLink); here rank r adds slice r of all ranks' partials (reduce-scatter: (world - 1) / world of the message
// read per rank), leaves the 16-bit sums in a second peer-visible slot, and after a second barrier every rank
// reads the other ranks' slices from there (all-gather: the same amount again).  An element is added once, by
// its owner, in rank order in fp32: every rank gets identical bits.  CTA b of a rank only ever exchanges with
// CTA b of the others (the same partition of a slice over the CTAs on every rank), so the barriers are per
// CTA, as in the one-shot kernel; they use two call numbers per launch.
struct TsParams {
  uint8_t* peers[kMaxRanks];
  int rank, world;
  size_t in_off, res_off;      // byte offsets inside the data region: partial sums (one slot), reduced slices
  void* out;
  const void* bias;
  int bias_dtype;
  int64_t n;                   // elements (multiple of 8)
  int N;
};

template <bool BF16>
__global__ void __launch_bounds__(1024) peer_allreduce_twoshot_kernel(const TsParams p) {
  grid_launch_dependents();
  grid_dependency_wait();  // our partial sums were written by the kernel ahead on the stream
  uint8_t* mine = p.peers[p.rank];
  uint32_t* my_epoch = reinterpret_cast<uint32_t*>(mine + kArOffEpoch3) + blockIdx.x;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) { s_epoch = *my_epoch + 1; *my_epoch = s_epoch + 1; s_ok = 1; }
  __syncthreads();
  const uint32_t e = s_epoch;
  // announce call number `v` to every rank and wait until every rank has announced it (or a later one)
  auto barrier = [&](uint32_t v) {
    __syncthreads();   // everything this CTA wrote is ordered before the announcement (release, cumulative)
    if (threadIdx.x < p.world) {
      uint32_t* theirs = reinterpret_cast<uint32_t*>(p.peers[threadIdx.x] + kArOffFlags3) + blockIdx.x * kMaxRanks + p.rank;
      st_flag(theirs, v);
      const uint32_t* ours = reinterpret_cast<const uint32_t*>(mine + kArOffFlags3) + blockIdx.x * kMaxRanks + threadIdx.x;
      const unsigned long long t0 = global_timer_ns(), limit = peer_wait_limit_ns(mine);
      uint32_t it = 0;
      while ((int32_t)(ld_flag(ours) - v) < 0) {
        if ((++it & 255u) == 0 && global_timer_ns() - t0 > limit) {
          atomicExch(reinterpret_cast<int*>(mine), NQB200_ERR_WAIT_TIMEOUT);
          s_ok = 0;
          break;
        }
      }
    }
    __syncthreads();
    return s_ok != 0;
  };
  if (!barrier(e)) return;
  const int64_t nvec = p.n >> 3, per = (nvec + p.world - 1) / p.world;
  const int64_t step = (int64_t)gridDim.x * blockDim.x, first = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  {
    const int64_t lo = per * p.rank, hi = lo + per < nvec ? lo + per : nvec;
    uint4* res = reinterpret_cast<uint4*>(mine + kArOffData + p.res_off);
    for (int64_t i = lo + first; i < hi; i += step) {
      uint4 v[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        v[r] = r < p.world ? ld_peer(reinterpret_cast<const uint4*>(p.peers[r] + kArOffData + p.in_off) + i) : make_uint4(0u, 0u, 0u, 0u);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < p.world) {
          const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] += raw16_to_float<BF16>((uint16_t)(w[j] & 0xFFFF));
            acc[2 * j + 1] += raw16_to_float<BF16>((uint16_t)(w[j] >> 16));
          }
        }
      }
      if (p.bias) {
        const int n0 = (int)((i * 8) % p.N);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += bias_to_float(p.bias, p.bias_dtype, n0 + j);
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = (uint32_t)float_to_raw16<BF16>(acc[2 * j]) | ((uint32_t)float_to_raw16<BF16>(acc[2 * j + 1]) << 16);
      const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
      res[i] = ov;
      reinterpret_cast<uint4*>(p.out)[i] = ov;
    }
  }
  if (!barrier(e + 1)) return;
  // All-gather: the same positions of every other rank's slice at once, so that a thread has up to seven peer
  // loads in flight (NVLink's latency needs megabytes outstanding); the last slice may be shorter.
  for (int64_t i = first; i < per; i += step) {
    uint4 v[kMaxRanks];
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
      const int64_t j = per * q + i;
      if (q < p.world && q != p.rank && j < nvec)
        v[q] = ld_peer(reinterpret_cast<const uint4*>(p.peers[q] + kArOffData + p.res_off) + j);
    }
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
      const int64_t j = per * q + i;
      if (q < p.world && q != p.rank && j < nvec) reinterpret_cast<uint4*>(p.out)[j] = v[q];
    }
  }
}

}  // namespace nqb200

using namespace nqb200;

// ---- set-up helpers (these, and only these, allocate: a communication buffer is created once) ----
extern "C" int nqb200_comm_alloc(void** ptr, size_t data_bytes) {
  if (!ptr) return NQB200_ERR_NULL_POINTER;
  const size_t total = kArOffData + data_bytes;
  if (cudaMalloc(ptr, total) != cudaSuccess) { cudaGetLastError(); return NQB200_ERR_LAUNCH; }
  if (cudaMemset(*ptr, 0, total) != cudaSuccess) { cudaGetLastError(); return NQB200_ERR_LAUNCH; }
  return NQB200_OK;
}
extern "C" int nqb200_comm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? NQB200_OK : NQB200_ERR_LAUNCH; }
extern "C" int nqb200_comm_export(void* ptr, void* handle64) {
  if (!ptr || !handle64) return NQB200_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) { cudaGetLastError(); return NQB200_ERR_LAUNCH; }
  memcpy(handle64, &h, sizeof(h));
  return NQB200_OK;
}
extern "C" int nqb200_comm_import(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return NQB200_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return NQB200_ERR_LAUNCH; }
  return NQB200_OK;
}
extern "C" int nqb200_comm_unimport(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? NQB200_OK : NQB200_ERR_LAUNCH; }
extern "C" size_t nqb200_comm_data_offset(void) { return kArOffData; }
extern "C" int nqb200_comm_set_wait_limit(void* own_buffer, uint64_t nanoseconds) {
  if (!own_buffer) return NQB200_ERR_NULL_POINTER;
  const unsigned long long v = nanoseconds;
  if (cudaMemcpy((char*)own_buffer + kArOffWaitNs, &v, sizeof(v), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaGetLastError();
    return NQB200_ERR_LAUNCH;
  }
  return NQB200_OK;
}
extern "C" int nqb200_comm_status(void* own_buffer, void* stream) {
  if (!own_buffer) return NQB200_ERR_NULL_POINTER;
  int v = 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemcpyAsync(&v, own_buffer, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    cudaGetLastError();
    return NQB200_ERR_LAUNCH;
  }
  if (v != 0 && cudaMemsetAsync(own_buffer, 0, sizeof(int), st) != cudaSuccess) { cudaGetLastError(); return NQB200_ERR_LAUNCH; }
  return v;
}

extern "C" int nqb200_peer_allreduce(void* const* peer_buffers, int rank, int world, size_t slot_offset, void* out,
                                     const void* bias, int bias_dtype, int64_t M, int64_t N, int dtype, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return NQB200_ERR_BAD_SHAPE;
  if (M < 0 || N <= 0 || (M * N) % 8 != 0 || slot_offset % 16 != 0) return NQB200_ERR_BAD_SHAPE;
  if (dtype != NQB200_F16 && dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  if (M == 0) return NQB200_OK;
  if (!peer_buffers || !out) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(out)) return NQB200_ERR_MISALIGNED;
  ArParams p;
  for (int r = 0; r < kMaxRanks; ++r) p.peers[r] = r < world ? (uint8_t*)peer_buffers[r] : nullptr;
  for (int r = 0; r < world; ++r) if (!p.peers[r]) return NQB200_ERR_NULL_POINTER;
  p.rank = rank; p.world = world; p.slot_off = slot_offset; p.out = out; p.bias = bias; p.bias_dtype = bias_dtype;
  p.n = M * N; p.N = (int)N;
  cudaStream_t st = (cudaStream_t)stream;
  // always the same number of CTAs: each CTA has its own flags and call counter
  const int threads = M * N * 2 >= (128 << 10) ? kArThreadsLarge : kArThreads;
  return launch_overlapped(dtype == NQB200_BF16 ? peer_allreduce_kernel<true> : peer_allreduce_kernel<false>, dim3(kArBlocks),
                           dim3(threads), 0, st, p);
}

extern "C" int nqb200_peer_allreduce_large(void* const* peer_buffers, int rank, int world, size_t in_offset, size_t result_offset,
                                           void* out, const void* bias, int bias_dtype, int64_t M, int64_t N, int dtype,
                                           void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return NQB200_ERR_BAD_SHAPE;
  if (M < 0 || N <= 0 || (M * N) % 8 != 0 || in_offset % 16 != 0 || result_offset % 16 != 0) return NQB200_ERR_BAD_SHAPE;
  if (dtype != NQB200_F16 && dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  if (M == 0) return NQB200_OK;
  if (!peer_buffers || !out) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(out)) return NQB200_ERR_MISALIGNED;
  TsParams p;
  for (int r = 0; r < kMaxRanks; ++r) p.peers[r] = r < world ? (uint8_t*)peer_buffers[r] : nullptr;
  for (int r = 0; r < world; ++r) if (!p.peers[r]) return NQB200_ERR_NULL_POINTER;
  p.rank = rank; p.world = world; p.in_off = in_offset; p.res_off = result_offset; p.out = out; p.bias = bias;
  p.bias_dtype = bias_dtype; p.n = M * N; p.N = (int)N;
  // always the same number of CTAs: each CTA has its own flags and call counter
  return launch_overlapped(dtype == NQB200_BF16 ? peer_allreduce_twoshot_kernel<true> : peer_allreduce_twoshot_kernel<false>,
                           dim3(kTsBlocks), dim3(1024), 0, (cudaStream_t)stream, p);
}
