// Shared helpers for the nqb200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>
#include "nqb200.h"

namespace nqb200 {

constexpr int kNumSMs = 148;          // B200: 2 dies x 74 SMs
constexpr int kCounterBytes = 1 << 16; // head of the workspace: tile-arrival counters
constexpr int kMaxDevices = 64;        // per-device host-side state (kernel attributes, symbol addresses)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline int check_launch() {
  return cudaGetLastError() == cudaSuccess ? NQB200_OK : NQB200_ERR_LAUNCH;
}

// Launch with programmatic stream serialisation: the grid may become resident while the kernel
// before it on the stream is still finishing, and must execute grid_dependency_wait() before it
// touches anything that kernel may write (or writes anything that kernel may read).  Read-only
// weights can be fetched before the wait, which hides the launch and first-byte latency of
// back-to-back layers.  Captured into a CUDA graph this becomes a programmatic dependency edge.
template <typename... KArgs, typename... Args>
static inline int launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) != cudaSuccess) { cudaGetLastError(); return NQB200_ERR_LAUNCH; }
  return NQB200_OK;
}

// How the split-K decode kernel tiles a problem; the same plan sizes the workspace.
struct DecodePlan {
  int mt;        // 8-token tiles per CTA (1 or 2)
  int ng;        // packed words per thread per row (4 -> 256-column CTA tile, 2 -> 128)
  int tile_n;    // 64 * ng
  int ntiles;    // ceil(N / tile_n)
  int mchunks;   // ceil(M / (8*mt))
  int gpc;       // quantisation groups per CTA
  int ksplit;    // CTAs along K
  size_t counter_bytes;
  size_t partial_bytes;
};
DecodePlan plan_decode(int64_t M, int64_t N, int64_t K, int64_t g);

struct PeerEpilogue;

struct GemmArgs {
  const void* x; const uint32_t* qw; const void* sc; const uint32_t* qz;
  const void* bias; int bias_dtype; void* out;
  int M, N, K, g;
  int dtype;
  void* ws; size_t ws_bytes;
  cudaStream_t stream;
  // streaming decode kernel only: RMSNorm of the input from per-tile sums of squares; residual add and
  // sums of squares of the output (see StreamParams)
  const float* norm_ssq = nullptr; int norm_tiles = 0; const void* norm_weight = nullptr; float norm_eps = 0.f;
  const void* residual_in = nullptr; float* ssq_out = nullptr;
  const PeerEpilogue* peer = nullptr;  // all-reduce over peer memory in the reducing kernel (streaming decode kernel only)
  int epilogue = 0;  // 1: the matrix is gate|up, out[M, N/2] = silu(gate) * up (streaming decode kernel only)
};

int launch_decode_mma(const GemmArgs& a);
int launch_generic(const GemmArgs& a);
int launch_stream(const GemmArgs& a);
int launch_umma_prefill(const GemmArgs& a);
bool umma_prefill_supports(int64_t M, int64_t N, int64_t K, int64_t g);
size_t umma_prefill_workspace_bytes(int64_t M, int64_t N, int64_t K);

bool stream_supports(int64_t M, int64_t N, int64_t K, int64_t g);
size_t stream_workspace_bytes(int64_t M, int64_t N, int64_t K);
int stream_launches(int64_t M, int64_t N, int64_t K);
int stream_tile_columns();
bool stream_silu_supported(int64_t M, int64_t N, int64_t K, int64_t g);
bool stream_allreduce_supported(int64_t M, int64_t N, int64_t K, int64_t g);
int umma_prefill_launches(int64_t M, int64_t N, int64_t K);
double umma_prefill_estimate_us(int64_t M, int64_t N, int64_t K);
// gemm_umma_pair.cu: the two-SM (cta_group::2) tcgen05 kernel for more than 128 tokens.
int launch_umma_pair(const GemmArgs& a);
bool umma_pair_supports(int64_t M, int64_t N, int64_t K, int64_t g);
size_t umma_pair_workspace_bytes(int64_t M, int64_t N, int64_t K);
int umma_pair_launches(int64_t M, int64_t N, int64_t K);
bool decode_mma_supports(int64_t M, int64_t N, int64_t K, int64_t g);

// ---- device helpers -------------------------------------------------------
#ifdef __CUDACC__
// Returns once the kernel before this one on the stream has completed and its writes are visible.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel on the stream (if launched for overlap) become resident as SMs free up.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif
__device__ __forceinline__ float bias_to_float(const void* bias, int bias_dtype, int n) {
  if (bias_dtype == NQB200_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n]);
  return __half2float(reinterpret_cast<const __half*>(bias)[n]);
}

template <bool BF16> __device__ __forceinline__ float raw16_to_float(uint16_t v) {
  if (BF16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
  return __half2float(__ushort_as_half(v));
}
template <bool BF16> __device__ __forceinline__ uint16_t float_to_raw16(float f) {
  if (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  return __half_as_ushort(__float2half_rn(f));
}

}  // namespace nqb200
