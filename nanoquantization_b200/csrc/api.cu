// C ABI of the library: argument checks and kernel choice.  No allocation,
// no exceptions; the only mutable state in the library is per-device set-up
// flags (kernel attributes, the address of the fixed scratch array), each
// guarded by a mutex.
#include "common.cuh"
#include "peer_layout.cuh"

using namespace nqb200;

extern "C" int nqb200_version(void) { return 100; }

extern "C" const char* nqb200_status_string(int status) {
  switch (status) {
    case NQB200_OK: return "ok";
    case NQB200_ERR_BAD_SHAPE: return "bad shape: sizes must be positive, K % group_size == 0 and N % 8 == 0";
    case NQB200_ERR_BAD_DTYPE: return "bad dtype: expected NQB200_F16 or NQB200_BF16";
    case NQB200_ERR_MISALIGNED: return "misaligned pointer: every buffer must be 16-byte aligned";
    case NQB200_ERR_NULL_POINTER: return "null pointer";
    case NQB200_ERR_WORKSPACE: return "workspace missing or smaller than nqb200_gemm_workspace_bytes()";
    case NQB200_ERR_UNSUPPORTED_DEVICE: return "unsupported device: the kernels are built for sm_100a (B200) only";
    case NQB200_ERR_LAUNCH: return "CUDA launch failed";
    case NQB200_ERR_WAIT_TIMEOUT: return "a bounded device-side wait timed out";
    case NQB200_ERR_TOO_LARGE: return "size exceeds the supported maximum";
    default: return "unknown status";
  }
}

extern "C" int nqb200_device_supported(int device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return major == 10 ? 1 : 0;
}

static int check_shape(int64_t M, int64_t N, int64_t K, int64_t g, int dtype) {
  if (M < 0 || N <= 0 || K <= 0 || g <= 0 || K % g != 0 || N % 8 != 0) return NQB200_ERR_BAD_SHAPE;
  if (M > (1 << 24) || N > (1 << 24) || K > (1 << 24)) return NQB200_ERR_TOO_LARGE;
  if (dtype != NQB200_F16 && dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  return NQB200_OK;
}

extern "C" size_t nqb200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int64_t g, int dtype) {
  if (check_shape(M, N, K, g, dtype) != NQB200_OK || M == 0) return 0;
  if (umma_pair_supports(M, N, K, g)) return umma_pair_workspace_bytes(M, N, K);
  if (umma_prefill_supports(M, N, K, g)) return umma_prefill_workspace_bytes(M, N, K);
  if (stream_supports(M, N, K, g)) return stream_workspace_bytes(M, N, K);
  if (!decode_mma_supports(M, N, K, g)) return 0;
  const DecodePlan p = plan_decode(M, N, K, g);
  return p.ksplit > 1 ? p.counter_bytes + p.partial_bytes : 0;
}

extern "C" const char* nqb200_gemm_kernel_name(int64_t M, int64_t N, int64_t K, int64_t g, int dtype) {
  if (check_shape(M, N, K, g, dtype) != NQB200_OK) return "invalid";
  if (umma_pair_supports(M, N, K, g)) return "prefill_tcgen05_pair";
  if (umma_prefill_supports(M, N, K, g)) return "prefill_tcgen05";
  if (stream_supports(M, N, K, g)) return "decode_stream";
  if (!decode_mma_supports(M, N, K, g)) return "generic";
  return "decode_mma";
}

extern "C" int nqb200_gemm_launch_count(int64_t M, int64_t N, int64_t K, int64_t g, int dtype) {
  if (check_shape(M, N, K, g, dtype) != NQB200_OK || M == 0) return 0;
  if (umma_pair_supports(M, N, K, g)) return umma_pair_launches(M, N, K);
  if (umma_prefill_supports(M, N, K, g)) return umma_prefill_launches(M, N, K);
  if (stream_supports(M, N, K, g)) return stream_launches(M, N, K);
  return 1;
}

extern "C" int nqb200_gemm(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                           const void* bias, int bias_dtype, void* out, int64_t M, int64_t N, int64_t K,
                           int64_t g, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  const int st = check_shape(M, N, K, g, dtype);
  if (st != NQB200_OK) return st;
  if (M == 0) return NQB200_OK;
  if (!x || !qweight || !qscales || !qzeros || !out) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(qscales) || !aligned16(qzeros) || !aligned16(out) ||
      (bias && !aligned16(bias)))
    return NQB200_ERR_MISALIGNED;
  if (bias && bias_dtype != NQB200_F16 && bias_dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  GemmArgs a;
  a.x = x; a.qw = (const uint32_t*)qweight; a.sc = qscales; a.qz = (const uint32_t*)qzeros;
  a.bias = bias; a.bias_dtype = bias_dtype; a.out = out;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.g = (int)g; a.dtype = dtype;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = (cudaStream_t)stream;
  if (umma_pair_supports(M, N, K, g)) return launch_umma_pair(a);
  if (umma_prefill_supports(M, N, K, g)) return launch_umma_prefill(a);
  if (stream_supports(M, N, K, g)) return launch_stream(a);
  if (decode_mma_supports(M, N, K, g)) return launch_decode_mma(a);
  return launch_generic(a);
}

extern "C" int nqb200_decode_tile_columns(void) { return stream_tile_columns(); }

extern "C" int nqb200_gemm_gate_up_silu_supported(int64_t M, int64_t N, int64_t K, int64_t g, int dtype) {
  if (check_shape(M, N, K, g, dtype) != NQB200_OK || M == 0) return 0;
  return !umma_prefill_supports(M, N, K, g) && stream_silu_supported(M, N, K, g) ? 1 : 0;
}

extern "C" int nqb200_gemm_gate_up_silu(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                                        const void* bias, int bias_dtype, void* out, int64_t M, int64_t N, int64_t K,
                                        int64_t g, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  const int st = check_shape(M, N, K, g, dtype);
  if (st != NQB200_OK) return st;
  if (M == 0) return NQB200_OK;
  if (!nqb200_gemm_gate_up_silu_supported(M, N, K, g, dtype)) return NQB200_ERR_BAD_SHAPE;
  if (!x || !qweight || !qscales || !qzeros || !out) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(qscales) || !aligned16(qzeros) || !aligned16(out) ||
      (bias && !aligned16(bias)))
    return NQB200_ERR_MISALIGNED;
  if (bias && bias_dtype != NQB200_F16 && bias_dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  GemmArgs a;
  a.x = x; a.qw = (const uint32_t*)qweight; a.sc = qscales; a.qz = (const uint32_t*)qzeros;
  a.bias = bias; a.bias_dtype = bias_dtype; a.out = out;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.g = (int)g; a.dtype = dtype;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = (cudaStream_t)stream;
  a.epilogue = 1;
  return launch_stream(a);
}

extern "C" int nqb200_gemm_allreduce_supported(int64_t M, int64_t N, int64_t K, int64_t g, int dtype, int world, size_t slot_bytes) {
  if (check_shape(M, N, K, g, dtype) != NQB200_OK || M == 0 || world < 2 || world > kMaxRanks) return 0;
  if ((size_t)world * (size_t)M * (size_t)N * 2 > slot_bytes) return 0;
  return !umma_prefill_supports(M, N, K, g) && stream_allreduce_supported(M, N, K, g) ? 1 : 0;
}

extern "C" int nqb200_gemm_allreduce(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                                     const void* bias, int bias_dtype, void* out, int64_t M, int64_t N, int64_t K, int64_t g,
                                     int dtype, void* workspace, size_t workspace_bytes, void* const* peer_buffers, int rank,
                                     int world, size_t slot_offset, size_t slot_bytes, void* stream) {
  const int st = check_shape(M, N, K, g, dtype);
  if (st != NQB200_OK) return st;
  if (M == 0) return NQB200_OK;
  if (rank < 0 || rank >= world || slot_offset % 16 != 0) return NQB200_ERR_BAD_SHAPE;
  if (!nqb200_gemm_allreduce_supported(M, N, K, g, dtype, world, slot_bytes)) return NQB200_ERR_BAD_SHAPE;
  if (!x || !qweight || !qscales || !qzeros || !out || !peer_buffers) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(qscales) || !aligned16(qzeros) || !aligned16(out) ||
      (bias && !aligned16(bias)))
    return NQB200_ERR_MISALIGNED;
  if (bias && bias_dtype != NQB200_F16 && bias_dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  PeerEpilogue pe;
  for (int r = 0; r < kMaxRanks; ++r) pe.peers[r] = r < world ? (uint8_t*)peer_buffers[r] : nullptr;
  for (int r = 0; r < world; ++r) if (!pe.peers[r]) return NQB200_ERR_NULL_POINTER;
  pe.rank = rank; pe.world = world; pe.slot_off = slot_offset;
  GemmArgs a;
  a.x = x; a.qw = (const uint32_t*)qweight; a.sc = qscales; a.qz = (const uint32_t*)qzeros;
  a.bias = bias; a.bias_dtype = bias_dtype; a.out = out;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.g = (int)g; a.dtype = dtype;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = (cudaStream_t)stream;
  a.peer = &pe;
  return launch_stream(a);
}

extern "C" int nqb200_gemm_decode_fused_supported(int64_t M, int64_t N, int64_t K, int64_t g, int dtype, int flags, int world,
                                                  size_t slot_bytes) {
  if (check_shape(M, N, K, g, dtype) != NQB200_OK || M == 0 || umma_prefill_supports(M, N, K, g)) return 0;
  if (!stream_supports(M, N, K, g)) return 0;
  const bool silu = flags & NQB200_FUSE_SILU_MUL, residual = flags & NQB200_FUSE_RESIDUAL, ar = flags & NQB200_FUSE_ALLREDUCE;
  if (silu && (residual || ar)) return 0;
  if (silu && !stream_silu_supported(M, N, K, g)) return 0;
  if ((residual || ar) && !stream_allreduce_supported(M, N, K, g)) return 0;  // every tile finished by the reducing kernel
  if (ar && (world < 2 || world > kMaxRanks || (size_t)world * (size_t)M * (size_t)N * 2 > slot_bytes)) return 0;
  return 1;
}

extern "C" int nqb200_gemm_decode_fused(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                                        const void* bias, int bias_dtype, void* out, int64_t M, int64_t N, int64_t K, int64_t g,
                                        int dtype, void* workspace, size_t workspace_bytes, const nqb200_decode_fusion* f,
                                        void* const* peer_buffers, int rank, int world, size_t slot_offset, size_t slot_bytes,
                                        void* stream) {
  const int st = check_shape(M, N, K, g, dtype);
  if (st != NQB200_OK) return st;
  if (M == 0) return NQB200_OK;
  if (!f) return NQB200_ERR_NULL_POINTER;
  const int flags = (f->norm_ssq ? NQB200_FUSE_RMSNORM : 0) | (f->residual_in ? NQB200_FUSE_RESIDUAL : 0) |
                    (f->silu_mul ? NQB200_FUSE_SILU_MUL : 0) | (peer_buffers ? NQB200_FUSE_ALLREDUCE : 0);
  if (!nqb200_gemm_decode_fused_supported(M, N, K, g, dtype, flags, world, slot_bytes)) return NQB200_ERR_BAD_SHAPE;
  if (!x || !qweight || !qscales || !qzeros || !out) return NQB200_ERR_NULL_POINTER;
  if (f->norm_ssq && (!f->norm_weight || f->norm_tiles <= 0)) return NQB200_ERR_NULL_POINTER;
  if (f->residual_in && !f->ssq_out) return NQB200_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(qscales) || !aligned16(qzeros) || !aligned16(out) ||
      (bias && !aligned16(bias)) || (f->residual_in && !aligned16(f->residual_in)) || (f->norm_weight && !aligned16(f->norm_weight)))
    return NQB200_ERR_MISALIGNED;
  if (bias && bias_dtype != NQB200_F16 && bias_dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  PeerEpilogue pe;
  if (peer_buffers) {
    if (rank < 0 || rank >= world || slot_offset % 16 != 0) return NQB200_ERR_BAD_SHAPE;
    for (int r = 0; r < kMaxRanks; ++r) pe.peers[r] = r < world ? (uint8_t*)peer_buffers[r] : nullptr;
    for (int r = 0; r < world; ++r) if (!pe.peers[r]) return NQB200_ERR_NULL_POINTER;
    pe.rank = rank; pe.world = world; pe.slot_off = slot_offset;
  }
  GemmArgs a;
  a.x = x; a.qw = (const uint32_t*)qweight; a.sc = qscales; a.qz = (const uint32_t*)qzeros;
  a.bias = bias; a.bias_dtype = bias_dtype; a.out = out;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.g = (int)g; a.dtype = dtype;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = (cudaStream_t)stream;
  a.norm_ssq = f->norm_ssq; a.norm_tiles = (int)f->norm_tiles; a.norm_weight = f->norm_weight; a.norm_eps = f->norm_eps;
  a.residual_in = f->residual_in; a.ssq_out = f->ssq_out;
  a.epilogue = f->silu_mul ? 1 : 0;
  a.peer = peer_buffers ? &pe : nullptr;
  return launch_stream(a);
}

extern "C" int nqb200_workspace_status(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace) return NQB200_ERR_NULL_POINTER;
  if (workspace_bytes < (size_t)kCounterBytes) return NQB200_ERR_WORKSPACE;
  int* word = reinterpret_cast<int*>(workspace) + (kCounterBytes / 4 - 1);
  int v = 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemcpyAsync(&v, word, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    cudaGetLastError();
    return NQB200_ERR_LAUNCH;
  }
  if (v != 0) {
    if (cudaMemsetAsync(word, 0, sizeof(int), st) != cudaSuccess) { cudaGetLastError(); return NQB200_ERR_LAUNCH; }
  }
  return v;
}
