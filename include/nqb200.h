/* nqb200 -- C ABI of the B200 (sm_100a) AWQ W4A16 linear kernels.
 *
 * Every entry point takes plain device pointers and sizes; nothing here
 * allocates, frees or retains device memory (except nqb200_comm_alloc /
 * nqb200_comm_free / nqb200_comm_import, the one-time set-up of a
 * tensor-parallel communication buffer), throws, aborts or traps.  All
 * functions returning int return NQB200_OK (0) or a nonzero status; the text
 * for a status comes from nqb200_status_string().
 *
 * Data layout (row-major, contiguous), as written by the reference packer
 * nanoquantization/layers/gemm.py:447-550:
 *   qweight  int32 [K, N/8]    nibble j of a word holds column 8*i + {0,2,4,6,1,3,5,7}[j]
 *   qscales  f16|bf16 [K/g, N]
 *   qzeros   int32 [K/g, N/8]  packed like qweight
 *   x        f16|bf16 [M, K]   (same dtype as qscales)
 *   out      f16|bf16 [M, N]
 * All pointers must be 16-byte aligned.  `stream` is a cudaStream_t passed as
 * void* (NULL = the legacy default stream).  Calls are asynchronous on it.
 */
#ifndef NQB200_H
#define NQB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  NQB200_OK = 0,
  NQB200_ERR_BAD_SHAPE = 1,     /* a size is <= 0 or violates K % g, N % 8 */
  NQB200_ERR_BAD_DTYPE = 2,
  NQB200_ERR_MISALIGNED = 3,    /* a pointer is not 16-byte aligned */
  NQB200_ERR_NULL_POINTER = 4,
  NQB200_ERR_WORKSPACE = 5,     /* workspace missing or too small */
  NQB200_ERR_UNSUPPORTED_DEVICE = 6, /* not compute capability 10.x */
  NQB200_ERR_LAUNCH = 7,        /* the CUDA runtime refused the launch */
  NQB200_ERR_WAIT_TIMEOUT = 8,  /* a bounded device-side wait gave up */
  NQB200_ERR_TOO_LARGE = 9      /* a size exceeds a stated maximum */
};

enum { NQB200_F16 = 0, NQB200_BF16 = 1 };

/* Library version (major*100 + minor). */
int nqb200_version(void);

/* Text for a status code; never NULL. */
const char* nqb200_status_string(int status);

/* 1 if `device` has compute capability 10.x (B200), 0 otherwise, <0 on a CUDA error. */
int nqb200_device_supported(int device);

/* Unpack int4 values to natural column order, one byte each (0..15).
 * out_u8[r, 8*i + e] = (words[r, i] >> {0,16,4,20,8,24,12,28}[e]) & 0xF.
 * Replaces the shift/mask step of the reference kernels, gemm.py:64-69 and
 * gemm.py:301-302; serves qweight and qzeros alike.  Bit-exact. */
int nqb200_unpack_int4(const void* words, void* out_u8, int64_t rows, int64_t cols_packed,
                       void* stream);

/* Dense weight W[K, N] = dtype(q - z) * s in the scale dtype, one rounding per
 * element.  Replaces awq_dequantize, gemm.py:126-180 (kernel gemm.py:10-123).
 * Bit-exact with that arithmetic, including at ragged N where the reference
 * kernel's load mask is wrong. */
int nqb200_dequant(const void* qweight, const void* qscales, const void* qzeros, void* out,
                   int64_t K, int64_t N, int64_t group_size, int dtype, void* stream);

/* Bytes of scratch nqb200_gemm needs for this problem.  The scratch must be
 * zero-filled once before its first use (the kernels restore it to zero), and
 * must not be shared by calls that can overlap on the GPU. */
size_t nqb200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int64_t group_size, int dtype);

/* out[M, N] = x[M, K] @ ((q - z) * s) (+ bias), fp32 accumulation, result in
 * `dtype`.  Replaces both branches of WQLinear_GEMM.forward, gemm.py:552-567:
 * awq_gemm (gemm.py:329-379, M < 256) and awq_dequantize + torch.matmul
 * (gemm.py:560-561, M >= 256), and the bias add gemm.py:565-566.
 * `bias` may be NULL; `bias_dtype` is NQB200_F16 or NQB200_BF16 (the reference
 * module stores its bias in bf16, gemm.py:435-443). */
int nqb200_gemm(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                const void* bias, int bias_dtype, void* out,
                int64_t M, int64_t N, int64_t K, int64_t group_size, int dtype,
                void* workspace, size_t workspace_bytes, void* stream);

/* The merged gate|up projection of a Qwen3 MLP with its activation, for decode-sized M:
 *   out[M, N/2] = silu(y[:, :N/2]) * y[:, N/2:],  y = x @ dequant(qweight, qscales, qzeros) (+ bias)
 * with the roundings of the separate steps (y, silu(gate) and the product each rounded to the
 * 16-bit type: models/qwen3_quantized.py:150 of the reference runs them as a linear, F.silu and a
 * multiply).  The activation runs in the kernel that adds the split-K partial sums, so it costs no
 * launch of its own.  Only where nqb200_gemm_gate_up_silu_supported() says 1 (M <= 16, group 128,
 * N a multiple of twice nqb200_decode_tile_columns(), K long enough that every column tile is split across
 * CTAs); elsewhere it
 * returns NQB200_ERR_BAD_SHAPE and the caller runs nqb200_gemm + nqb200_silu_mul.  Workspace as
 * for nqb200_gemm with the same M, N, K. */
int nqb200_gemm_gate_up_silu_supported(int64_t M, int64_t N, int64_t K, int64_t group_size, int dtype);
int nqb200_gemm_gate_up_silu(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                             const void* bias, int bias_dtype, void* out, int64_t M, int64_t N, int64_t K,
                             int64_t group_size, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* The decode-sized linear with what surrounds it in a Qwen3 block, in its own two launches (the
 * streaming kernel and the kernel that adds its split-K partial sums).  Any combination that
 * nqb200_gemm_decode_fused_supported() accepts (flags = OR of NQB200_FUSE_*):
 *   RMSNORM   x is the residual stream h [M, K]; the linear's input is RMSNorm(h) * norm_weight
 *             (layers/norm.py:18-32 of the reference, same roundings), with mean(h^2) taken from sums
 *             of squares per token and column tile of h (nqb200_decode_tile_columns() columns per tile):
 *             norm_ssq [M, norm_tiles], fp32.
 *   RESIDUAL  out [M, N] = 16-bit(16-bit(y) + residual_in) (models/qwen3_quantized.py:213-214), the
 *             new residual stream, and ssq_out [M, ceil(N / nqb200_decode_tile_columns())] = its sums of squares per token and
 *             tile: what the RMSNORM prologue of the next linear reads.
 *   SILU_MUL  as nqb200_gemm_gate_up_silu (out is [M, N/2]); not together with RESIDUAL or ALLREDUCE.
 *   ALLREDUCE as nqb200_gemm_allreduce (peer_buffers != NULL); the residual is added after the sum.
 * A block then costs two launches per linear and nothing for its norms, activation and all-reduces.
 * No counterpart in the reference (its block is separate modules). */
/* Columns per tile of the decode-sized kernels: the granularity of norm_ssq / ssq_out below. */
int nqb200_decode_tile_columns(void);
enum { NQB200_FUSE_RMSNORM = 1, NQB200_FUSE_RESIDUAL = 2, NQB200_FUSE_SILU_MUL = 4, NQB200_FUSE_ALLREDUCE = 8 };
typedef struct nqb200_decode_fusion {
  const float* norm_ssq;   /* NULL: x is used as it is */
  int64_t norm_tiles;
  const void* norm_weight; /* [K], the model dtype */
  float norm_eps;
  int silu_mul;
  const void* residual_in; /* NULL: out = y */
  float* ssq_out;
} nqb200_decode_fusion;
int nqb200_gemm_decode_fused_supported(int64_t M, int64_t N, int64_t K, int64_t group_size, int dtype, int flags,
                                       int world, size_t slot_bytes);
int nqb200_gemm_decode_fused(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                             const void* bias, int bias_dtype, void* out, int64_t M, int64_t N, int64_t K,
                             int64_t group_size, int dtype, void* workspace, size_t workspace_bytes,
                             const nqb200_decode_fusion* fusion, void* const* peer_buffers, int rank, int world,
                             size_t slot_offset, size_t slot_bytes, void* stream);

/* nqb200_gemm for up to 16 tokens without any device allocation by anyone.
 * It has no counterpart in the reference.  It is for callers that cannot
 * provide a scratch buffer because they cannot allocate: hosts that own all
 * device memory themselves (a serving engine whose KV-cache pool already holds
 * every free byte, a plugin interface without an allocator in which a
 * cudaMalloc from the plugin is an error).  The scratch is a fixed array inside
 * the library, about 9.4 MiB, resident on every GPU that loads the library
 * until the process exits.  Limits: 1 <= M <= 16, group_size == 128,
 * N % 32 == 0; anything else returns NQB200_ERR_TOO_LARGE (NQB200_ERR_BAD_SHAPE
 * for sizes no entry point accepts).  It calls no cudaMalloc, cudaFree or other
 * allocating routine.  The first call on a device looks up the array's device
 * address (with that device current); make that first call outside any stream
 * capture.  All calls share the one array: calls that can overlap on the GPU
 * (different streams, no dependency between them) race and must be serialised
 * by the caller.  Results are bit-identical to nqb200_gemm for the same inputs. */
int nqb200_gemm_decode_noalloc(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                               const void* bias, int bias_dtype, void* out,
                               int64_t M, int64_t N, int64_t K, int64_t group_size, int dtype, void* stream);

/* Quantise an nn.Linear weight [N, K] (weight_dtype: 0 f16, 1 bf16, 2 f32) group-wise to int4 with
 * zero-points and pack it into qweight / qscales (scales_dtype) / qzeros, in one kernel.  Replaces,
 * rounding for rounding, pseudo_quantize (nanoquantization/utils/quantization.py:20-41) followed by
 * WQLinear_GEMM.from_linear (gemm.py:478-548), the pair the quantizer runs per layer
 * (awq/quantizer.py:150-170). */
int nqb200_quantize_pack(const void* weight, int weight_dtype, void* qweight, void* qscales, void* qzeros,
                         int64_t N, int64_t K, int64_t group_size, int scales_dtype, void* stream);

/* Elementwise steps either side of the linears in a Qwen3 block, one launch each.
 * nqb200_add_rmsnorm: h = x (+ residual); residual_out = h (may alias residual; may be NULL);
 *   out = RMSNorm(h) * weight.  Replaces the residual adds models/qwen3_quantized.py:213-214 and
 *   RMSNorm layers/norm.py:18-32.  x, residual, out: [T, H]; weight: [H].
 * nqb200_qknorm_rope: in place on a fused [T, row_stride] buffer holding q heads, then k heads, then v:
 *   per-head RMSNorm (models/qwen3_quantized.py:88) then rotary embedding (layers/rope.py:24-45) with the
 *   fp32 table cos_sin [max_pos, head_dim] = cos | sin and int64 positions [T].  head_dim must be 128.
 * nqb200_silu_mul: out[T, I] = silu(gate_up[:, :I]) * gate_up[:, I:] (models/qwen3_quantized.py:150). */
int nqb200_add_rmsnorm(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                       int64_t T, int64_t H, float eps, int dtype, void* stream);
int nqb200_qknorm_rope(void* qkv, const void* q_weight, const void* k_weight, const float* cos_sin,
                       const int64_t* positions, int64_t T, int64_t num_q_heads, int64_t num_kv_heads,
                       int64_t head_dim, int64_t row_stride, float eps, int dtype, void* stream);
int nqb200_silu_mul(const void* gate_up, void* out, int64_t T, int64_t I, int dtype, void* stream);
/* nqb200_qknorm_rope that also stores the rotated k and the v of every token in a paged KV cache:
 * k_cache and v_cache are [slots, num_kv_heads, 128] in the model dtype, slots[t] (int64) is
 * token t's slot (block * block_size + offset).  No counterpart in the reference (it has no cache). */
int nqb200_qknorm_rope_kv(void* qkv, const void* q_weight, const void* k_weight, const float* cos_sin,
                          const int64_t* positions, const int64_t* slots, void* k_cache, void* v_cache, int64_t T,
                          int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim, int64_t row_stride, float eps,
                          int dtype, void* stream);

/* One-shot all-reduce (sum) over NVLink peer memory for the small [M, N] partial results of a
 * row-parallel linear.  No counterpart in the reference (it has no distributed code).
 * Set-up, once: every rank calls nqb200_comm_alloc (a cudaMalloc'd, zeroed buffer: a header of
 * nqb200_comm_data_offset() bytes, then `data_bytes` of slots), exports it with nqb200_comm_export
 * (a 64-byte CUDA IPC handle), exchanges handles with its peers by any host channel, and maps each
 * peer's buffer with nqb200_comm_import.  Per call: every rank's GEMM writes its partial result at
 * `slot_offset` inside its own data region, then every rank calls nqb200_peer_allreduce with the
 * same arguments (peer_buffers[r] = rank r's buffer as mapped here; peer_buffers[rank] = its own).
 * The kernel waits (at most about a second; then the first int of the rank's buffer holds
 * NQB200_ERR_WAIT_TIMEOUT) until all ranks have arrived, then adds the slots in rank order and an
 * optional bias and writes `out` in local memory.  Use slots round-robin: a slot may be rewritten
 * once two later calls have been issued.  M * N must be a multiple of 8. */
int nqb200_comm_alloc(void** ptr, size_t data_bytes);
int nqb200_comm_free(void* ptr);
int nqb200_comm_export(void* ptr, void* handle64);
int nqb200_comm_import(const void* handle64, void** ptr);
int nqb200_comm_unimport(void* ptr);
size_t nqb200_comm_data_offset(void);
/* How long this rank's all-reduce kernels wait for their peers before they give up (default one
 * second); `own_buffer` is the rank's own nqb200_comm_alloc buffer.  Synchronous; call it between
 * steps. */
int nqb200_comm_set_wait_limit(void* own_buffer, uint64_t nanoseconds);
/* Waits for `stream`, then returns what this rank's all-reduce kernels recorded in its own buffer:
 * NQB200_OK, or NQB200_ERR_WAIT_TIMEOUT if a wait for a peer ran out (the kernel then returned
 * without writing its output: the result of that call, and of everything computed from it, is
 * undefined and must be discarded).  The record is cleared. */
int nqb200_comm_status(void* own_buffer, void* stream);
/* A row-parallel linear and its all-reduce in one call, for decode-sized M: every rank calls it with
 * its shard (x [M, K/world], weights [K/world, N]); the kernel that finishes the GEMM stores the
 * rank's partial result (rounded to the 16-bit type) straight into the slot at `slot_offset` of
 * every rank's buffer, waits for every rank (bounded, flags in peer memory) and adds the ranks'
 * partials in rank order, plus `bias` once, into `out` [M, N]: the same bits as nqb200_gemm into the
 * slot followed by nqb200_peer_allreduce, with one launch and one NVLink crossing less.  The slot
 * must hold world * M * N * 2 bytes (`slot_bytes` = its size); use slots round-robin (at least 3).
 * Only where nqb200_gemm_allreduce_supported() says 1, else NQB200_ERR_BAD_SHAPE.  Workspace as for
 * nqb200_gemm.  No counterpart in the reference (single GPU). */
int nqb200_gemm_allreduce_supported(int64_t M, int64_t N, int64_t K, int64_t group_size, int dtype, int world,
                                    size_t slot_bytes);
int nqb200_gemm_allreduce(const void* x, const void* qweight, const void* qscales, const void* qzeros,
                          const void* bias, int bias_dtype, void* out, int64_t M, int64_t N, int64_t K,
                          int64_t group_size, int dtype, void* workspace, size_t workspace_bytes,
                          void* const* peer_buffers, int rank, int world, size_t slot_offset, size_t slot_bytes,
                          void* stream);
int nqb200_peer_allreduce(void* const* peer_buffers, int rank, int world, size_t slot_offset, void* out,
                          const void* bias, int bias_dtype, int64_t M, int64_t N, int dtype, void* stream);
/* The same sum for large messages (prefill-sized partial results: megabytes), in two shots: every rank
 * adds its slice (1 / world of the message) of all ranks' partial results at `in_offset`, leaves the 16-bit
 * sums in its slot at `result_offset`, and after a second barrier reads the other ranks' slices from their
 * result slots: 2 (world - 1) / world of the message crosses NVLink per rank instead of world - 1 times
 * it.  Same rules as nqb200_peer_allreduce; the result slots must alternate between two offsets from call
 * to call (a peer may still be reading the previous one), the slot at `in_offset` may be the same every
 * time.  No counterpart in the reference (single GPU). */
int nqb200_peer_allreduce_large(void* const* peer_buffers, int rank, int world, size_t in_offset, size_t result_offset,
                                void* out, const void* bias, int bias_dtype, int64_t M, int64_t N, int dtype,
                                void* stream);

/* Waits for `stream`, then returns the status the kernels recorded in this
 * workspace: NQB200_OK, or NQB200_ERR_WAIT_TIMEOUT if a bounded device-side wait
 * (an mbarrier or a tile counter) gave up; the record is cleared.  The kernels
 * never trap or spin without limit; this is how the host learns of a give-up.
 * No counterpart in the reference (its Triton kernels have no waits). */
int nqb200_workspace_status(void* workspace, size_t workspace_bytes, void* stream);

/* Name of the kernel family nqb200_gemm would pick for this problem
 * ("decode_stream", "decode_mma", "prefill_tcgen05", "generic"); for logs and tests. */
const char* nqb200_gemm_kernel_name(int64_t M, int64_t N, int64_t K, int64_t group_size, int dtype);

/* Kernels one nqb200_gemm call launches for this problem: 1, or 2 when K is split across CTAs
 * and a small second kernel adds the partial sums; 0 for an invalid or empty problem. */
int nqb200_gemm_launch_count(int64_t M, int64_t N, int64_t K, int64_t group_size, int dtype);

#ifdef __cplusplus
}
#endif
#endif /* NQB200_H */
