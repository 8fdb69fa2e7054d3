// The elementwise steps either side of the linears in a Qwen3 block, one kernel
// each instead of the 5-10 small launches PyTorch needs: residual add + RMSNorm,
// per-head QK-norm + rotary embedding, SiLU(gate) * up.  At decode these launches
// cost as much as the GEMVs.  Roundings follow the reference modules exactly
// (nanoquantization/layers/norm.py:18-32, layers/rope.py:24-45,
// models/qwen3_quantized.py:150,213-214): fp32 inside, one rounding to the
// 16-bit type wherever the reference materialises a 16-bit tensor.
#include "common.cuh"

namespace nqb200 {

template <bool BF16> __device__ __forceinline__ float rnd16(float v) { return raw16_to_float<BF16>(float_to_raw16<BF16>(v)); }

// One CTA per token.  h = x (+ residual), rounded; residual_out = h; out = (round16(h * rsqrt(mean(h^2)+eps))) * w.
template <bool BF16>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const uint16_t* __restrict__ x, const uint16_t* residual,
                                                          const uint16_t* __restrict__ weight, uint16_t* __restrict__ out,
                                                          uint16_t* residual_out, int H, float eps) {
  extern __shared__ float hbuf[];  // H floats
  __shared__ float red[8];
  grid_launch_dependents();  // the next kernel's weight fetch may start now
  grid_dependency_wait();    // x and residual come from the kernel ahead
  const size_t row = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float h = raw16_to_float<BF16>(x[row + i]);
    if (residual) h = rnd16<BF16>(h + raw16_to_float<BF16>(residual[row + i]));
    if (residual_out) residual_out[row + i] = float_to_raw16<BF16>(h);
    hbuf[i] = h;
    ss += h * h;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float inv = rsqrtf(tot / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[row + i] = float_to_raw16<BF16>(rnd16<BF16>(hbuf[i] * inv) * raw16_to_float<BF16>(weight[i]));
}

// One warp per (token, head) of q and k inside a fused [T, (Hq + 2*Hkv) * D] buffer, D = 128, in place:
// RMSNorm over the head (weight qw / kw), then the half-split rotation with the fp32 cos|sin table row
// of the token's position.  v is untouched.  With a paged cache given ([slots, Hkv, D] for k and for v,
// slot_of[t] = the token's slot), the rotated k and the v of every token are also stored there by
// the warps that hold them, which saves the two scatter launches that would follow.
template <bool BF16>
__global__ void __launch_bounds__(256) qknorm_rope_kernel(uint16_t* __restrict__ qkv, const uint16_t* __restrict__ qw,
                                                          const uint16_t* __restrict__ kw, const float* __restrict__ cos_sin,
                                                          const int64_t* __restrict__ positions, int T, int Hq, int Hkv,
                                                          int row_stride, float eps, const int64_t* __restrict__ slot_of,
                                                          uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache) {
  constexpr int D = 128;
  grid_launch_dependents();
  grid_dependency_wait();
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = Hq + Hkv + (slot_of ? Hkv : 0);  // with a cache, the v heads get a warp each too
  if (gw >= T * heads) return;
  const int t = gw / heads, hd = gw % heads;
  uint16_t* p = qkv + (size_t)t * row_stride + (size_t)hd * D;  // q heads first, then k heads, then v heads
  if (hd >= Hq + Hkv) {
    // a v head: 256 bytes to its slot
    uint16_t* dst = v_cache + ((size_t)slot_of[t] * Hkv + (hd - Hq - Hkv)) * D;
    reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(p)[lane];
    return;
  }
  const uint16_t* w = hd < Hq ? qw : kw;
  // lane owns elements lane, lane+32, lane+64, lane+96: (lane, lane+64) and (lane+32, lane+96) are rotation pairs
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = raw16_to_float<BF16>(p[lane + 32 * j]); ss += v[j] * v[j]; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    v[j] = rnd16<BF16>(rnd16<BF16>(v[j] * inv) * raw16_to_float<BF16>(w[lane + 32 * j]));
  const float* cs = cos_sin + (size_t)positions[t] * D;  // [cos(64) | sin(64)]
  uint16_t* kdst = (slot_of && hd >= Hq) ? k_cache + ((size_t)slot_of[t] * Hkv + (hd - Hq)) * D : nullptr;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int i = lane + 32 * j;
    const float c = cs[i], s = cs[64 + i];
    const float a = v[j], b = v[j + 2];
    const uint16_t lo = float_to_raw16<BF16>(a * c - b * s), hi = float_to_raw16<BF16>(a * s + b * c);
    p[i] = lo;
    p[i + 64] = hi;
    if (kdst) { kdst[i] = lo; kdst[i + 64] = hi; }
  }
}

// out[t, i] = round16(silu(gate)) * up, gate = gate_up[t, i], up = gate_up[t, I + i]
template <bool BF16>
__global__ void __launch_bounds__(256) silu_mul_kernel(const uint16_t* __restrict__ gate_up, uint16_t* __restrict__ out,
                                                       int64_t T, int I) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t total = T * (int64_t)I;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = raw16_to_float<BF16>(gate_up[t * 2 * I + i]);
    const float u = raw16_to_float<BF16>(gate_up[t * 2 * I + I + i]);
    const float s = rnd16<BF16>(g / (1.f + expf(-g)));
    out[idx] = float_to_raw16<BF16>(s * u);
  }
}

}  // namespace nqb200

using namespace nqb200;

extern "C" int nqb200_add_rmsnorm(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                                  int64_t T, int64_t H, float eps, int dtype, void* stream) {
  if (T < 0 || H <= 0 || H > 65536) return NQB200_ERR_BAD_SHAPE;
  if (dtype != NQB200_F16 && dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  if (T == 0) return NQB200_OK;
  if (!x || !weight || !out) return NQB200_ERR_NULL_POINTER;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)H * sizeof(float);
  return launch_overlapped(dtype == NQB200_BF16 ? add_rmsnorm_kernel<true> : add_rmsnorm_kernel<false>, dim3((unsigned)T), dim3(256), smem, st,
                           (const uint16_t*)x, (const uint16_t*)residual, (const uint16_t*)weight, (uint16_t*)out,
                           (uint16_t*)residual_out, (int)H, eps);
}

static int qknorm_rope_launch(void* qkv, const void* q_weight, const void* k_weight, const float* cos_sin,
                              const int64_t* positions, const int64_t* slots, void* k_cache, void* v_cache, int64_t T,
                              int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim, int64_t row_stride, float eps,
                              int dtype, void* stream) {
  if (T < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim != 128) return NQB200_ERR_BAD_SHAPE;
  if (dtype != NQB200_F16 && dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  if (T == 0) return NQB200_OK;
  if (!qkv || !q_weight || !k_weight || !cos_sin || !positions) return NQB200_ERR_NULL_POINTER;
  if (slots && (!k_cache || !v_cache)) return NQB200_ERR_NULL_POINTER;
  const int64_t warps = T * (num_q_heads + num_kv_heads + (slots ? num_kv_heads : 0));
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
  return launch_overlapped(dtype == NQB200_BF16 ? qknorm_rope_kernel<true> : qknorm_rope_kernel<false>, dim3(blocks), dim3(256), 0, st,
                           (uint16_t*)qkv, (const uint16_t*)q_weight, (const uint16_t*)k_weight, cos_sin, positions, (int)T,
                           (int)num_q_heads, (int)num_kv_heads, (int)row_stride, eps, slots, (uint16_t*)k_cache, (uint16_t*)v_cache);
}

extern "C" int nqb200_qknorm_rope(void* qkv, const void* q_weight, const void* k_weight, const float* cos_sin,
                                  const int64_t* positions, int64_t T, int64_t num_q_heads, int64_t num_kv_heads,
                                  int64_t head_dim, int64_t row_stride, float eps, int dtype, void* stream) {
  return qknorm_rope_launch(qkv, q_weight, k_weight, cos_sin, positions, nullptr, nullptr, nullptr, T, num_q_heads, num_kv_heads,
                            head_dim, row_stride, eps, dtype, stream);
}

extern "C" int nqb200_qknorm_rope_kv(void* qkv, const void* q_weight, const void* k_weight, const float* cos_sin,
                                     const int64_t* positions, const int64_t* slots, void* k_cache, void* v_cache, int64_t T,
                                     int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim, int64_t row_stride, float eps,
                                     int dtype, void* stream) {
  if (!slots) return NQB200_ERR_NULL_POINTER;
  return qknorm_rope_launch(qkv, q_weight, k_weight, cos_sin, positions, slots, k_cache, v_cache, T, num_q_heads, num_kv_heads,
                            head_dim, row_stride, eps, dtype, stream);
}

extern "C" int nqb200_silu_mul(const void* gate_up, void* out, int64_t T, int64_t I, int dtype, void* stream) {
  if (T < 0 || I <= 0 || I > INT32_MAX) return NQB200_ERR_BAD_SHAPE;
  if (dtype != NQB200_F16 && dtype != NQB200_BF16) return NQB200_ERR_BAD_DTYPE;
  if (T == 0) return NQB200_OK;
  if (!gate_up || !out) return NQB200_ERR_NULL_POINTER;
  const int64_t total = T * I;
  const int64_t want = (total + 255) / 256;
  const unsigned blocks = (unsigned)(want < (int64_t)kNumSMs * 16 ? want : (int64_t)kNumSMs * 16);
  cudaStream_t st = (cudaStream_t)stream;
  return launch_overlapped(dtype == NQB200_BF16 ? silu_mul_kernel<true> : silu_mul_kernel<false>, dim3(blocks), dim3(256), 0, st,
                           (const uint16_t*)gate_up, (uint16_t*)out, T, (int)I);
}
