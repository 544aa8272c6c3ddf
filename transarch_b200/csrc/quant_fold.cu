// Index-query quantisation with the scale folded into the head weights:
//   scale[t,h] = max(amax_d |q[t,h,d]|, 1e-10) / 448, rounded UP to a power of two when the
//   "ue8m0" scale format is asked for;  q_fp8 = e4m3(q / scale)  (round to nearest even)
//   weights[t,h] = w[t,h] * scale[t,h] * fold
// so that  sum_h weights * relu(<q_fp8, k_fp8>) * k_scale  equals the unquantised score up to
// FP8 rounding.  One warp per (t, h) row of 128 values, four per lane.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

// Smallest power of two that is >= x (x positive and finite): the "ue8m0" scale format, i.e.
// exp2(ceil(log2(x))) evaluated exactly on the bit pattern instead of through log2f / exp2f.
__device__ __forceinline__ float pow2_round_up(float x) {
  const uint32_t u = __float_as_uint(x);
  uint32_t e = u >> 23;
  if (e == 0) return 1.17549435e-38f;          // subnormal input: the smallest normal power of two
  if (u & 0x7fffffu) ++e;
  return __uint_as_float(e << 23);
}

__global__ void __launch_bounds__(256) quant_q_fold_kernel(const __nv_bfloat16* __restrict__ q,
                                                           const float* __restrict__ w, int64_t n_rows, float fold,
                                                           int use_ue8m0, uint8_t* __restrict__ q_fp8,
                                                           float* __restrict__ weights) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(q + row * 128) + lane);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float x[4] = {__low2float(a), __high2float(a), __low2float(b), __high2float(b)};
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float scale = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
  if (use_ue8m0) scale = pow2_round_up(scale);
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float y = fminf(fmaxf(__fdiv_rn(x[j], scale), -448.0f), 448.0f);
    packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
  }
  reinterpret_cast<uint32_t*>(q_fp8 + row * 128)[lane] = packed;
  if (lane == 0) weights[row] = __ldg(w + row) * scale * fold;
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_quant_q_fold_weights(const void* q_bf16, const float* w, int64_t n_rows, float fold,
                                            int32_t use_ue8m0, void* q_fp8, float* weights, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!q_bf16 || !w || !q_fp8 || !weights || n_rows < 0) {
    set_last_error("b200dsa_quant_q_fold_weights: bad argument");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(q_bf16) & 7) || (reinterpret_cast<uintptr_t>(q_fp8) & 3)) {
    set_last_error("b200dsa_quant_q_fold_weights: q must be 8-byte and q_fp8 4-byte aligned");
    return B200DSA_EALIGN;
  }
  const unsigned grid = static_cast<unsigned>((n_rows + 7) / 8);
  cudaError_t e_launch = launch_chained(quant_q_fold_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(q_bf16), w, n_rows, fold, static_cast<int>(use_ue8m0 != 0),
      static_cast<uint8_t*>(q_fp8), weights);
  cudaError_t e = e_launch != cudaSuccess ? e_launch : cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

// Index-key insert: quantise each new key row to e4m3 with a per-token scale (max(amax, 1e-4)/448,
// rounded up to a power of two for the "ue8m0" scale format) and write it into
// its slot of the paged cache (page = P*128 fp8 bytes then P fp32 scales).  One warp per token.
namespace b200dsa {

__global__ void __launch_bounds__(256) k_quant_and_cache_kernel(const __nv_bfloat16* __restrict__ k,
                                                                const int64_t* __restrict__ slot_mapping,
                                                                int64_t n_tokens, int page_size, int64_t num_pages,
                                                                int use_ue8m0, uint8_t* __restrict__ cache,
                                                                int32_t* __restrict__ status) {
  const int64_t tok = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (tok >= n_tokens) return;
  const int lane = threadIdx.x & 31;
  const int64_t slot = slot_mapping[tok];
  if (slot < 0) return;  // padding token
  const int64_t page = slot / page_size;
  const int off = static_cast<int>(slot - page * page_size);
  if (page >= num_pages) {
    if (lane == 0) atomicMax(status, kDevBadIndex);
    return;
  }
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(k + tok * 128) + lane);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float x[4] = {__low2float(a), __high2float(a), __low2float(b), __high2float(b)};
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float scale = __fdiv_rn(fmaxf(amax, 1e-4f), 448.0f);
  if (use_ue8m0) scale = pow2_round_up(scale);
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float y = fminf(fmaxf(__fdiv_rn(x[j], scale), -448.0f), 448.0f);
    packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
  }
  uint8_t* pg = cache + page * (static_cast<int64_t>(page_size) * 132);
  reinterpret_cast<uint32_t*>(pg + off * 128)[lane] = packed;
  if (lane == 0) reinterpret_cast<float*>(pg + page_size * 128)[off] = scale;
}

}  // namespace b200dsa

extern "C" int b200dsa_indexer_k_quant_and_cache(const void* k_bf16, const int64_t* slot_mapping, int64_t n_tokens,
                                                 void* cache, int64_t num_pages, int32_t page_size,
                                                 int32_t use_ue8m0, int32_t* status, void* stream) {
  if (n_tokens == 0) return B200DSA_OK;
  if (!k_bf16 || !slot_mapping || !cache || !status || n_tokens < 0 || num_pages < 1 || page_size < 1 ||
      (page_size & 3)) {
    b200dsa::set_last_error("b200dsa_indexer_k_quant_and_cache: bad argument (page_size must be a multiple of 4)");
    return B200DSA_EINVAL;
  }
  const unsigned grid = static_cast<unsigned>((n_tokens + 7) / 8);
  b200dsa::k_quant_and_cache_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(k_bf16), slot_mapping, n_tokens, page_size, num_pages,
      static_cast<int>(use_ue8m0 != 0), static_cast<uint8_t*>(cache), status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    b200dsa::set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
