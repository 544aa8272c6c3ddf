// Log-sum-exp combine of attention partials computed over disjoint key shards.
//
//   m = max_r lse_r;  w_r = exp(lse_r - m);  out = sum_r w_r * ctx_r / sum_r w_r;
//   lse_out = m + log(sum_r w_r).  Rows whose every partial is empty (lse = -inf) give 0 / -inf.
// One CTA of 128 threads per (item, head) row; each thread owns 4 of the 512 value dims.
#include <cuda_bf16.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kCombineDv = 512;
constexpr int kCombineMaxParts = 64;

__global__ void __launch_bounds__(128) lse_combine_kernel(const float* __restrict__ ctx_parts,
                                                          const float* __restrict__ lse_parts, int n_parts,
                                                          int64_t n_rows, float* __restrict__ ctx_out,
                                                          float* __restrict__ lse_out) {
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x;
  float m = -INFINITY;
  for (int r = 0; r < n_parts; ++r) m = fmaxf(m, __ldg(lse_parts + r * n_rows + row));
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.f;
  if (m != -INFINITY) {
    for (int r = 0; r < n_parts; ++r) {
      const float l = __ldg(lse_parts + r * n_rows + row);
      if (l == -INFINITY) continue;
      const float w = expf(l - m);
      const float4 v = __ldg(reinterpret_cast<const float4*>(ctx_parts + (r * n_rows + row) * kCombineDv) + tid);
      acc.x = fmaf(w, v.x, acc.x);
      acc.y = fmaf(w, v.y, acc.y);
      acc.z = fmaf(w, v.z, acc.z);
      acc.w = fmaf(w, v.w, acc.w);
      den += w;
    }
    const float inv = 1.0f / den;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
  }
  reinterpret_cast<float4*>(ctx_out + row * kCombineDv)[tid] = acc;
  if (tid == 0 && lse_out) lse_out[row] = (m == -INFINITY) ? -INFINITY : m + logf(den);
}

// All-reduce form of the same merge: after a MAX all-reduce of lse gives m, every rank
// contributes ctx * exp(lse - m) and exp(lse - m); a SUM all-reduce (or reduce-scatter) of the
// 516-wide rows (512 values, the weight, 3 pad) follows and `finalize` divides.
constexpr int kWireRow = 516;

__global__ void __launch_bounds__(128) lse_prescale_kernel(const float* __restrict__ ctx, const float* __restrict__ lse,
                                                           const float* __restrict__ lse_max,
                                                           float* __restrict__ wire) {
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x;
  const float l = __ldg(lse + row), m = __ldg(lse_max + row);
  const float w = (l == -INFINITY || m == -INFINITY) ? 0.f : expf(l - m);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (w != 0.f) {
    v = __ldg(reinterpret_cast<const float4*>(ctx + row * kCombineDv) + tid);
    v.x *= w; v.y *= w; v.z *= w; v.w *= w;
  }
  reinterpret_cast<float4*>(wire + row * kWireRow)[tid] = v;
  if (tid == 0) reinterpret_cast<float4*>(wire + row * kWireRow)[128] = make_float4(w, 0.f, 0.f, 0.f);
}

__global__ void __launch_bounds__(128) lse_finalize_kernel(const float* __restrict__ wire,
                                                           const float* __restrict__ lse_max,
                                                           float* __restrict__ ctx_out, float* __restrict__ lse_out) {
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x;
  const float den = __ldg(wire + row * kWireRow + kCombineDv);
  float4 v = __ldg(reinterpret_cast<const float4*>(wire + row * kWireRow) + tid);
  const float inv = den > 0.f ? 1.0f / den : 0.f;
  v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
  reinterpret_cast<float4*>(ctx_out + row * kCombineDv)[tid] = v;
  if (tid == 0 && lse_out) lse_out[row] = den > 0.f ? __ldg(lse_max + row) + logf(den) : -INFINITY;
}

// Per row: move the positions that fall into [pos_lo, pos_hi) to the front (order kept), fill the
// rest with -1 and report how many there are.  One CTA of 256 threads per row.
__global__ void __launch_bounds__(256) compact_owned_kernel(const int32_t* __restrict__ idx, int64_t idx_stride, int n_idx,
                                                            int pos_lo, int pos_hi, int32_t* __restrict__ out,
                                                            int64_t out_stride, int32_t* __restrict__ count) {
  pdl_launch_dependents();
  pdl_wait_prior();
  __shared__ int s_warp[8];
  __shared__ int s_base;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* src = idx + row * idx_stride;
  int32_t* dst = out + row * out_stride;
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int j0 = 0; j0 < n_idx; j0 += 256) {
    const int j = j0 + tid;
    const int v = (j < n_idx) ? src[j] : -1;
    const bool own = v >= pos_lo && v < pos_hi;
    const unsigned m = __ballot_sync(0xffffffffu, own);
    if (lane == 0) s_warp[warp] = __popc(m);
    __syncthreads();
    int off = s_base;
    for (int w = 0; w < warp; ++w) off += s_warp[w];
    if (own) dst[off + __popc(m & ((1u << lane) - 1))] = v;
    __syncthreads();
    if (tid == 0) {
      int t = 0;
      for (int w = 0; w < 8; ++w) t += s_warp[w];
      s_base += t;
    }
    __syncthreads();
  }
  const int total = s_base;
  for (int j = total + tid; j < n_idx; j += 256) dst[j] = -1;
  if (tid == 0) count[row] = total;
}

// Compact wire form: with every rank's lse gathered first (tiny), a rank knows the common
// maximum and the exact denominator, so it contributes its normalised share
//   out = bf16( ctx * exp(lse_me - m) / sum_r exp(lse_r - m) )
// and a single SUM all-reduce of the bf16 rows yields the merged context directly.
__global__ void __launch_bounds__(128) lse_prescale_norm_kernel(const float* __restrict__ ctx,
                                                                const float* __restrict__ lse_all, int n_parts,
                                                                int my_part, int64_t n_rows,
                                                                __nv_bfloat16* __restrict__ out,
                                                                float* __restrict__ lse_out) {
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x;
  float m = -INFINITY;
  for (int r = 0; r < n_parts; ++r) m = fmaxf(m, __ldg(lse_all + r * n_rows + row));
  float den = 0.f, mine = 0.f;
  if (m != -INFINITY) {
    for (int r = 0; r < n_parts; ++r) {
      const float l = __ldg(lse_all + r * n_rows + row);
      const float w = (l == -INFINITY) ? 0.f : expf(l - m);
      den += w;
      if (r == my_part) mine = w;
    }
  }
  const float w = den > 0.f ? mine / den : 0.f;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (w != 0.f) v = __ldg(reinterpret_cast<const float4*>(ctx + row * kCombineDv) + tid);
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x * w, v.y * w);
  __nv_bfloat162 b = __floats2bfloat162_rn(v.z * w, v.w * w);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t*>(&a);
  packed.y = *reinterpret_cast<uint32_t*>(&b);
  reinterpret_cast<uint2*>(out + row * kCombineDv)[tid] = packed;
  if (tid == 0 && lse_out) lse_out[row] = den > 0.f ? m + logf(den) : -INFINITY;
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_lse_combine(const float* ctx_parts, const float* lse_parts, int32_t n_parts, int64_t n_rows,
                                   float* ctx_out, float* lse_out, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!ctx_parts || !lse_parts || !ctx_out || n_parts < 1 || n_parts > kCombineMaxParts || n_rows < 0) {
    set_last_error("b200dsa_lse_combine: bad argument (1 <= n_parts <= 64)");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(ctx_parts) & 15) || (reinterpret_cast<uintptr_t>(ctx_out) & 15)) {
    set_last_error("b200dsa_lse_combine: ctx buffers must be 16-byte aligned");
    return B200DSA_EALIGN;
  }
  lse_combine_kernel<<<static_cast<unsigned>(n_rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ctx_parts, lse_parts, n_parts, n_rows, ctx_out, lse_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_lse_prescale(const float* ctx, const float* lse, const float* lse_max, int64_t n_rows,
                                    float* wire, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!ctx || !lse || !lse_max || !wire || n_rows < 0 || (reinterpret_cast<uintptr_t>(ctx) & 15) ||
      (reinterpret_cast<uintptr_t>(wire) & 15)) {
    set_last_error("b200dsa_lse_prescale: bad argument or buffers not 16-byte aligned");
    return B200DSA_EINVAL;
  }
  lse_prescale_kernel<<<static_cast<unsigned>(n_rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(ctx, lse, lse_max,
                                                                                                    wire);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_lse_finalize(const float* wire, const float* lse_max, int64_t n_rows, float* ctx_out,
                                    float* lse_out, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!wire || !lse_max || !ctx_out || n_rows < 0 || (reinterpret_cast<uintptr_t>(ctx_out) & 15) ||
      (reinterpret_cast<uintptr_t>(wire) & 15)) {
    set_last_error("b200dsa_lse_finalize: bad argument or buffers not 16-byte aligned");
    return B200DSA_EINVAL;
  }
  lse_finalize_kernel<<<static_cast<unsigned>(n_rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(wire, lse_max,
                                                                                                    ctx_out, lse_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_compact_owned(const int32_t* indices, int64_t idx_stride, int32_t n_rows, int32_t n_idx,
                                     int32_t pos_lo, int32_t pos_hi, int32_t* out, int64_t out_stride,
                                     int32_t* count, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!indices || !out || !count || n_rows < 0 || n_idx < 0 || idx_stride < n_idx || out_stride < n_idx ||
      indices == out) {
    set_last_error("b200dsa_compact_owned: bad argument (out must not alias indices)");
    return B200DSA_EINVAL;
  }
  cudaError_t e = launch_chained(compact_owned_kernel, dim3(n_rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                 indices, idx_stride, n_idx, pos_lo, pos_hi, out, out_stride, count);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_lse_prescale_norm(const float* ctx, const float* lse_all, int32_t n_parts, int32_t my_part,
                                         int64_t n_rows, void* out_bf16, float* lse_out, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!ctx || !lse_all || !out_bf16 || n_parts < 1 || n_parts > kCombineMaxParts || my_part < 0 ||
      my_part >= n_parts || n_rows < 0 || (reinterpret_cast<uintptr_t>(ctx) & 15) ||
      (reinterpret_cast<uintptr_t>(out_bf16) & 7)) {
    set_last_error("b200dsa_lse_prescale_norm: bad argument (1 <= n_parts <= 64, 0 <= my_part < n_parts, aligned buffers)");
    return B200DSA_EINVAL;
  }
  lse_prescale_norm_kernel<<<static_cast<unsigned>(n_rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ctx, lse_all, n_parts, my_part, n_rows, static_cast<__nv_bfloat16*>(out_bf16), lse_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
