// Backward of the sparse MLA attention: the two memory-bound steps around the dense products.
//
//   p[t,h,j]  = exp(scale * s[t,h,j] - lse[t,h])   for valid j, else 0      (probabilities rebuilt from the
//   ds[t,h,j] = p * (dp[t,h,j] - delta[t,h]) * scale                           saved log-sum-exp, no second softmax)
//
//   d_latent[idx[t,j], :] += d_sel_qk[t,j,:] (576 wide)  +  d_sel_v[t,j,:] (first 512 columns)
//
// s = q . k and dp = d_ctx . v come from library GEMMs on the gathered rows; so do the products that
// turn ds and p into d_q and the per-(query, key) row gradients d_sel_*.  The first kernel is one pass over
// [t, h, j] (the same done with framework element-wise operations takes five); the second accumulates a
// million 576-wide rows per query chunk into fp32 with 16-byte vector reductions, reading the two bf16
// sources once (the reference's autograd does this scatter in bf16, where rows selected by thousands of
// queries lose every digit).  Follows OpenDSA/opendsa/ops/sparse_mla.py:39-43 differentiated by hand.
#include <cuda_bf16.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __low2float(h[i]);
      v[2 * i + 1] = __high2float(h[i]);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 x;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = x;
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};

// one CTA per (t, h) row; its threads walk the K / 8 column groups
template <typename T>
__global__ void __launch_bounds__(256) attn_bwd_pointwise_kernel(const T* __restrict__ s, const T* __restrict__ dp,
                                                                 const float* __restrict__ lse,
                                                                 const float* __restrict__ delta,
                                                                 const int32_t* __restrict__ indices,
                                                                 const int32_t* __restrict__ q_pos, int H, int K,
                                                                 float scale, T* __restrict__ p_out,
                                                                 T* __restrict__ ds_out) {
  const int64_t row = blockIdx.x;                 // t * H + h
  const int t = static_cast<int>(row / H);
  const float l = lse[row], dl = delta[row];
  const int qp = q_pos[t];
  const bool row_ok = (l - l) == 0.f;             // finite log-sum-exp (a query without keys has -inf)
  for (int j8 = threadIdx.x; j8 * 8 < K; j8 += blockDim.x) {
    const int j = j8 * 8;
    float sv[8], dv[8], pv[8], gv[8];
    Vec8<T>::load(s + row * K + j, sv);
    Vec8<T>::load(dp + row * K + j, dv);
    const int4 i0 = *reinterpret_cast<const int4*>(indices + static_cast<int64_t>(t) * K + j);
    const int4 i1 = *reinterpret_cast<const int4*>(indices + static_cast<int64_t>(t) * K + j + 4);
    const int id[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const bool ok = row_ok && id[u] >= 0 && id[u] <= qp;
      pv[u] = ok ? __expf(sv[u] * scale - l) : 0.f;
      gv[u] = pv[u] * (dv[u] - dl) * scale;
    }
    Vec8<T>::store(p_out + row * K + j, pv);
    Vec8<T>::store(ds_out + row * K + j, gv);
  }
}

__device__ __forceinline__ void red_add_v4(float* dst, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
  v[0] = __low2float(h[0]); v[1] = __high2float(h[0]); v[2] = __low2float(h[1]); v[3] = __high2float(h[1]);
}
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}

// One group of width/4 threads per source row, two rows per CTA pass; rows whose index is negative, beyond
// the query's position or outside the destination are skipped (their contributions are zero by construction).
template <typename T>
__global__ void __launch_bounds__(288) scatter_add_rows_kernel(float* __restrict__ dst, int64_t n_dst,
                                                               const T* __restrict__ a, const T* __restrict__ b,
                                                               const int32_t* __restrict__ indices,
                                                               const int32_t* __restrict__ q_pos, int64_t n_src,
                                                               int K, int32_t* __restrict__ status) {
  constexpr int kW = 576, kWb = 512, kLanes = kW / 4;      // 144 threads per row
  const int sub = threadIdx.x / kLanes, c4 = (threadIdx.x - sub * kLanes) * 4;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * 2 + sub; r < n_src; r += static_cast<int64_t>(gridDim.x) * 2) {
    const int idx = __ldg(indices + r);
    if (idx < 0 || idx > __ldg(q_pos + r / K)) continue;
    if (idx >= n_dst) {
      if (c4 == 0) atomicMax(status, kDevBadIndex);
      continue;
    }
    float v[4];
    load4<T>(a + r * kW + c4, v);
    if (b != nullptr && c4 < kWb) {
      float w[4];
      load4<T>(b + r * kWb + c4, w);
      v[0] += w[0]; v[1] += w[1]; v[2] += w[2]; v[3] += w[3];
    }
    red_add_v4(dst + static_cast<int64_t>(idx) * kW + c4, v[0], v[1], v[2], v[3]);
  }
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_sparse_attn_bwd_pointwise(const void* s, const void* dp, int32_t is_bf16, const float* lse,
                                                 const float* delta, const int32_t* indices, const int32_t* q_pos,
                                                 int32_t n_queries, int32_t n_heads, int32_t n_idx, float scale,
                                                 void* p_out, void* ds_out, void* stream) {
  if (n_queries == 0 || n_heads == 0 || n_idx == 0) return B200DSA_OK;
  if (!s || !dp || !lse || !delta || !indices || !q_pos || !p_out || !ds_out || n_queries < 0 || n_heads < 1 ||
      n_idx < 0 || (n_idx & 7) || static_cast<int64_t>(n_queries) * n_heads > 0x7fffffff) {
    set_last_error("b200dsa_sparse_attn_bwd_pointwise: bad argument (n_idx a multiple of 8)");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(dp) | reinterpret_cast<uintptr_t>(p_out) |
       reinterpret_cast<uintptr_t>(ds_out) | reinterpret_cast<uintptr_t>(indices)) & 15) {
    set_last_error("b200dsa_sparse_attn_bwd_pointwise: buffers must be 16-byte aligned");
    return B200DSA_EALIGN;
  }
  dim3 grid(static_cast<unsigned>(n_queries) * static_cast<unsigned>(n_heads));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    attn_bwd_pointwise_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(s), static_cast<const __nv_bfloat16*>(dp), lse, delta, indices, q_pos, n_heads,
        n_idx, scale, static_cast<__nv_bfloat16*>(p_out), static_cast<__nv_bfloat16*>(ds_out));
  else
    attn_bwd_pointwise_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(s), static_cast<const float*>(dp),
                                                          lse, delta, indices, q_pos, n_heads, n_idx, scale,
                                                          static_cast<float*>(p_out), static_cast<float*>(ds_out));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_scatter_add_latent_rows(float* d_latent, int64_t n_latent_rows, const void* rows_qk,
                                               const void* rows_v, int32_t is_bf16, const int32_t* indices,
                                               const int32_t* q_pos, int32_t n_queries, int32_t n_idx,
                                               int32_t* status, void* stream) {
  if (n_queries == 0 || n_idx == 0) return B200DSA_OK;
  if (!d_latent || !rows_qk || !indices || !q_pos || !status || n_latent_rows < 1 || n_queries < 0 || n_idx < 0) {
    set_last_error("b200dsa_scatter_add_latent_rows: bad argument");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(d_latent) | reinterpret_cast<uintptr_t>(rows_qk) | reinterpret_cast<uintptr_t>(rows_v)) & 15) {
    set_last_error("b200dsa_scatter_add_latent_rows: buffers must be 16-byte aligned");
    return B200DSA_EALIGN;
  }
  const int64_t n_src = static_cast<int64_t>(n_queries) * n_idx;
  const int grid = static_cast<int>(n_src / 2 + 1 < 148 * 16 ? n_src / 2 + 1 : 148 * 16);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    scatter_add_rows_kernel<__nv_bfloat16><<<grid, 288, 0, st>>>(d_latent, n_latent_rows,
                                                                static_cast<const __nv_bfloat16*>(rows_qk),
                                                                static_cast<const __nv_bfloat16*>(rows_v), indices, q_pos,
                                                                n_src, n_idx, status);
  else
    scatter_add_rows_kernel<float><<<grid, 288, 0, st>>>(d_latent, n_latent_rows, static_cast<const float*>(rows_qk),
                                                        static_cast<const float*>(rows_v), indices, q_pos, n_src, n_idx,
                                                        status);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
