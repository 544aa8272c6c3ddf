// Value up-projection after the latent-space attention: out[t, h, :] = ctx[t, h, :] @ W_UV[h]^T,
// a batch of per-head GEMMs [T x 512] x [512 x Dv] on tcgen05.
//
// CTA (token tile of 128, head): tokens are the UMMA M dimension (one TMEM lane per token), the Dv
// value dims are N (rounded up to a multiple of 16; rows of W_UV beyond Dv are zero-filled by TMA), the
// 512 latent dims are K, streamed as eight 64-element chunks through a 4-stage ring.  Both operands are
// K-major rows of 128 bytes written by TMA with the 128-byte swizzle.  Roles: warp 0 issues the loads,
// warp 1 the MMAs, warps 2-5 read the accumulator (thread = token) and store bf16 or fp32 rows.
// The kernel moves W_UV once per token tile (16.8 MB at 128 heads x 128 x 512) and is bound by that read.
#include <cuda_bf16.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kWuvThreads = 192;
constexpr int kWuvStages = 4;
constexpr int kWuvK = 512;
constexpr int kWuvChunks = kWuvK / 64;
constexpr int kWuvABytes = 128 * 128;          // 128 tokens x 64 bf16
constexpr int kWuvBBytes = 256 * 128;          // up to 256 value rows x 64 bf16
constexpr int kWuvSmem = kWuvStages * (kWuvABytes + kWuvBBytes) + 1024 + 256;

struct WuvParams {
  int32_t n_tokens, n_heads, dv, n_pad;   // n_pad = dv rounded up to 16
  void* out;                               // [n_tokens, n_heads, dv] bf16 or fp32
  int out_f32;
  int32_t* status;
};

__global__ void __launch_bounds__(kWuvThreads, 1)
wuv_proj_kernel(const __grid_constant__ CUtensorMap tmap_ctx, const __grid_constant__ CUtensorMap tmap_w,
                const WuvParams p) {
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + kWuvStages * (kWuvABytes + kWuvBBytes));
  uint64_t* full = bars;                 // [stages]
  uint64_t* empty = bars + kWuvStages;   // [stages]
  uint64_t* acc_full = empty + kWuvStages;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = blockIdx.x * 128, head = blockIdx.y;
  volatile int* abort_flag = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < kWuvStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&s_tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const uint32_t b_bytes = static_cast<uint32_t>(p.n_pad) * 128;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_ctx);
      tma_prefetch_desc(&tmap_w);
    }
    for (int c = 0; c < kWuvChunks; ++c) {
      const int s = c % kWuvStages;
      const bool ok = mbar_wait(&empty[s], ((c / kWuvStages) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) break;
      if (elect_one()) {
        uint8_t* a = smem_al + s * (kWuvABytes + kWuvBBytes);
        mbar_arrive_expect_tx(&full[s], kWuvABytes + b_bytes);
        tma_load_3d(a, &tmap_ctx, &full[s], c * 64, head, t0);             // rows beyond n_tokens: zeros
        tma_load_3d(a + kWuvABytes, &tmap_w, &full[s], c * 64, 0, head);   // rows beyond dv: zeros
      }
    }
  } else if (warp == 1) {
    const uint32_t idesc = make_idesc(kFmtBF16, kFmtBF16, 128, static_cast<uint32_t>(p.n_pad));
    for (int c = 0; c < kWuvChunks; ++c) {
      const int s = c % kWuvStages;
      const bool ok = mbar_wait(&full[s], (c / kWuvStages) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_addr = smem_base + s * (kWuvABytes + kWuvBBytes);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_f16_ss(tmem_base, make_desc_k_sw128(a_addr + kk * 32), make_desc_k_sw128(a_addr + kWuvABytes + kk * 32),
                     idesc, (c | kk) != 0);
        tc_commit(&empty[s]);
        if (c == kWuvChunks - 1) tc_commit(acc_full);
      }
      __syncwarp();
    }
  } else {
    const int lane_base = (warp & 3) * 32;
    const int tok = t0 + lane_base + lane;
    const bool ok = mbar_wait(acc_full, 0, abort_flag);
    if (__all_sync(0xffffffffu, ok)) {
      tc_fence_after();
      const int64_t row_off = (static_cast<int64_t>(tok) * p.n_heads + head) * p.dv;
      for (int n0 = 0; n0 < p.n_pad; n0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(lane_base) << 16) + n0, v);
        tc_wait_ld();
        if (tok < p.n_tokens) {
          if (p.out_f32) {
            float* o = static_cast<float*>(p.out) + row_off + n0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.dv) o[j] = __uint_as_float(v[j]);
          } else {
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + row_off + n0;
            if (n0 + 32 <= p.dv && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 w;
                __nv_bfloat162 h;
                h = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1])); w.x = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])); w.y = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5])); w.z = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7])); w.w = *reinterpret_cast<uint32_t*>(&h);
                *reinterpret_cast<uint4*>(o + j) = w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.dv) o[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
            }
          }
        }
      }
      tc_fence_before();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 256);
  if (tid == 0 && s_abort) atomicMax(p.status, kDevWaitTimeout);
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_wuv_up_project(const void* ctx_bf16, const void* w_uv_bf16, int32_t n_tokens, int32_t n_heads,
                                      int32_t dv, void* out, int32_t out_f32, int32_t* status, void* stream) {
  if (n_tokens == 0) return B200DSA_OK;
  if (!ctx_bf16 || !w_uv_bf16 || !out || !status || n_tokens < 0 || n_heads < 1 || dv < 1 || dv > 256) {
    set_last_error("b200dsa_wuv_up_project: bad argument (1 <= dv <= 256)");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(ctx_bf16) & 15) || (reinterpret_cast<uintptr_t>(w_uv_bf16) & 15)) {
    set_last_error("b200dsa_wuv_up_project: ctx and W_UV must be 16-byte aligned");
    return B200DSA_EALIGN;
  }
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return B200DSA_ECUDA;
  const int n_pad = (dv + 15) / 16 * 16;
  CUtensorMap mc, mw;
  cuuint32_t es[3] = {1, 1, 1};
  {
    cuuint64_t dims[3] = {512, static_cast<cuuint64_t>(n_heads), static_cast<cuuint64_t>(n_tokens)};
    cuuint64_t strides[2] = {512 * 2, static_cast<cuuint64_t>(n_heads) * 512 * 2};
    cuuint32_t box[3] = {64, 1, 128};
    if (enc(&mc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ctx_bf16), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      set_last_error("b200dsa_wuv_up_project: cuTensorMapEncodeTiled rejected ctx");
      return B200DSA_ECUDA;
    }
  }
  {
    cuuint64_t dims[3] = {512, static_cast<cuuint64_t>(dv), static_cast<cuuint64_t>(n_heads)};
    cuuint64_t strides[2] = {512 * 2, static_cast<cuuint64_t>(dv) * 512 * 2};
    cuuint32_t box[3] = {64, static_cast<cuuint32_t>(n_pad), 1};
    if (enc(&mw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w_uv_bf16), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      set_last_error("b200dsa_wuv_up_project: cuTensorMapEncodeTiled rejected W_UV");
      return B200DSA_ECUDA;
    }
  }
  cudaError_t e = cudaFuncSetAttribute(wuv_proj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWuvSmem);
  WuvParams p{n_tokens, n_heads, dv, n_pad, out, out_f32, status};
  if (e == cudaSuccess)
    e = launch_chained(wuv_proj_kernel, dim3((n_tokens + 127) / 128, n_heads), dim3(kWuvThreads), kWuvSmem,
                       static_cast<cudaStream_t>(stream), mc, mw, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
