// Tensor-pipe peak probe: every CTA issues back-to-back tcgen05 FP8 (e4m3 x e4m3 -> fp32) or bf16
// MMAs of shape M=128, N=256 on operands that stay in shared memory, with no global traffic at all.
// What it measures is the denominator of a tensor-pipe roofline for FP8 contractions on this part,
// under the clocks and the power cap the GPU runs at while the pipe is saturated.
#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kPeakThreads = 64;
constexpr int kPeakABytes = 128 * 128;   // 128 rows x 128 bytes (K-major, 128-byte swizzle)
constexpr int kPeakBBytes = 256 * 128;   // 256 rows x 128 bytes
constexpr int kPeakSmem = kPeakABytes + kPeakBBytes + 1024 + 64;

template <bool kFp8>
__global__ void __launch_bounds__(kPeakThreads, 1) mma_peak_kernel(int iters, int32_t* status) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_al + kPeakABytes + kPeakBBytes);
  const int tid = threadIdx.x, warp = tid >> 5;
  // operand bytes: a fixed pseudo-random pattern of small finite values (sign, exponent and mantissa
  // bits all toggle; no NaN encodings)
  for (int i = tid; i < (kPeakABytes + kPeakBBytes) / 4; i += kPeakThreads) {
    uint32_t x = (i + 1) * 2654435761u + blockIdx.x * 40503u;
    x ^= x >> 15;
    reinterpret_cast<uint32_t*>(smem_al)[i] = kFp8 ? (x & 0xB7B7B7B7u) : (x & 0xBF7FBF7Fu);
  }
  if (tid == 0) {
    s_abort = 0;
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&s_tmem_base, 512);
    tmem_relinquish();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  if (warp == 0) {
    constexpr uint32_t idesc = kFp8 ? make_idesc(kFmtE4M3, kFmtE4M3, 128, 256) : make_idesc(kFmtBF16, kFmtBF16, 128, 256);
    if (elect_one()) {
      const uint64_t a0 = make_desc_k_sw128(smem_base);
      const uint64_t b0 = make_desc_k_sw128(smem_base + kPeakABytes);
      for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int acc = 0; acc < 2; ++acc) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {           // 32 bytes of K per instruction
            if constexpr (kFp8) mma_f8f6f4_ss(tmem_base + acc * 256, a0 + 2 * kk, b0 + 2 * kk, idesc, (it | kk) != 0);
            else mma_f16_ss(tmem_base + acc * 256, a0 + 2 * kk, b0 + 2 * kk, idesc, (it | kk) != 0);
          }
        }
      }
      tc_commit(bar);
    }
    __syncwarp();
    if (!mbar_wait(bar, 0, &s_abort) && (tid & 31) == 0) atomicMax(status, kDevWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

// Flops of one launch: ctas * iters * 8 MMAs * 2*128*256*K, K = 32 (fp8) or 16 (bf16).
extern "C" int b200dsa_mma_peak_probe(int32_t fp8, int32_t ctas, int32_t iters, int32_t* status, void* stream) {
  if (ctas < 1 || iters < 1 || iters > (1 << 22) || !status) {
    set_last_error("b200dsa_mma_peak_probe: bad argument");
    return B200DSA_EINVAL;
  }
  cudaError_t e;
  if (fp8) {
    e = cudaFuncSetAttribute(mma_peak_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem);
    if (e == cudaSuccess)
      mma_peak_kernel<true><<<ctas, kPeakThreads, kPeakSmem, static_cast<cudaStream_t>(stream)>>>(iters, status);
  } else {
    e = cudaFuncSetAttribute(mma_peak_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem);
    if (e == cudaSuccess)
      mma_peak_kernel<false><<<ctas, kPeakThreads, kPeakSmem, static_cast<cudaStream_t>(stream)>>>(iters, status);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
