// Measurement kernels.  Tensor-pipe peak probe: every CTA issues back-to-back tcgen05 FP8 (e4m3 x e4m3 ->
// fp32) or bf16 MMAs of shape M=128, N=256 on operands that stay in shared memory, with no global traffic at all.
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

// The same loop for one bf16 instruction shape: M = 64 or 128, N, the A operand read from shared memory
// (SS) or from tensor memory (TS).  What a kernel design needs to know before it picks its tile: which
// shapes run at the full rate of the pipe.
__device__ __forceinline__ void mma_f16_ts_probe(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
      : "memory");
}

template <int M, int N, bool kTs>
__global__ void __launch_bounds__(kPeakThreads, 1) mma_shape_kernel(int iters, int64_t* clocks_out, int32_t* status) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_al + kPeakABytes + kPeakBBytes);
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < (kPeakABytes + kPeakBBytes) / 4; i += kPeakThreads) {
    uint32_t x = (i + 1) * 2654435761u + blockIdx.x * 40503u;
    x ^= x >> 15;
    reinterpret_cast<uint32_t*>(smem_al)[i] = x & 0x3F7F3F7Fu;    // finite bf16 pairs
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
    constexpr uint32_t idesc = make_idesc(kFmtBF16, kFmtBF16, M, N);
    if (elect_one()) {
      const uint64_t a0 = make_desc_k_sw128(smem_base);
      const uint64_t b0 = make_desc_k_sw128(smem_base + kPeakABytes);
      const long long t0 = clock64();
      for (int it = 0; it < iters; ++it) {
        // two accumulators where they fit (N <= 128), A from columns 384.. in the TS form
        const uint32_t d = tmem_base + (((it & 1) && N <= 128) ? 128u : 0u);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          if constexpr (kTs) mma_f16_ts_probe(d, tmem_base + 384 + kk * 8, b0 + 2 * kk, idesc);
          else mma_f16_ss(d, a0 + 2 * kk, b0 + 2 * kk, idesc, 1);
        }
      }
      tc_commit(bar);
      // SM clocks from the first issue until the last MMA has retired
      long long spins = 0;
      while (!mbar_test(bar, 0) && ++spins < (1ll << 28)) {}
      if (clocks_out) clocks_out[blockIdx.x] = clock64() - t0;
    }
    __syncwarp();
    if (!mbar_wait(bar, 0, &s_abort) && (tid & 31) == 0) atomicMax(status, kDevWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

template <int M, int N, bool kTs>
static cudaError_t launch_shape(int ctas, int iters, int64_t* clocks_out, int32_t* status, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(mma_shape_kernel<M, N, kTs>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem);
  if (e == cudaSuccess) mma_shape_kernel<M, N, kTs><<<ctas, kPeakThreads, kPeakSmem, st>>>(iters, clocks_out, status);
  return e;
}

// HBM read probe: every CTA pulls chunks (pages) of a buffer into a shared-memory ring with bulk copies
// and drops them: the rate at which a given list of chunks can be read at all, which is what bounds a
// streaming kernel over a paged cache (random 8 KB pages read a little slower than one linear stream).
constexpr int kReadStages = 5;
constexpr int kReadMaxChunk = 16896;   // two pages of 64 keys with their scales

__global__ void __launch_bounds__(64) hbm_read_probe_kernel(const uint8_t* __restrict__ base,
                                                            const int64_t* __restrict__ offsets, int n_chunks,
                                                            int chunk_bytes, int per_stage, int32_t* status) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ int s_abort;
  const uint32_t sb = (smem_u32(smem_dyn) + 127u) & ~127u;
  uint8_t* sm = smem_dyn + (sb - smem_u32(smem_dyn));
  const int stage_bytes = chunk_bytes * per_stage;
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + kReadStages * kReadMaxChunk);
  uint64_t* empty = full + kReadStages;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kReadStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  const int n_groups = n_chunks / per_stage;
  int it = 0;
  if (warp == 0) {
    // the offsets of the next slot are fetched while this one is issued: a load the copies depend on would
    // sit on the producer's critical path once per slot
    int64_t nxt[4] = {0, 0, 0, 0};
    auto fetch = [&](int c) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (j < per_stage && c < n_groups) nxt[j] = __ldg(offsets + static_cast<int64_t>(c) * per_stage + j);
    };
    fetch(blockIdx.x);
    for (int c = blockIdx.x; c < n_groups; c += gridDim.x, ++it) {
      const int s = it % kReadStages;
      const int64_t cur[4] = {nxt[0], nxt[1], nxt[2], nxt[3]};
      fetch(c + gridDim.x);
      const bool ok = mbar_wait(&empty[s], ((it / kReadStages) & 1) ^ 1, &s_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(&full[s], stage_bytes);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j < per_stage) bulk_load_1d(sm + s * kReadMaxChunk + j * chunk_bytes, base + cur[j], chunk_bytes, &full[s]);
      }
      __syncwarp();
    }
    // copies still in flight must land before the shared memory is given back
    for (int j = 0; j < min(it, kReadStages); ++j) {
      const int k = it - 1 - j;
      mbar_wait(&full[k % kReadStages], (k / kReadStages) & 1, &s_abort);
    }
  } else {
    unsigned acc = 0;
    for (int c = blockIdx.x; c < n_groups; c += gridDim.x, ++it) {
      const int s = it % kReadStages;
      const bool ok = mbar_wait(&full[s], (it / kReadStages) & 1, &s_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      acc += reinterpret_cast<volatile unsigned*>(sm + s * kReadMaxChunk)[threadIdx.x & 31];
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(&empty[s]);
    }
    if (acc == 0x9e3779b9u) atomicAdd(status, 0);   // keeps the reads alive
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_abort) atomicMax(status, kDevWaitTimeout);
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

// Flops of one launch: ctas * iters * 4 MMAs * 2*m*n*16.
extern "C" int b200dsa_mma_shape_probe(int32_t m, int32_t n, int32_t a_from_tmem, int32_t ctas, int32_t iters,
                                       int64_t* clocks_out, int32_t* status, void* stream) {
  if (ctas < 1 || iters < 1 || iters > (1 << 22) || !status) {
    set_last_error("b200dsa_mma_shape_probe: bad argument");
    return B200DSA_EINVAL;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaErrorInvalidValue;
  const int key = m * 1000 + n;
#define B200DSA_SHAPE(M_, N_)                                                              \
  if (key == M_ * 1000 + N_)                                                               \
    e = a_from_tmem ? launch_shape<M_, N_, true>(ctas, iters, clocks_out, status, st)                            \
                    : launch_shape<M_, N_, false>(ctas, iters, clocks_out, status, st);
  B200DSA_SHAPE(128, 256) B200DSA_SHAPE(128, 128) B200DSA_SHAPE(128, 64) B200DSA_SHAPE(128, 32)
  B200DSA_SHAPE(64, 256) B200DSA_SHAPE(64, 128) B200DSA_SHAPE(64, 64) B200DSA_SHAPE(64, 32)
#undef B200DSA_SHAPE
  if (e == cudaErrorInvalidValue) {
    set_last_error("b200dsa_mma_shape_probe: m must be 64 or 128 and n one of 32, 64, 128, 256");
    return B200DSA_EUNSUPPORTED;
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_hbm_read_probe(const void* base, const int64_t* offsets, int32_t n_chunks, int32_t chunk_bytes,
                                      int32_t chunks_per_stage, int32_t ctas, int32_t* status, void* stream) {
  if (!base || !offsets || !status || n_chunks < 1 || ctas < 1 || chunk_bytes < 16 || (chunk_bytes & 15) ||
      chunks_per_stage < 1 || chunks_per_stage > 4 || chunk_bytes * chunks_per_stage > kReadMaxChunk ||
      (reinterpret_cast<uintptr_t>(base) & 15)) {
    set_last_error("b200dsa_hbm_read_probe: chunk_bytes a multiple of 16, 1..4 chunks per stage, together <= 16896 bytes");
    return B200DSA_EINVAL;
  }
  const int smem = kReadStages * kReadMaxChunk + 2 * kReadStages * 8 + 128;
  cudaError_t e = cudaFuncSetAttribute(hbm_read_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess)
    hbm_read_probe_kernel<<<ctas, 64, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(base), offsets, n_chunks, chunk_bytes, chunks_per_stage, status);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
