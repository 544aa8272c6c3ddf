// Block mean pooling of index keys (the coarse keys of HISA stage 1 and of MISA's block-score
// head router).  HBM-bound streaming reductions: one CTA per pooled block, one thread per
// key dimension, rows read as whole 128/256-byte lines; fp32 accumulation; the tail block is
// divided by its true length.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

__global__ void __launch_bounds__(128) block_mean_pool_bf16_kernel(const __nv_bfloat16* __restrict__ keys, int n_keys,
                                                                   int block, __nv_bfloat16* __restrict__ out_bf16,
                                                                   float* __restrict__ out_f32) {
  const int b = blockIdx.x, d = threadIdx.x;
  const int r0 = b * block;
  const int r1 = min(r0 + block, n_keys);
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
  int r = r0;
  for (; r + 3 < r1; r += 4) {
    acc0 += __bfloat162float(keys[static_cast<int64_t>(r) * 128 + d]);
    acc1 += __bfloat162float(keys[static_cast<int64_t>(r + 1) * 128 + d]);
    acc2 += __bfloat162float(keys[static_cast<int64_t>(r + 2) * 128 + d]);
    acc3 += __bfloat162float(keys[static_cast<int64_t>(r + 3) * 128 + d]);
  }
  for (; r < r1; ++r) acc0 += __bfloat162float(keys[static_cast<int64_t>(r) * 128 + d]);
  const float mean = ((acc0 + acc1) + (acc2 + acc3)) / static_cast<float>(r1 - r0);
  if (out_bf16) out_bf16[static_cast<int64_t>(b) * 128 + d] = __float2bfloat16_rn(mean);
  if (out_f32) out_f32[static_cast<int64_t>(b) * 128 + d] = mean;
}

// Paged FP8 cache: pooled[b, j, :] = mean over positions [j*block, min((j+1)*block, ctx_b)) of
// fp8(key) * scale.  Pooled blocks at or beyond ceil(ctx_b / block) are zero.
__global__ void __launch_bounds__(128)
paged_mean_pool_fp8_kernel(const uint8_t* __restrict__ cache, int page_size, int num_pages,
                           const int32_t* __restrict__ context_lens, const int32_t* __restrict__ block_table,
                           int64_t table_stride, int block, int max_pool_blocks, float* __restrict__ out,
                           int32_t* __restrict__ status) {
  const int req = blockIdx.y, j = blockIdx.x, d = threadIdx.x;
  const int ctx = context_lens[req];
  const int r0 = j * block;
  const int r1 = min(r0 + block, ctx);
  float acc = 0.f;
  const int64_t page_bytes = static_cast<int64_t>(page_size) * 132;
  for (int r = r0; r < r1; ++r) {
    const int pg = __ldg(block_table + req * table_stride + r / page_size);
    if (pg < 0 || pg >= num_pages) {
      if (d == 0) atomicMax(status, kDevBadIndex);
      continue;
    }
    const int slot = r % page_size;
    const uint8_t* page = cache + pg * page_bytes;
    const __nv_fp8_e4m3 v = *reinterpret_cast<const __nv_fp8_e4m3*>(page + slot * 128 + d);
    const float sc = __ldg(reinterpret_cast<const float*>(page + page_size * 128) + slot);
    acc += static_cast<float>(v) * sc;
  }
  out[(static_cast<int64_t>(req) * max_pool_blocks + j) * 128 + d] = (r1 > r0) ? acc / static_cast<float>(r1 - r0) : 0.f;
}

// Incremental form of the kernel above: a request whose context grew from prev_b to ctx_b keys only
// reads the new keys.  sums[b, j, :] carries the running fp32 sum of block j in position order, which is
// the order the full kernel adds in, so sums / count is bit-identical to pooling the whole cache again.
// The CTAs of request b (gridDim.x of them) stride over the blocks that hold a position in [prev_b, ctx_b);
// with prev_b = 0 they rebuild every block of the request and clear the blocks beyond its context.
__global__ void __launch_bounds__(128)
paged_mean_pool_fp8_update_kernel(const uint8_t* __restrict__ cache, int page_size, int num_pages,
                                  const int32_t* __restrict__ prev_lens, const int32_t* __restrict__ context_lens,
                                  const int32_t* __restrict__ block_table, int64_t table_stride, int block,
                                  int max_pool_blocks, float* __restrict__ sums, float* __restrict__ out,
                                  int32_t* __restrict__ status) {
  const int req = blockIdx.y, d = threadIdx.x;
  const int ctx = context_lens[req];
  const int prev = min(max(prev_lens[req], 0), ctx);
  const int j_begin = (prev == 0) ? 0 : prev / block;
  const int j_end = (prev == 0) ? max_pool_blocks : min(max_pool_blocks, (ctx + block - 1) / block);
  const int64_t page_bytes = static_cast<int64_t>(page_size) * 132;
  for (int j = j_begin + blockIdx.x; j < j_end; j += gridDim.x) {
    const int r0 = j * block;
    const int r1 = min(r0 + block, ctx);
    const int64_t o = (static_cast<int64_t>(req) * max_pool_blocks + j) * 128 + d;
    if (r1 <= r0) {          // beyond the context (only reached when the request is rebuilt)
      sums[o] = 0.f;
      out[o] = 0.f;
      continue;
    }
    const int ra = max(r0, prev);
    if (ra >= r1) continue;  // nothing new in this block
    float acc = (ra > r0) ? sums[o] : 0.f;
    for (int r = ra; r < r1; ++r) {
      const int pg = __ldg(block_table + req * table_stride + r / page_size);
      if (pg < 0 || pg >= num_pages) {
        if (d == 0) atomicMax(status, kDevBadIndex);
        continue;
      }
      const int slot = r % page_size;
      const uint8_t* page = cache + pg * page_bytes;
      const __nv_fp8_e4m3 v = *reinterpret_cast<const __nv_fp8_e4m3*>(page + slot * 128 + d);
      const float sc = __ldg(reinterpret_cast<const float*>(page + page_size * 128) + slot);
      acc += static_cast<float>(v) * sc;
    }
    sums[o] = acc;
    out[o] = acc / static_cast<float>(r1 - r0);
  }
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_block_mean_pool_bf16(const void* keys_bf16, int32_t n_keys, int32_t block, void* out_bf16,
                                            float* out_f32, void* stream) {
  if (n_keys == 0) return B200DSA_OK;
  if (!keys_bf16 || n_keys < 0 || block < 1 || (!out_bf16 && !out_f32)) {
    set_last_error("b200dsa_block_mean_pool_bf16: bad argument");
    return B200DSA_EINVAL;
  }
  const int nb = (n_keys + block - 1) / block;
  block_mean_pool_bf16_kernel<<<nb, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(keys_bf16), n_keys, block, static_cast<__nv_bfloat16*>(out_bf16), out_f32);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_paged_mean_pool_fp8(const void* cache, int32_t num_pages, int32_t page_size,
                                           const int32_t* context_lens, const int32_t* block_table,
                                           int64_t block_table_stride, int32_t n_requests, int32_t block,
                                           int32_t max_pool_blocks, float* out, int32_t* status, void* stream) {
  if (n_requests == 0 || max_pool_blocks == 0) return B200DSA_OK;
  if (!cache || !context_lens || !block_table || !out || !status || n_requests < 0 || block < 1 || page_size < 1 ||
      num_pages < 1 || max_pool_blocks < 0) {
    set_last_error("b200dsa_paged_mean_pool_fp8: bad argument");
    return B200DSA_EINVAL;
  }
  dim3 grid(max_pool_blocks, n_requests);
  paged_mean_pool_fp8_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(cache), page_size, num_pages, context_lens, block_table, block_table_stride, block,
      max_pool_blocks, out, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_paged_mean_pool_fp8_update(const void* cache, int32_t num_pages, int32_t page_size,
                                                  const int32_t* prev_lens, const int32_t* context_lens,
                                                  const int32_t* block_table, int64_t block_table_stride,
                                                  int32_t n_requests, int32_t block, int32_t max_pool_blocks,
                                                  int32_t ctas_per_request, float* sums, float* out,
                                                  int32_t* status, void* stream) {
  if (n_requests == 0 || max_pool_blocks == 0) return B200DSA_OK;
  if (!cache || !prev_lens || !context_lens || !block_table || !sums || !out || !status || n_requests < 0 ||
      block < 1 || page_size < 1 || num_pages < 1 || max_pool_blocks < 0 || ctas_per_request < 1 ||
      ctas_per_request > 65535) {
    set_last_error("b200dsa_paged_mean_pool_fp8_update: bad argument");
    return B200DSA_EINVAL;
  }
  dim3 grid(ctas_per_request, n_requests);
  paged_mean_pool_fp8_update_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(cache), page_size, num_pages, prev_lens, context_lens, block_table,
      block_table_stride, block, max_pool_blocks, sums, out, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
