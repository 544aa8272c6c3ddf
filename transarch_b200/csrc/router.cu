// MISA head routing: which n of the 64 index heads score tokens for a query.  Every router
// emits (a) the kept head ids and (b) a dense [64] weight row that is zero on the dropped heads,
// so the 64-head indexer kernels apply the gating through their weight operand (a zero weight
// removes the head from the sum exactly).
//
//   q-norm      : heads with the largest ||q[t,h,:]||_2; kept heads keep their weight w[t,h]
//   block-score : heads with the largest sum over pooled key blocks of |w[t,h]*relu(<q[t,h],kblk>)|
//   linear      : logits = x[t,:] @ W_r; top-n heads; weights = softmax over the kept logits
// Ties go to the lowest head id.  One CTA of 256 threads per query token.
#include <cuda_bf16.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kRouterHeads = 64;

// Warp 0: pick the n largest of score[0..63] (ties: lowest id).  Writes ids to sel[0..n) in
// descending score order and keep[h] = 1 for the chosen heads.
__device__ void select_top_heads(const float* score, int n, int* sel, int* keep) {
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  float a = score[lane], b = score[lane + 32];
  bool ta = false, tb = false;
  keep[lane] = 0;
  keep[lane + 32] = 0;
  __syncwarp();
  for (int i = 0; i < n; ++i) {
    // candidate of this lane: its larger remaining value (lower id on ties)
    float v = -INFINITY;
    int id = 0x7fffffff;
    if (!ta) { v = a; id = lane; }
    if (!tb && (id == 0x7fffffff || b > v)) { v = b; id = lane + 32; }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oid = __shfl_xor_sync(0xffffffffu, id, o);
      if (ov > v || (ov == v && oid < id)) { v = ov; id = oid; }
    }
    if (id == lane) ta = true;
    if (id == lane + 32) tb = true;
    if (lane == 0 && id < kRouterHeads) {
      sel[i] = id;
      keep[id] = 1;
    }
  }
  __syncwarp();
}

constexpr int kLinThreads = 1024;          // 128 row groups x 8 threads (8 heads each)
constexpr int kLinGroups = kLinThreads / 8;
__global__ void __launch_bounds__(kLinThreads) router_linear_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ w_r, int hidden, int n_keep,
                                                            const float* __restrict__ out_scale,
                                                            float* __restrict__ weights_out,
                                                            int32_t* __restrict__ head_idx,
                                                            float* __restrict__ logits_out) {
  // Thread (grp, h8): rows grp, grp+128, ... of W_r, heads 8*h8 .. 8*h8+7 (one 16-byte load per row),
  // eight rows in flight per thread (the kernel is bound by the latency of these loads: one CTA per
  // token, a few tokens per step); x is staged in shared memory once.
  extern __shared__ __nv_bfloat16 xs[];
  __shared__ float part[kLinGroups][kRouterHeads + 1];
  __shared__ float logit[kRouterHeads];
  __shared__ int sel[kRouterHeads], keep[kRouterHeads];
  const int t = blockIdx.x, tid = threadIdx.x, h8 = tid & 7, grp = tid >> 3;
  const __nv_bfloat16* xr = x + static_cast<int64_t>(t) * hidden;
  for (int i = tid; i < hidden; i += kLinThreads) xs[i] = xr[i];
  __syncthreads();
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const uint4* wv = reinterpret_cast<const uint4*>(w_r) + h8;   // row i: 8 uint4 (64 bf16)
  int i = grp;
  for (; i + 7 * kLinGroups < hidden; i += 8 * kLinGroups) {
    uint4 r[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) r[u] = __ldg(wv + static_cast<int64_t>(i + kLinGroups * u) * 8);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float xv = __bfloat162float(xs[i + kLinGroups * u]);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&r[u]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] = fmaf(xv, __low2float(w2[j]), acc[2 * j]);
        acc[2 * j + 1] = fmaf(xv, __high2float(w2[j]), acc[2 * j + 1]);
      }
    }
  }
  for (; i < hidden; i += kLinGroups) {
    const uint4 r = __ldg(wv + static_cast<int64_t>(i) * 8);
    const float xv = __bfloat162float(xs[i]);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[2 * j] = fmaf(xv, __low2float(w2[j]), acc[2 * j]);
      acc[2 * j + 1] = fmaf(xv, __high2float(w2[j]), acc[2 * j + 1]);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[grp][8 * h8 + j] = acc[j];
  __syncthreads();
  if (tid < 256) {     // four partial sums per head, then one add tree through the warp
    const int h = tid >> 2, q4 = tid & 3;
    float sum = 0.f;
    for (int g = q4; g < kLinGroups; g += 4) sum += part[g][h];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (q4 == 0) {
      logit[h] = sum;
      if (logits_out) logits_out[static_cast<int64_t>(t) * 64 + h] = sum;
    }
  }
  __syncthreads();
  select_top_heads(logit, n_keep, sel, keep);
  __syncthreads();
  if (tid < 64) {
    const int h = tid;
    // softmax over the kept logits (sel[0] holds the largest)
    const float mx = logit[sel[0]];
    float den = 0.f;
    for (int j = 0; j < n_keep; ++j) den += expf(logit[sel[j]] - mx);
    const float sc = out_scale ? out_scale[static_cast<int64_t>(t) * 64 + h] : 1.0f;
    weights_out[static_cast<int64_t>(t) * 64 + h] = keep[h] ? expf(logit[h] - mx) / den * sc : 0.f;
    if (h < n_keep) head_idx[static_cast<int64_t>(t) * n_keep + h] = sel[h];
  }
}

__global__ void __launch_bounds__(256) router_qnorm_kernel(const __nv_bfloat16* __restrict__ q,
                                                           const float* __restrict__ w, int n_keep,
                                                           float* __restrict__ weights_out,
                                                           int32_t* __restrict__ head_idx) {
  __shared__ float score[kRouterHeads];
  __shared__ int sel[kRouterHeads], keep[kRouterHeads];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int hh = 0; hh < 8; ++hh) {
    const int h = warp * 8 + hh;
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(q + (static_cast<int64_t>(t) * 64 + h) * 128) + lane);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float s = __low2float(a) * __low2float(a) + __high2float(a) * __high2float(a) +
              __low2float(b) * __low2float(b) + __high2float(b) * __high2float(b);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) score[h] = s;  // squared norm: same order as the norm
  }
  __syncthreads();
  select_top_heads(score, n_keep, sel, keep);
  __syncthreads();
  if (threadIdx.x < 64) {
    const int h = threadIdx.x;
    weights_out[static_cast<int64_t>(t) * 64 + h] = keep[h] ? w[static_cast<int64_t>(t) * 64 + h] : 0.f;
    if (h < n_keep) head_idx[static_cast<int64_t>(t) * n_keep + h] = sel[h];
  }
}

// kblk: pooled keys fp32 [n_sets, kblk_stride_rows, 128]; token t uses set kb_set[t] (or 0) and
// blocks [blk_lo[t], blk_hi[t]).
__global__ void __launch_bounds__(256)
router_block_score_kernel(const __nv_bfloat16* __restrict__ q, const float* __restrict__ w,
                          const float* __restrict__ kblk, int64_t kblk_set_stride, const int32_t* __restrict__ kb_set,
                          const int32_t* __restrict__ blk_lo, const int32_t* __restrict__ blk_hi, int n_keep,
                          float* __restrict__ weights_out, int32_t* __restrict__ head_idx,
                          float* __restrict__ scores_out) {
  __shared__ __nv_bfloat16 qT[128][kRouterHeads + 2];  // transposed: conflict-free per-head reads
  __shared__ float kb[4][128];
  __shared__ float part[4][kRouterHeads];
  __shared__ float score[kRouterHeads];
  __shared__ int sel[kRouterHeads], keep[kRouterHeads];
  const int t = blockIdx.x, h = threadIdx.x & 63, g = threadIdx.x >> 6;
  for (int i = threadIdx.x; i < 64 * 128; i += 256) {
    const int hh = i >> 7, d = i & 127;
    qT[d][hh] = q[(static_cast<int64_t>(t) * 64 + hh) * 128 + d];
  }
  const float wh = w[static_cast<int64_t>(t) * 64 + h];
  const float* kbase = kblk + (kb_set ? kb_set[t] : 0) * kblk_set_stride;
  const int lo = blk_lo[t], hi = blk_hi[t];
  float acc = 0.f;
  __syncthreads();
  for (int j0 = lo; j0 < hi; j0 += 4) {
    // four blocks per round, one per thread group
    for (int i = threadIdx.x; i < 4 * 128; i += 256) {
      const int jj = i >> 7, d = i & 127;
      kb[jj][d] = (j0 + jj < hi) ? __ldg(kbase + static_cast<int64_t>(j0 + jj) * 128 + d) : 0.f;
    }
    __syncthreads();
    if (j0 + g < hi) {
      float dot = 0.f;
#pragma unroll 8
      for (int d = 0; d < 128; ++d) dot = fmaf(__bfloat162float(qT[d][h]), kb[g][d], dot);
      acc += fabsf(wh * fmaxf(dot, 0.f));
    }
    __syncthreads();
  }
  part[g][h] = acc;
  __syncthreads();
  if (threadIdx.x < 64) {
    score[h] = (part[0][h] + part[1][h]) + (part[2][h] + part[3][h]);
    if (scores_out) scores_out[static_cast<int64_t>(t) * 64 + h] = score[h];
  }
  __syncthreads();
  select_top_heads(score, n_keep, sel, keep);
  __syncthreads();
  if (threadIdx.x < 64) {
    weights_out[static_cast<int64_t>(t) * 64 + h] = keep[h] ? wh : 0.f;
    if (h < n_keep) head_idx[static_cast<int64_t>(t) * n_keep + h] = sel[h];
  }
}

void set_last_error(const char* msg);

static int finish_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_router_linear_topk_softmax(const void* x_bf16, const void* w_r_bf16, int32_t n_tokens,
                                                  int32_t hidden, int32_t n_keep, const float* out_scale,
                                                  float* weights_out, int32_t* head_idx, float* logits_out,
                                                  void* stream) {
  if (n_tokens == 0) return B200DSA_OK;
  if (!x_bf16 || !w_r_bf16 || !weights_out || !head_idx || n_tokens < 0 || hidden < 1 || n_keep < 1 || n_keep > 64) {
    set_last_error("b200dsa_router_linear_topk_softmax: bad argument (1 <= n_keep <= 64)");
    return B200DSA_EINVAL;
  }
  if (hidden > 24576 || (reinterpret_cast<uintptr_t>(w_r_bf16) & 15)) {
    set_last_error("b200dsa_router_linear_topk_softmax: hidden must be <= 24576 and W_r 16-byte aligned");
    return B200DSA_EINVAL;
  }
  router_linear_kernel<<<n_tokens, kLinThreads, static_cast<size_t>(hidden) * 2, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), static_cast<const __nv_bfloat16*>(w_r_bf16), hidden, n_keep,
      out_scale, weights_out, head_idx, logits_out);
  return finish_launch();
}

extern "C" int b200dsa_router_qnorm_topk(const void* q_bf16, const float* w, int32_t n_tokens, int32_t n_keep,
                                         float* weights_out, int32_t* head_idx, void* stream) {
  if (n_tokens == 0) return B200DSA_OK;
  if (!q_bf16 || !w || !weights_out || !head_idx || n_tokens < 0 || n_keep < 1 || n_keep > 64 ||
      (reinterpret_cast<uintptr_t>(q_bf16) & 7)) {
    set_last_error("b200dsa_router_qnorm_topk: bad argument (1 <= n_keep <= 64, q 8-byte aligned)");
    return B200DSA_EINVAL;
  }
  router_qnorm_kernel<<<n_tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q_bf16), w, n_keep, weights_out, head_idx);
  return finish_launch();
}

extern "C" int b200dsa_router_block_score_topk(const void* q_bf16, const float* w, const float* pooled_keys,
                                               int64_t pooled_set_stride, const int32_t* pooled_set,
                                               const int32_t* blk_lo, const int32_t* blk_hi, int32_t n_tokens,
                                               int32_t n_keep, float* weights_out, int32_t* head_idx,
                                               float* scores_out, void* stream) {
  if (n_tokens == 0) return B200DSA_OK;
  if (!q_bf16 || !w || !pooled_keys || !blk_lo || !blk_hi || !weights_out || !head_idx || n_tokens < 0 ||
      n_keep < 1 || n_keep > 64) {
    set_last_error("b200dsa_router_block_score_topk: bad argument (1 <= n_keep <= 64)");
    return B200DSA_EINVAL;
  }
  router_block_score_kernel<<<n_tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q_bf16), w, pooled_keys, pooled_set_stride, pooled_set, blk_lo, blk_hi, n_keep,
      weights_out, head_idx, scores_out);
  return finish_launch();
}
