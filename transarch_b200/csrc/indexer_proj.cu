// The elementwise tails of the indexer's projections, one warp per 128-wide row (four values per lane):
//
//   key rows    k = LayerNorm(wk(h)) over the 128 dims (biased variance, eps inside the square root),
//               then RoPE on the rope dims; written as bf16 / fp32 rows, or quantised to e4m3 with a
//               per-token scale and stored straight into the paged cache (no bf16 round trip);
//   query rows  RoPE on the rope dims of every (token, head) row of wq(q_in); written as rows, or
//               quantised to e4m3 with the scale folded into the head weight.
//
// RoPE is the rotate-half form on 64 rope dims: out[i] = x[i] cos[i] - x[i+32] sin[i],
// out[i+32] = x[i+32] cos[i+32] + x[i] sin[i+32] (i < 32), the rope dims being the LAST 64 of the row
// (OpenDSA's indexer) or the FIRST 64 (the vLLM model code).  A lane holds dims 4l..4l+3, so the
// partner of a rope value sits 8 lanes away.  All arithmetic is fp32.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdio.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

struct ProjParams {
  const void* in;            // [n_rows, 128] bf16 or fp32
  int in_f32;
  int64_t n_rows;
  int rows_per_token;        // 1 for keys, n_heads for queries: token of a row = row / rows_per_token
  const float* ln_w;         // nullable [128]: LayerNorm weight / bias (keys)
  const float* ln_b;
  float ln_eps;
  const float* cos;          // nullable [n_tokens, 64]
  const float* sin;
  int rope_first;            // rope dims are the first 64 of the row instead of the last 64
  void* out;                 // nullable [n_rows, 128] rows in the input's dtype
  // quantised outputs
  uint8_t* q_fp8;            // nullable [n_rows, 128] e4m3 (queries)
  const float* w;            // [n_rows] head weights (queries)
  float fold;
  float* weights;            // [n_rows] w * scale * fold
  uint8_t* cache;            // nullable: paged cache (keys)
  const int64_t* slot_mapping;
  int page_size;
  int64_t num_pages;
  int use_ue8m0;
  float eps_amax;            // floor of amax before the division by 448 (1e-10 queries, 1e-4 keys)
  int32_t* status;
};

__device__ __forceinline__ float pow2_round_up_proj(float x) {
  const uint32_t u = __float_as_uint(x);
  uint32_t e = u >> 23;
  if (e == 0) return 1.17549435e-38f;
  if (u & 0x7fffffu) ++e;
  return __uint_as_float(e << 23);
}

__global__ void __launch_bounds__(256) proj_rows_kernel(const ProjParams p) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= p.n_rows) return;
  const int lane = threadIdx.x & 31;
  float x[4];
  if (p.in_f32) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p.in) + row * 128) + lane);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.in) + row * 128) + lane);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
  }
  if (p.ln_w) {
    float s = x[0] + x[1] + x[2] + x[3];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s * (1.0f / 128.0f);
    float v = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) v += (x[j] - mean) * (x[j] - mean);
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const float rstd = rsqrtf(v * (1.0f / 128.0f) + p.ln_eps);
    const float4 g = __ldg(reinterpret_cast<const float4*>(p.ln_w) + lane);
    const float4 b = __ldg(reinterpret_cast<const float4*>(p.ln_b) + lane);
    x[0] = (x[0] - mean) * rstd * g.x + b.x;
    x[1] = (x[1] - mean) * rstd * g.y + b.y;
    x[2] = (x[2] - mean) * rstd * g.z + b.z;
    x[3] = (x[3] - mean) * rstd * g.w + b.w;
  }
  if (p.cos) {
    // every lane takes part in the shuffles; only the 16 lanes that hold rope dims apply the rotation
    const int rl = p.rope_first ? lane : lane - 16;          // lane index inside the rope half (0..15)
    const bool in_rope = rl >= 0 && rl < 16;
    const int64_t tok = row / p.rows_per_token;
    float c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
    if (in_rope) {
      const float4 cv = __ldg(reinterpret_cast<const float4*>(p.cos + tok * 64) + rl);
      const float4 sv = __ldg(reinterpret_cast<const float4*>(p.sin + tok * 64) + rl);
      c[0] = cv.x; c[1] = cv.y; c[2] = cv.z; c[3] = cv.w;
      sn[0] = sv.x; sn[1] = sv.y; sn[2] = sv.z; sn[3] = sv.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, x[j], 8);
      // first half of the rope dims (rl < 8) pairs with +32: rotate_half gives -x[i+32]; second half +x[i-32]
      const float rot = (rl < 8) ? -other : other;
      if (in_rope) x[j] = x[j] * c[j] + rot * sn[j];
    }
  }
  if (p.out) {
    if (p.in_f32) {
      reinterpret_cast<float4*>(static_cast<float*>(p.out) + row * 128)[lane] = make_float4(x[0], x[1], x[2], x[3]);
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + row * 128)[lane] = o;
    }
  }
  if (!p.q_fp8 && !p.cache) return;
  // The quantisers see what the reference's quantisers see: the row rounded to bf16 first.
  if (!p.in_f32) {
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = __bfloat162float(__float2bfloat16_rn(x[j]));
  }
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float scale = __fdiv_rn(fmaxf(amax, p.eps_amax), 448.0f);
  if (p.use_ue8m0) scale = pow2_round_up_proj(scale);
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float y = fminf(fmaxf(__fdiv_rn(x[j], scale), -448.0f), 448.0f);
    packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
  }
  if (p.q_fp8) {
    reinterpret_cast<uint32_t*>(p.q_fp8 + row * 128)[lane] = packed;
    if (lane == 0) p.weights[row] = __ldg(p.w + row) * scale * p.fold;
  } else {
    const int64_t slot = p.slot_mapping[row];
    if (slot < 0) return;                                  // padding token
    const int64_t page = slot / p.page_size;
    const int off = static_cast<int>(slot - page * p.page_size);
    if (page >= p.num_pages) {
      if (lane == 0) atomicMax(p.status, kDevBadIndex);
      return;
    }
    uint8_t* pg = p.cache + page * (static_cast<int64_t>(p.page_size) * 132);
    reinterpret_cast<uint32_t*>(pg + off * 128)[lane] = packed;
    if (lane == 0) reinterpret_cast<float*>(pg + p.page_size * 128)[off] = scale;
  }
}

void set_last_error(const char* msg);

static int launch_proj(const ProjParams& p, const char* who, void* stream) {
  if (p.n_rows == 0) return B200DSA_OK;
  if (!p.in || p.n_rows < 0 || p.rows_per_token < 1 || ((p.cos == nullptr) != (p.sin == nullptr)) ||
      ((p.ln_w == nullptr) != (p.ln_b == nullptr)) || (reinterpret_cast<uintptr_t>(p.in) & 15) ||
      (p.out && (reinterpret_cast<uintptr_t>(p.out) & 15))) {
    char msg[160];
    snprintf(msg, sizeof(msg), "%s: bad argument (rows of 128 values, 16-byte aligned)", who);
    set_last_error(msg);
    return B200DSA_EINVAL;
  }
  const unsigned grid = static_cast<unsigned>((p.n_rows + 7) / 8);
  cudaError_t e = launch_chained(proj_rows_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_indexer_k_norm_rope(const void* k_proj, int32_t in_f32, int64_t n_tokens, const float* ln_w,
                                           const float* ln_b, float ln_eps, const float* cos, const float* sin,
                                           int32_t rope_first, void* k_out, const int64_t* slot_mapping, void* cache,
                                           int64_t num_pages, int32_t page_size, int32_t use_ue8m0, int32_t* status,
                                           void* stream) {
  ProjParams p{};
  p.in = k_proj; p.in_f32 = in_f32; p.n_rows = n_tokens; p.rows_per_token = 1;
  p.ln_w = ln_w; p.ln_b = ln_b; p.ln_eps = ln_eps; p.cos = cos; p.sin = sin; p.rope_first = rope_first;
  p.out = k_out;
  p.cache = static_cast<uint8_t*>(cache); p.slot_mapping = slot_mapping; p.page_size = page_size;
  p.num_pages = num_pages; p.use_ue8m0 = use_ue8m0; p.eps_amax = 1e-4f; p.status = status;
  if ((!k_out && !cache) || (cache && (!slot_mapping || !status || page_size < 4 || (page_size & 3) || num_pages < 1))) {
    set_last_error("b200dsa_indexer_k_norm_rope: needs k_out and / or a cache with slot_mapping, status, page_size % 4 == 0");
    return B200DSA_EINVAL;
  }
  return launch_proj(p, "b200dsa_indexer_k_norm_rope", stream);
}

extern "C" int b200dsa_indexer_q_rope(const void* q_proj, int32_t in_f32, int64_t n_tokens, int32_t n_heads,
                                      const float* cos, const float* sin, int32_t rope_first, void* q_out,
                                      const float* w, float fold, int32_t use_ue8m0, void* q_fp8, float* weights,
                                      void* stream) {
  ProjParams p{};
  p.in = q_proj; p.in_f32 = in_f32; p.n_rows = n_tokens * n_heads; p.rows_per_token = n_heads;
  p.cos = cos; p.sin = sin; p.rope_first = rope_first; p.out = q_out;
  p.q_fp8 = static_cast<uint8_t*>(q_fp8); p.w = w; p.fold = fold; p.weights = weights; p.use_ue8m0 = use_ue8m0;
  p.eps_amax = 1e-10f;
  if (n_heads < 1 || (!q_out && !q_fp8) || (q_fp8 && (!w || !weights))) {
    set_last_error("b200dsa_indexer_q_rope: needs q_out and / or q_fp8 with w and weights");
    return B200DSA_EINVAL;
  }
  return launch_proj(p, "b200dsa_indexer_q_rope", stream);
}
