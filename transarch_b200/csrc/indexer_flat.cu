// Lightning-indexer token logits for flat (unpaged) bf16 keys with causal / document intervals: the
// prefill form.  Four consecutive query rows share every key tile:
//
//   logit[r, c] = out_scale * sum_h w[r,h] * relu(<q[r,h,:], k[pos,:]>),  pos = col0[r] + c,
//   col0[r] = 128 * (pos_lo[r] / 128), for pos_lo[r] <= pos < pos_hi[r]; -inf for the other columns of
//   the row's range [0, row_cols[r]).
//
// Orientation: the 128 keys of a tile are the UMMA M dimension (one TMEM lane per key); N = 256 =
// 4 queries x 64 heads; K = 128.  One MMA pass over a key tile therefore serves four queries, and the
// tile is fetched once per group instead of once per query (a per-query N = 64 pass re-reads every 32 KB
// key tile from L2 for each query).  A group's tiles run from the lowest block any of its rows starts in
// to the highest block any of them ends in; rows mask their own interval in the epilogue.
//
// Roles (320 threads): warp 0 issues TMA loads (keys into a 4-stage ring, the group's 64 KB of queries
// into a single buffer that is refilled when the previous group's MMAs have retired), warp 1 issues the
// MMAs into two 256-column TMEM accumulators, warps 2-9 read them: two warps per 32-lane TMEM quadrant
// (thread = key), one taking queries 0-1 of the group and the other queries 2-3, so that every scheduler
// has two epilogue warps to switch between.  A warp keeps the 128 head weights of its two queries in its
// own slice of shared memory (reloaded when the group changes), loads the second query's accumulator
// columns while it reduces the first, and sums the heads in four independent chains.  Persistent grid over
// the list of (group, tile) pairs; bounded waits throughout.
#include <stdio.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kFlatTile = 128;
constexpr int kFlatGroup = 4;                     // queries per MMA with all 64 heads
constexpr int kFlatHeads = 64;
// Routed form (MISA stage 1): the router kept kRoutedHeads of a query's heads and they were gathered into
// q [n_rows, 8, 128]; an MMA then serves 32 queries (N = 256 = 32 x 8), which is where the routing saves
// flops: the key tile is contracted with 8 heads per query instead of 64.
constexpr int kRoutedHeads = 8;
constexpr int kFlatThreads = 320;
constexpr int kFlatStages = 4;
constexpr int kFlatStageBytes = kFlatTile * 128 * 2;          // 32 KB
constexpr int kFlatQBytes = kFlatGroup * kFlatHeads * 128 * 2;  // 64 KB
constexpr int kFlatMaxGroups = 1024;              // groups per launch (4096 rows; 32768 in the routed form)
constexpr int kFlatWBytes = 8 * 128 * 4;                      // per epilogue warp: the weights of its queries
constexpr int kFlatRowParamBytes = 8 * 16 * 16;               // routed form, per epilogue warp: lo, hi, col0, ncol of 16 queries
constexpr int kFlatSmem = kFlatStages * kFlatStageBytes + kFlatQBytes + 1024 + 256 + kFlatWBytes + kFlatRowParamBytes;

struct FlatParams {
  const float* weights;      // [n_rows, heads per query]
  const int32_t* pos_lo;     // [n_rows]
  const int32_t* pos_hi;     // [n_rows]
  const int32_t* row_cols;   // [n_rows] columns of the row's range (a multiple of 128)
  int32_t n_rows, n_blocks;  // key blocks of 128 in the key tensor
  float out_scale;
  float* logits;
  int64_t logits_stride;
  int32_t logits_cols;
  int32_t* status;
};

template <int kHq>   // heads per query: 64 (all heads) or 8 (routed)
__global__ void __launch_bounds__(kFlatThreads, 1)
indexer_flat_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_q,
                    const FlatParams p) {
  constexpr int kGroup = 256 / kHq;     // queries per MMA (4 or 32)
  constexpr int kQW = 128 / kHq;        // queries per epilogue warp (2 or 16)
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ uint8_t smem_dyn[];
  __shared__ int s_prefix[kFlatMaxGroups + 1];
  __shared__ int s_b0[kFlatMaxGroups];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
  uint8_t* q_mem = smem_al + kFlatStages * kFlatStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(q_mem + kFlatQBytes);
  uint64_t* full = bars;                        // [stages]
  uint64_t* empty = bars + kFlatStages;         // [stages]
  uint64_t* q_full = empty + kFlatStages;       // [1]
  uint64_t* q_empty = q_full + 1;               // [1]
  uint64_t* acc_full = q_empty + 1;             // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  float* w_mem = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);   // [8 warps][2 queries][64]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_groups = (p.n_rows + kGroup - 1) / kGroup;

  if (tid == 0) s_abort = 0;
  for (int g = tid; g < n_groups; g += kFlatThreads) {
    int b0 = 0x7fffffff, b1 = 0;
    for (int j = 0; j < kGroup; ++j) {
      const int r = g * kGroup + j;
      if (r >= p.n_rows) break;
      const int lo = p.pos_lo[r], hi = min(p.pos_hi[r], p.n_blocks * kFlatTile);
      if (hi > lo && p.row_cols[r] > 0) {
        b0 = min(b0, lo >> 7);
        b1 = max(b1, (hi + kFlatTile - 1) >> 7);
      }
    }
    s_b0[g] = (b1 > b0) ? b0 : 0;
    s_prefix[g + 1] = (b1 > b0) ? b1 - b0 : 0;
  }
  if (tid == 0) s_prefix[0] = 0;
  __syncthreads();
  if (warp == 0) warp_prefix_inplace(s_prefix, n_groups);
  if (tid == 0) {
    for (int s = 0; s < kFlatStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 256);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&s_tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int total = s_prefix[n_groups];
  const int g0 = static_cast<int>((static_cast<int64_t>(total) * blockIdx.x) / gridDim.x);
  const int g1 = static_cast<int>((static_cast<int64_t>(total) * (blockIdx.x + 1)) / gridDim.x);
  volatile int* abort_flag = &s_abort;
  int grp0 = 0;
  if (g0 < g1) {
    int lo = 0, hi = n_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= g0) lo = mid; else hi = mid;
    }
    grp0 = lo;
  }
  int issued = 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_q);
    }
    int grp = grp0, prev = -1, it = 0, qit = 0;
    for (int g = g0; g < g1; ++g) {
      while (g >= s_prefix[grp + 1]) ++grp;
      if (grp != prev) {
        const bool okq = mbar_wait(q_empty, (qit & 1) ^ 1, abort_flag);
        if (!__all_sync(0xffffffffu, okq)) break;
        if (elect_one()) {
          mbar_arrive_expect_tx(q_full, kFlatQBytes);   // rows beyond the last query are zero-filled
          tma_load_2d(q_mem, &tmap_q, q_full, 0, grp * 256);
          tma_load_2d(q_mem + kFlatQBytes / 2, &tmap_q, q_full, 64, grp * 256);
        }
        ++qit;
        prev = grp;
      }
      const int blk = s_b0[grp] + (g - s_prefix[grp]);
      const int s = it % kFlatStages;
      const bool oke = mbar_wait(&empty[s], ((it / kFlatStages) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, oke)) break;
      if (elect_one()) {
        uint8_t* dst = smem_al + s * kFlatStageBytes;
        mbar_arrive_expect_tx(&full[s], kFlatStageBytes);
        tma_load_2d(dst, &tmap_k, &full[s], 0, blk * kFlatTile);
        tma_load_2d(dst + kFlatStageBytes / 2, &tmap_k, &full[s], 64, blk * kFlatTile);
      }
      ++it;
    }
    issued = it;
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc(kFmtBF16, kFmtBF16, 128, 256);
    int grp = grp0, prev = -1, it = 0, qit = 0;
    for (int g = g0; g < g1; ++g) {
      while (g >= s_prefix[grp + 1]) ++grp;
      if (grp != prev) {
        const bool okq = mbar_wait(q_full, qit & 1, abort_flag);
        if (!__all_sync(0xffffffffu, okq)) break;
        ++qit;
        prev = grp;
      }
      const bool last_of_grp = (g + 1 == g1) || (g + 1 >= s_prefix[grp + 1]);
      const int s = it % kFlatStages, as = it & 1;
      const bool okf = mbar_wait(&full[s], (it / kFlatStages) & 1, abort_flag) &&
                       mbar_wait(&acc_empty[as], ((it >> 1) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, okf)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_addr = smem_base + s * kFlatStageBytes;
        const uint32_t b_addr = smem_base + kFlatStages * kFlatStageBytes;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t a_off = (kk >> 2) * (kFlatStageBytes / 2) + (kk & 3) * 32;
          const uint32_t b_off = (kk >> 2) * (kFlatQBytes / 2) + (kk & 3) * 32;
          mma_f16_ss(tmem_base + as * 256, make_desc_k_sw128(a_addr + a_off), make_desc_k_sw128(b_addr + b_off), idesc,
                     kk > 0);
        }
        tc_commit(&empty[s]);
        tc_commit(&acc_full[as]);
        if (last_of_grp) tc_commit(q_empty);
      }
      __syncwarp();
      ++it;
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int lane_base = (warp & 3) * 32;          // TMEM lanes this warp may read
    const int qh = (warp >= 6) ? kQW : 0;           // first query of the group this warp reduces
    float* wq = w_mem + (warp - 2) * 128;
    int grp = grp0, prev = -1, it = 0;
    if constexpr (kHq == kRoutedHeads) {
      // ---- routed form: 16 queries x 8 heads per warp; the queries' intervals live in shared memory
      int4* rp = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(w_mem) + kFlatWBytes) + (warp - 2) * 16;
      for (int g = g0; g < g1; ++g) {
        while (g >= s_prefix[grp + 1]) ++grp;
        if (grp != prev) {
          __syncwarp();
          const int r0 = grp * kGroup + qh;
          if (lane < kQW) {
            const int r = r0 + lane;
            int4 v = make_int4(0, 0, 0, 0);
            if (r < p.n_rows) {
              v.x = p.pos_lo[r];
              v.y = p.pos_hi[r];
              v.z = (v.x >> 7) << 7;
              v.w = max(0, min(p.row_cols[r], p.logits_cols));
            }
            rp[lane] = v;
          }
          // 128 weights = 32 lanes x float4 = 16 queries x 8 heads, contiguous in the weight matrix
          float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
          if (r0 + (lane >> 1) < p.n_rows)
            wv = __ldg(reinterpret_cast<const float4*>(p.weights + static_cast<int64_t>(r0) * kHq) + lane);
          reinterpret_cast<float4*>(wq)[lane] = wv;
          __syncwarp();
          prev = grp;
        }
        const int blk = s_b0[grp] + (g - s_prefix[grp]);
        const int pos = blk * kFlatTile + lane_base + lane;
        const int as = it & 1;
        const bool ready = mbar_wait(&acc_full[as], (it >> 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ready)) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + as * 256 + (warp >= 6 ? 128 : 0);
        uint32_t va[64], vb[64];
        tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(va));
        tmem_ld_32x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(va + 32));
        tc_wait_ld();
        tmem_ld_32x32(taddr + 64, *reinterpret_cast<uint32_t(*)[32]>(vb));       // lands while queries 0-7 are reduced
        tmem_ld_32x32(taddr + 96, *reinterpret_cast<uint32_t(*)[32]>(vb + 32));
        const int r0 = grp * kGroup + qh;
#pragma unroll
        for (int jq = 0; jq < kQW; ++jq) {
          if (jq == 8) {
            tc_wait_ld();
            tc_fence_before();
            mbar_arrive(&acc_empty[as]);       // both halves are in registers
          }
          const uint32_t* v = (jq < 8 ? va : vb) + (jq & 7) * 8;
          const float4 w0 = reinterpret_cast<const float4*>(wq + jq * 8)[0];     // same address in every lane
          const float4 w1 = reinterpret_cast<const float4*>(wq + jq * 8)[1];
          float a0 = fmaxf(__uint_as_float(v[0]), 0.f) * w0.x, a1 = fmaxf(__uint_as_float(v[1]), 0.f) * w0.y;
          a0 = fmaf(fmaxf(__uint_as_float(v[2]), 0.f), w0.z, a0);
          a1 = fmaf(fmaxf(__uint_as_float(v[3]), 0.f), w0.w, a1);
          a0 = fmaf(fmaxf(__uint_as_float(v[4]), 0.f), w1.x, a0);
          a1 = fmaf(fmaxf(__uint_as_float(v[5]), 0.f), w1.y, a1);
          a0 = fmaf(fmaxf(__uint_as_float(v[6]), 0.f), w1.z, a0);
          a1 = fmaf(fmaxf(__uint_as_float(v[7]), 0.f), w1.w, a1);
          const int4 q = rp[jq];
          const int c = pos - q.z;
          if (r0 + jq < p.n_rows && c >= 0 && c < q.w) {            // inside the row's column range
            const bool keep = pos >= q.x && pos < q.y;
            p.logits[static_cast<int64_t>(r0 + jq) * p.logits_stride + c] = keep ? (a0 + a1) * p.out_scale : -INFINITY;
          }
        }
        ++it;
      }
    } else {
      // ---- all heads: two queries x 64 heads per warp
    int lo[2], hi[2], col0[2], ncol[2];
    for (int g = g0; g < g1; ++g) {
      while (g >= s_prefix[grp + 1]) ++grp;
      if (grp != prev) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int r = grp * kGroup + qh + j;
          lo[j] = hi[j] = col0[j] = ncol[j] = 0;
          if (r < p.n_rows) {
            lo[j] = p.pos_lo[r];
            hi[j] = p.pos_hi[r];
            col0[j] = (lo[j] >> 7) << 7;
            ncol[j] = max(0, min(p.row_cols[r], p.logits_cols));
          }
        }
        // 128 weights = 32 lanes x float4: rows r0, r0+1 are contiguous in the weight matrix
        const int r0 = grp * kGroup + qh;
        float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r0 + (lane >> 4) < p.n_rows)
          wv = __ldg(reinterpret_cast<const float4*>(p.weights + static_cast<int64_t>(r0) * kFlatHeads) + lane);
        reinterpret_cast<float4*>(wq)[lane] = wv;
        __syncwarp();
        prev = grp;
      }
      const int blk = s_b0[grp] + (g - s_prefix[grp]);
      const int pos = blk * kFlatTile + lane_base + lane;
      const int as = it & 1;
      const bool ready = mbar_wait(&acc_full[as], (it >> 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + as * 256 + qh * 64;
      uint32_t va[64], vb[64];
      tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(va));
      tmem_ld_32x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(va + 32));
      tc_wait_ld();
      tmem_ld_32x32(taddr + 64, *reinterpret_cast<uint32_t(*)[32]>(vb));       // lands while query 0 is reduced
      tmem_ld_32x32(taddr + 96, *reinterpret_cast<uint32_t(*)[32]>(vb + 32));
      float res[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (j == 1) tc_wait_ld();
        const uint32_t* v = j ? vb : va;
        const float4* w4 = reinterpret_cast<const float4*>(wq + j * 64);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int q4 = 0; q4 < 16; ++q4) {
          const float4 ww = w4[q4];                                               // same address in every lane
          a0 = fmaf(fmaxf(__uint_as_float(v[4 * q4 + 0]), 0.f), ww.x, a0);
          a1 = fmaf(fmaxf(__uint_as_float(v[4 * q4 + 1]), 0.f), ww.y, a1);
          a2 = fmaf(fmaxf(__uint_as_float(v[4 * q4 + 2]), 0.f), ww.z, a2);
          a3 = fmaf(fmaxf(__uint_as_float(v[4 * q4 + 3]), 0.f), ww.w, a3);
        }
        res[j] = (a0 + a1) + (a2 + a3);
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int r = grp * kGroup + qh + j;
        const int c = pos - col0[j];
        if (r < p.n_rows && c >= 0 && c < ncol[j]) {          // inside the row's column range
          const bool keep = pos >= lo[j] && pos < hi[j];
          p.logits[static_cast<int64_t>(r) * p.logits_stride + c] = keep ? res[j] * p.out_scale : -INFINITY;
        }
      }
      ++it;
    }
    }
  }

  if (s_abort && warp == 0 && lane == 0) {
    const int n = min(issued, kFlatStages);
    for (int j = 0; j < n; ++j) {
      const int it = issued - 1 - j;
      const int s = it % kFlatStages;
      const long long t0 = clock64();
      while (!mbar_test(&full[s], (it / kFlatStages) & 1)) {
        if (clock64() - t0 > (1ll << 22)) break;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
  if (tid == 0 && s_abort) atomicMax(p.status, kDevWaitTimeout);
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

template <int kHq>
static int flat_launch(const void* q_bf16, const float* weights, const void* keys_bf16, int32_t n_keys,
                       const int32_t* pos_lo, const int32_t* pos_hi, const int32_t* row_cols, int32_t n_rows,
                       int32_t max_cols, float out_scale, float* logits, int64_t logits_stride, int32_t* status,
                       void* stream) {
  constexpr int kGroup = 256 / kHq;
  if (n_rows == 0) return B200DSA_OK;
  if (!q_bf16 || !weights || !keys_bf16 || !pos_lo || !pos_hi || !row_cols || !logits || !status || n_rows < 0 ||
      n_keys < 1 || max_cols < 0 || logits_stride < max_cols) {
    set_last_error("b200dsa_indexer_flat_bf16_logits: bad argument");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(q_bf16) & 15) || (reinterpret_cast<uintptr_t>(keys_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(weights) & 15)) {
    set_last_error("b200dsa_indexer_flat_bf16_logits: q, weights and keys must be 16-byte aligned");
    return B200DSA_EALIGN;
  }
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return B200DSA_ECUDA;
  cuuint32_t es[2] = {1, 1};
  CUtensorMap mk, mq;
  {
    cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(n_keys)};
    cuuint64_t strides[1] = {256};
    cuuint32_t box[2] = {64, kFlatTile};
    if (enc(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(keys_bf16), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      set_last_error("b200dsa_indexer_flat_bf16_logits: cuTensorMapEncodeTiled rejected the keys");
      return B200DSA_ECUDA;
    }
  }
  cudaError_t e = cudaFuncSetAttribute(indexer_flat_kernel<kHq>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFlatSmem);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int rows_per_launch = kFlatMaxGroups * kGroup;
  for (int r0 = 0; r0 < n_rows; r0 += rows_per_launch) {
    const int nr = n_rows - r0 < rows_per_launch ? n_rows - r0 : rows_per_launch;
    const uint8_t* qbase = static_cast<const uint8_t*>(q_bf16) + static_cast<int64_t>(r0) * kHq * 256;
    cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(nr) * kHq};
    cuuint64_t strides[1] = {256};
    cuuint32_t box[2] = {64, 256};
    if (enc(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint8_t*>(qbase), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      set_last_error("b200dsa_indexer_flat_bf16_logits: cuTensorMapEncodeTiled rejected the queries");
      return B200DSA_ECUDA;
    }
    FlatParams p{};
    p.weights = weights + static_cast<int64_t>(r0) * kHq;
    p.pos_lo = pos_lo + r0;
    p.pos_hi = pos_hi + r0;
    p.row_cols = row_cols + r0;
    p.n_rows = nr;
    p.n_blocks = (n_keys + kFlatTile - 1) / kFlatTile;
    p.out_scale = out_scale;
    p.logits = logits + static_cast<int64_t>(r0) * logits_stride;
    p.logits_stride = logits_stride;
    p.logits_cols = max_cols;
    p.status = status;
    e = launch_chained(indexer_flat_kernel<kHq>, dim3(sms), dim3(kFlatThreads), kFlatSmem, static_cast<cudaStream_t>(stream),
                       mk, mq, p);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_last_error(cudaGetErrorString(e));
      return B200DSA_ECUDA;
    }
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_indexer_flat_bf16_logits(const void* q_bf16, const float* weights, const void* keys_bf16,
                                                int32_t n_keys, const int32_t* pos_lo, const int32_t* pos_hi,
                                                const int32_t* row_cols, int32_t n_rows, int32_t max_cols,
                                                float out_scale, float* logits, int64_t logits_stride,
                                                int32_t* status, void* stream) {
  return flat_launch<kFlatHeads>(q_bf16, weights, keys_bf16, n_keys, pos_lo, pos_hi, row_cols, n_rows, max_cols,
                                 out_scale, logits, logits_stride, status, stream);
}

extern "C" int b200dsa_indexer_flat_bf16_logits_routed(const void* q8_bf16, const float* weights8,
                                                       const void* keys_bf16, int32_t n_keys, const int32_t* pos_lo,
                                                       const int32_t* pos_hi, const int32_t* row_cols,
                                                       int32_t n_rows, int32_t max_cols, float out_scale,
                                                       float* logits, int64_t logits_stride, int32_t* status,
                                                       void* stream) {
  return flat_launch<kRoutedHeads>(q8_bf16, weights8, keys_bf16, n_keys, pos_lo, pos_hi, row_cols, n_rows, max_cols,
                                   out_scale, logits, logits_stride, status, stream);
}

// ---------------------------------------------------------------------------------------------
// Causal intervals of packed queries in one launch (the reference builds them with a Python loop over the
// documents, OpenDSA/opendsa/ops/flashkl_warmup.py:41-56, or a searchsorted, :235-248; as separate torch
// operations they cost about fifteen launches in front of the logits kernel): for row t at position
// p = q_pos[t] (or t), doc = the last document whose start is <= p, lo = its start, hi = p + 1, and the
// column frame of the logits kernels: col0 = lo rounded down to a 128-key block, row_cols = blocks covering
// [col0, hi) in keys.
// ---------------------------------------------------------------------------------------------
namespace b200dsa {
__global__ void __launch_bounds__(256) causal_row_intervals_kernel(const int32_t* __restrict__ cu, int n_cu,
                                                                   const int32_t* __restrict__ q_pos, int n_rows,
                                                                   int32_t* __restrict__ lo, int32_t* __restrict__ hi,
                                                                   int32_t* __restrict__ col0,
                                                                   int32_t* __restrict__ row_cols) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_rows) return;
  const int p = q_pos ? q_pos[t] : t;
  // first index whose start is > p (searchsorted right), minus one, kept inside the documents
  int a = 0, b = n_cu;
  while (a < b) {
    const int m = (a + b) >> 1;
    if (__ldg(cu + m) <= p) a = m + 1; else b = m;
  }
  int d = a - 1;
  d = max(0, min(d, n_cu - 2));
  const int s = __ldg(cu + d);
  const int e = p + 1;
  const int c0 = (s >> 7) << 7;
  lo[t] = s;
  hi[t] = e;
  col0[t] = c0;
  row_cols[t] = max(0, (((e + 127) >> 7) << 7) - c0);
}
}  // namespace b200dsa

extern "C" int b200dsa_causal_row_intervals(const int32_t* cu_seqlens, int32_t n_cu, const int32_t* q_pos,
                                            int32_t n_rows, int32_t* lo, int32_t* hi, int32_t* col0,
                                            int32_t* row_cols, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!cu_seqlens || n_cu < 2 || n_rows < 0 || !lo || !hi || !col0 || !row_cols) {
    set_last_error("b200dsa_causal_row_intervals: bad argument (cu_seqlens needs at least two entries)");
    return B200DSA_EINVAL;
  }
  causal_row_intervals_kernel<<<(n_rows + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      cu_seqlens, n_cu, q_pos, n_rows, lo, hi, col0, row_cols);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
