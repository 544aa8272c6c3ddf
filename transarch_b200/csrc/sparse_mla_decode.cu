// Sparse MLA attention in the absorbed latent space, one query token per work item.
//
//   s[h, j]  = sm_scale * <q[h, 0:576], kv[idx_j, 0:576]>          (j over the selected keys)
//   p        = softmax_j(s)  over valid j
//   ctx[h,:] = sum_j p[h, j] * kv[idx_j, 0:512]                    (latent-space context)
//   lse[h]   = log sum_j exp(s[h, j])
//
// Work split: CTA (item, hh) computes heads [64*hh, 64*hh+64) of one item over all selected
// keys.  Heads are the UMMA M dimension (M = 64: accumulator row m lives in TMEM lane
// 32*(m/16) + m%16, i.e. the lower half of each 32-lane sub-partition), 64 gathered keys are
// N of the score MMA and K of the value MMA.  TMEM plan (512 columns):
//   lower half-lanes, columns 0..511 : O accumulator (64 x 512 fp32)
//   upper half-lanes, columns 0..127 : two score buffers (64 x 64 fp32 each)
//   upper half-lanes, columns 128..415: Q (64 x 576 bf16, two per cell), the A operand of the
//                                        score MMA, stored once by the softmax threads
// The 576-wide rows are gathered with 16-byte cp.async into the 128-byte-swizzled K-major layout
// the score MMA reads; the same bytes serve, read MN-major, as the value operand.  Softmax:
// lane 16+i of warp 4+w owns head row 16w+i (row max / sum are thread-local); lane i of the
// same warp owns that row of O.
//
// Roles (288 threads): warps 0-3 gather (warp w owns 16 rows of every tile, one row per three
// instructions), warps 4-7 softmax, warp 8 issues the score and the value MMAs.
// All waits are bounded.
#include "sparse_mla.cuh"

namespace b200dsa {

__global__ void __launch_bounds__(kMlaThreads, 1)
sparse_mla_decode_kernel(const MlaParams p) {
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ uint32_t s_mask[kMlaStages][2];  // validity bit per key of the stage

  const int item = blockIdx.x >> 1;
  const int hh = blockIdx.x & 1;
  auto signal_peers = [&]() { mla_signal_peers(p); };
  if (hh * kMlaHeadsTile >= p.n_heads) {  // nothing to do for this head half (whole CTA)
    signal_peers();
    return;
  }

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const uint32_t kv_addr = smem_base;
  const uint32_t p_addr = kv_addr + kMlaStages * kMlaStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + kMlaStages * kMlaStageBytes + kMlaPBytes);
  uint64_t* q_full = bars;                       // [1]
  uint64_t* s_full = bars + 1;                   // [2] score MMA retired
  uint64_t* s_empty = bars + 3;                  // [2] 128 softmax-warp threads have read the scores
  uint64_t* p_full = bars + 5;                   // [1] 128 softmax-warp threads: P written
  uint64_t* pv_done = bars + 6;                  // [1] value MMA retired (P buffer free, O stable)
  uint64_t* kv_full = bars + 7;                  // [stages] 128 gather threads (arrivals of their copies)
  uint64_t* kv_empty = bars + 7 + kMlaStages;    // [stages] value MMA retired
  uint64_t* q_land = bars + 7 + 2 * kMlaStages;  // [1] bytes of the Q rows

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_idx = p.n_idx_item ? max(0, min(p.n_idx, p.n_idx_item[blockIdx.x >> 1])) : p.n_idx;
  const int n_tiles = (n_idx + kMlaTile - 1) / kMlaTile;
  volatile int* abort_flag = &s_abort;

  if (tid == 0) {
    s_abort = 0;
    mbar_init(q_full, 128);   // the softmax threads, once Q sits in TMEM
    for (int s = 0; s < kMlaStages; ++s) {
      mbar_init(&kv_full[s], 128);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    mbar_init(q_land, 1);
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(&s_tmem_base, kMlaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  const int qpos = p.q_pos ? p.q_pos[item] + p.q_pos_bias : 0x7fffffff;
  const int64_t row_base = (p.kv_row_base ? p.kv_row_base[item] : 0) - p.pos_lo;

  if (warp < 4) {
    // ------------------------------------------------------------------ gather producers
    // Warp w gathers rows 8w..8w+7 of every 32-key tile.  A row (1152 B) is copied by the whole
    // warp in three instructions (32 + 32 + 8 lanes x 16 B), so that one instruction touches at
    // most four consecutive 128-byte lines; lanes 0..7 hold the row indices, fetched one tile ahead.
    const int32_t* idx_row = p.indices + static_cast<int64_t>(item) * p.idx_stride;
    constexpr int kRowsPerWarp = kMlaTile / 4;   // 8 or 16
    const int r0 = warp * kRowsPerWarp;
    auto load_idx = [&](int t) {
      const int j = t * kMlaTile + r0 + lane;
      return (lane < kRowsPerWarp && j < n_idx) ? __ldg(idx_row + j) : -1;
    };
    int idx_next = load_idx(0);
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % kMlaStages;
      const int idx = idx_next;
      if (t + 1 < n_tiles) idx_next = load_idx(t + 1);
      bool valid = idx >= 0 && idx <= qpos && idx >= p.pos_lo && idx < p.pos_hi;
      const int64_t grow = row_base + idx;
      if (valid && (grow < 0 || grow >= p.kv_rows)) {
        valid = false;
        atomicMax(p.status, kDevBadIndex);
      }
      bool ok = mbar_wait(&kv_empty[s], ((t / kMlaStages) & 1) ^ 1, abort_flag);
      // the tail of the ring holds the Q rows until the softmax threads have moved them to TMEM
      if (t < kMlaStages && (t + 1) * kMlaStageBytes > kMlaQStageOff) ok = ok && mbar_wait(q_full, 0, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) break;
      const unsigned vmask = __ballot_sync(0xffffffffu, valid) & ((1u << kRowsPerWarp) - 1u);
      const uint32_t stage_addr = kv_addr + s * kMlaStageBytes;
#pragma unroll
      for (int rr = 0; rr < kRowsPerWarp; ++rr) {
        const int64_t g = __shfl_sync(0xffffffffu, grow, rr);
        const bool v = (vmask >> rr) & 1u;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.kv) + (v ? g : 0) * (kMlaD * 2);
        const int r = r0 + rr;
        const uint32_t dst_row = stage_addr + r * 128;
#pragma unroll
        for (int u = 0; u < 3; ++u) {
          const int c16 = lane + 32 * u;          // 16-byte chunk of the 1152-byte row
          if (c16 < 72) {
            const int c = c16 >> 3, w8 = c16 & 7;  // 128-byte chunk, position inside it
            cp_async_16(dst_row + c * kMlaChunkBytesK + ((w8 ^ (r & 7)) << 4), src + c16 * 16, v);
          }
        }
      }
      if (lane == 0) {
        if constexpr (kRowsPerWarp == 8) reinterpret_cast<volatile uint8_t*>(&s_mask[s][0])[warp] = static_cast<uint8_t>(vmask);
        else reinterpret_cast<volatile uint16_t*>(&s_mask[s][0])[warp] = static_cast<uint16_t>(vmask);
      }
      __threadfence_block();
      __syncwarp();
      // the barrier receives this thread's arrival once all its copies above have landed
      cp_async_mbar_arrive(&kv_full[s]);
    }
    cp_async_wait_all();
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax
    // lanes 16..31: score row `row`; lanes 0..15: the same row of O (partner lane = lane ^ 16)
    const int wq = warp & 3;
    const int row = wq * 16 + (lane & 15);          // head row inside this CTA's 64
    const bool is_s = lane >= 16;
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;  // sub-partition base lane
    float m_ref = -INFINITY, l = 0.f;
    bool aborted = false;
    {
      // Q -> TMEM once.  The 64 rows of this CTA (72 KB) are fetched by one bulk copy per row into the
      // tail of the key ring, which the gather does not touch before q_full (rows padded by 16 bytes so
      // that one row per lane reads without bank conflicts; the last row spills into the P tile, unused
      // so far): one memory round trip instead of nine dependent ones.  Then lane 16+i of this warp
      // stores head row 16*wq+i into the upper half-lanes (two bf16 per 32-bit cell, 288 cells per row).
      // The lower half-lanes of these columns belong to O, which nothing has written yet.
      const int qhead = hh * kMlaHeadsTile + row;
      const bool have = is_s && qhead < p.n_heads;
      const int rows_have = min(kMlaHeadsTile, p.n_heads - hh * kMlaHeadsTile);
      if (warp == 4) {
        if (lane == 0) mbar_arrive_expect_tx(q_land, static_cast<uint32_t>(rows_have) * (kMlaD * 2));
        __syncwarp();
        const __nv_bfloat16* q0 = p.q + (static_cast<int64_t>(item) * p.n_heads + hh * kMlaHeadsTile) * kMlaD;
        for (int r = lane; r < rows_have; r += 32)
          bulk_load_1d(smem_al + kMlaQStageOff + r * kMlaQRowBytes, q0 + static_cast<int64_t>(r) * kMlaD, kMlaD * 2, q_land);
      }
      const bool okq = mbar_wait(q_land, 0, abort_flag);
      aborted = !__all_sync(0xffffffffu, okq);
      const uint32_t qrow = smem_base + kMlaQStageOff + row * kMlaQRowBytes;
#pragma unroll 1
      for (int c = 0; c < kMlaD / 64 && !aborted; ++c) {
        uint32_t qv[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (have) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(qv[4 * j]), "=r"(qv[4 * j + 1]), "=r"(qv[4 * j + 2]), "=r"(qv[4 * j + 3])
                         : "r"(qrow + c * 128 + j * 16));
          } else {
            qv[4 * j] = qv[4 * j + 1] = qv[4 * j + 2] = qv[4 * j + 3] = 0u;
          }
        }
        tmem_st_32x32(tmem_base + lane_addr + 128 + c * 32, qv);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(q_full);
    }
    for (int t = 0; t < n_tiles && !aborted; ++t) {
      const int sb = t & 1;
      bool ok = mbar_wait(&s_full[sb], (t >> 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
      tc_fence_after();
      const int ks = t % kMlaStages;
      constexpr int kNV = kMlaTile / 32;   // 32-column groups per tile
      uint32_t v[kNV][32];
#pragma unroll
      for (int h = 0; h < kNV; ++h)
        tmem_ld_32x32(tmem_base + lane_addr + sb * kMlaTile + 32 * h, v[h]);   // lanes 16-31: score rows
      tc_wait_ld();
      float mt = -INFINITY;   // tile maximum of the raw scores, scaled once below (the scale is positive)
#pragma unroll
      for (int h = 0; h < kNV; ++h) {
        const uint32_t mk = s_mask[ks][h];
        if (mk == 0xffffffffu) {   // common case: all 32 keys of the group are valid
#pragma unroll
          for (int j = 0; j < 32; ++j) mt = fmaxf(mt, __uint_as_float(v[h][j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float a = ((mk >> j) & 1u) ? __uint_as_float(v[h][j]) : -INFINITY;
            v[h][j] = __float_as_uint(a);
            mt = fmaxf(mt, a);
          }
        }
      }
      mt *= p.scale_log2;
      if (!is_s) mt = -INFINITY;
      bool waited_pv = false;
      // lazy rescale: only when the running maximum grows by more than 2^8
      const bool grow = is_s && (mt > m_ref + 8.0f);
      if (__any_sync(0xffffffffu, grow) && t > 0) {
        ok = mbar_wait(pv_done, (t - 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
        waited_pv = true;
        if (t + 1 < n_tiles) {
          // the write-back below also touches the upper half-lanes of columns 0..127, where the
          // next tile's scores may still be landing: let that MMA finish first
          ok = mbar_wait(&s_full[(t + 1) & 1], ((t + 1) >> 1) & 1, abort_flag);
          if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
        }
        tc_fence_after();
        float f = grow ? ((m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mt)) : 1.0f;
        if (is_s) l *= f;
        f = __shfl_xor_sync(0xffffffffu, f, 16);   // O-row lanes take the factor of their partner
#pragma unroll 1
        for (int c = 0; c < kMlaDv / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + lane_addr + kMlaTmemO + c * 32, o);
          tc_wait_ld();
          if (!is_s) {
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
          }
          // upper lanes write back what they read (score buffers and unused cells)
          tmem_st_32x32(tmem_base + lane_addr + kMlaTmemO + c * 32, o);
        }
        tc_wait_st();
        tc_fence_before();
      }
      // Only now may the score issuer overwrite this buffer (two tiles ahead): the write-back of a
      // rescale above also touches the score cells.
      tc_fence_before();
      mbar_arrive(&s_empty[sb]);
      if (grow) m_ref = mt;
      uint32_t pk[kMlaTile / 2];
      float lsum = 0.f;
      // p = 2^(s*scale - m_ref) as one FMA and one ex2; masked scores are -inf and give exactly 0
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
#pragma unroll
      for (int h = 0; h < kNV; ++h) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[h][j]), p.scale_log2, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(v[h][j + 1]), p.scale_log2, neg_m));
          lsum += p0 + p1;
          __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1);
          pk[16 * h + (j >> 1)] = *reinterpret_cast<uint32_t*>(&h01);
        }
      }
      if (is_s) l += lsum;
      if (t > 0 && !waited_pv) {
        ok = mbar_wait(pv_done, (t - 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
      }
      if (is_s) {
        // P row (tile bf16) as core-matrix rows of 16 bytes: (row/8)*(tile/8*128) + c*128 + (row%8)*16
        const uint32_t prow = p_addr + (row >> 3) * (kMlaTile / 8 * 128) + (row & 7) * 16;
#pragma unroll
        for (int c = 0; c < kMlaTile / 8; ++c) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + c * 128), "r"(pk[4 * c]),
                       "r"(pk[4 * c + 1]), "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3])
                       : "memory");
        }
      }
      fence_proxy_async();
      mbar_arrive(p_full);
    }
    // ---- output: lanes 0..15 own the O rows; l and m_ref come from the partner lane
    const float l_o = __shfl_xor_sync(0xffffffffu, l, 16);
    const float m_o = __shfl_xor_sync(0xffffffffu, m_ref, 16);
    const int head = hh * kMlaHeadsTile + row;
    const int64_t ctx_off = (static_cast<int64_t>(item) * p.n_heads + head) * kMlaDv;
    float* ctx_row = static_cast<float*>(p.ctx) + ctx_off;
    __nv_bfloat16* ctx_row_h = static_cast<__nv_bfloat16*>(p.ctx) + ctx_off;
    const bool write = !is_s && head < p.n_heads;
    if (n_tiles == 0 || aborted) {
      if (write && !aborted) {
        if (p.ctx_bf16) {
          for (int j = 0; j < kMlaDv; j += 8) *reinterpret_cast<uint4*>(ctx_row_h + j) = make_uint4(0, 0, 0, 0);
        } else {
          for (int j = 0; j < kMlaDv; j += 4) *reinterpret_cast<float4*>(ctx_row + j) = make_float4(0, 0, 0, 0);
        }
        p.lse[static_cast<int64_t>(item) * p.n_heads + head] = -INFINITY;
      }
    } else {
      const bool ok = mbar_wait(pv_done, (n_tiles - 1) & 1, abort_flag);
      if (__all_sync(0xffffffffu, ok)) {
        tc_fence_after();
        const float inv = (l_o > 0.f) ? 1.0f / l_o : 0.f;
#pragma unroll 1
        for (int c = 0; c < kMlaDv / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + lane_addr + kMlaTmemO + c * 32, o);
          tc_wait_ld();
          if (write && p.ctx_bf16) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
              *reinterpret_cast<uint4*>(ctx_row_h + c * 32 + j) = v;
            }
          } else if (write) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              *reinterpret_cast<float4*>(ctx_row + c * 32 + j) =
                  make_float4(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv,
                              __uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
            }
          }
        }
        tc_fence_before();
        if (write)
          p.lse[static_cast<int64_t>(item) * p.n_heads + head] =
              (l_o > 0.f) ? (m_o + log2f(l_o)) * 0.6931471805599453f : -INFINITY;
      }
    }
  } else {
    // ------------------------------------------------------------------ MMA issuer (warp 8)
    // One warp issues everything, in the order S(0), S(1), PV(0), S(2), PV(1), ...: the tensor pipe runs
    // its instructions in issue order, so S(t+1) keeps it busy while the softmax of tile t runs, and the
    // ring stage that PV(t-1) frees is not needed before S(t+2), a whole tile of tensor work later, which
    // is the time the gather of tile t+2 has to land.  (Issuing the scores as early as their buffers allow
    // puts S(t+2) directly behind PV(t-1) and exposes the whole gather latency on every tile.)
    constexpr uint32_t idesc_s = make_idesc(kFmtBF16, kFmtBF16, kMlaHeadsTile, kMlaTile);
    constexpr uint32_t idesc_pv = make_idesc(kFmtBF16, kFmtBF16, kMlaHeadsTile, 256, 0, 1);
    auto issue_scores = [&](int t) -> bool {
      const int s = t % kMlaStages, sb = t & 1;
      const bool w = mbar_wait(&kv_full[s], (t / kMlaStages) & 1, abort_flag) &&
                     mbar_wait(&s_empty[sb], ((t >> 1) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, w)) return false;
      fence_proxy_async();  // gathered rows were written through the generic proxy
      tc_fence_after();
      if (elect_one()) {
        const uint32_t d = tmem_base + kMlaTmemS + sb * kMlaTile;
        // descriptors differ only in the 16-byte-granular start address: one add per operand
        const uint64_t b0 = make_desc_k_sw128(kv_addr + s * kMlaStageBytes);
#pragma unroll
        for (int c = 0; c < kMlaChunks; ++c) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            mma_f16_ts(d, tmem_base + kMlaTmemQ + c * 32 + kk * 8, b0 + ((c * kMlaChunkBytesK + kk * 32) >> 4),
                       idesc_s, (c | kk) != 0);
          }
        }
        tc_commit(&s_full[sb]);
      }
      __syncwarp();
      return true;
    };
    bool ok = mbar_wait(q_full, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_tiles > 0) ok = issue_scores(0);
    for (int t = 0; ok && t < n_tiles; ++t) {
      if (t + 1 < n_tiles && !issue_scores(t + 1)) break;
      const int s = t % kMlaStages;
      const bool w = mbar_wait(p_full, t & 1, abort_flag);
      if (!__all_sync(0xffffffffu, w)) break;
      fence_proxy_async();
      tc_fence_after();
      if (elect_one()) {
        const uint64_t pa0 = make_desc_k_noswz(p_addr, 128, kMlaTile / 8 * 128);
        const uint64_t vb0 = make_desc_mn_sw128(kv_addr + s * kMlaStageBytes, kMlaChunkBytesK, 1024);
#pragma unroll
        for (int j = 0; j < kMlaTile / 16; ++j) {  // 16 keys per MMA
#pragma unroll
          for (int nh = 0; nh < 2; ++nh) {        // value dims [256*nh, 256*nh+256)
            mma_f16_ss(tmem_base + kMlaTmemO + nh * 256, pa0 + ((j * 256) >> 4),
                       vb0 + (((4 * nh) * kMlaChunkBytesK + j * 2048) >> 4), idesc_pv, (t | j) != 0);
          }
        }
        tc_commit(&kv_empty[s]);
        tc_commit(pv_done);
      }
      __syncwarp();
    }
  }

  // ---------------------------------------------------------------------- common tail
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 8) tmem_dealloc(tmem_base, kMlaTmemCols);
  if (tid == 0 && s_abort) atomicMax(p.status, kDevWaitTimeout);
  signal_peers();
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

static int mla_decode_launch(const void* q_bf16, const void* kv_bf16, int64_t kv_rows, const int64_t* kv_row_base,
                             const int32_t* indices, int64_t idx_stride, int32_t n_idx, const int32_t* n_idx_item,
                             const int32_t* q_pos, int32_t q_pos_bias, int32_t pos_lo, int32_t pos_hi, int32_t n_items,
                             int32_t n_heads, float sm_scale, void* ctx, int32_t ctx_bf16, float* lse, int32_t* status,
                             const PeerLinkDev* link, int32_t* ticket, int use_pair, void* stream);

extern "C" int b200dsa_sparse_mla_decode(const void* q_bf16, const void* kv_bf16, int64_t kv_rows,
                                         const int64_t* kv_row_base, const int32_t* indices, int64_t idx_stride,
                                         int32_t n_idx, const int32_t* n_idx_item, const int32_t* q_pos,
                                         int32_t q_pos_bias, int32_t pos_lo, int32_t pos_hi,
                                         int32_t n_items, int32_t n_heads, float sm_scale, void* ctx, int32_t ctx_bf16,
                                         float* lse, int32_t* status, void* stream) {
  return mla_decode_launch(q_bf16, kv_bf16, kv_rows, kv_row_base, indices, idx_stride, n_idx, n_idx_item, q_pos,
                           q_pos_bias, pos_lo, pos_hi, n_items, n_heads, sm_scale, ctx, ctx_bf16, lse, status, nullptr,
                           nullptr, 0, stream);
}

extern "C" int b200dsa_sparse_mla_decode_pair(const void* q_bf16, const void* kv_bf16, int64_t kv_rows,
                                              const int64_t* kv_row_base, const int32_t* indices, int64_t idx_stride,
                                              int32_t n_idx, const int32_t* n_idx_item, const int32_t* q_pos,
                                              int32_t q_pos_bias, int32_t pos_lo, int32_t pos_hi, int32_t n_items,
                                              int32_t n_heads, float sm_scale, void* ctx, int32_t ctx_bf16, float* lse,
                                              int32_t* status, void* stream) {
  return mla_decode_launch(q_bf16, kv_bf16, kv_rows, kv_row_base, indices, idx_stride, n_idx, n_idx_item, q_pos,
                           q_pos_bias, pos_lo, pos_hi, n_items, n_heads, sm_scale, ctx, ctx_bf16, lse, status, nullptr,
                           nullptr, 1, stream);
}

extern "C" int b200dsa_sparse_mla_decode_signal(const void* q_bf16, const void* kv_bf16, int64_t kv_rows,
                                                const int64_t* kv_row_base, const int32_t* indices,
                                                int64_t idx_stride, int32_t n_idx, const int32_t* n_idx_item,
                                                const int32_t* q_pos, int32_t q_pos_bias, int32_t pos_lo,
                                                int32_t pos_hi, int32_t n_items, int32_t n_heads, float sm_scale,
                                                void* ctx, int32_t ctx_bf16, float* lse,
                                                const b200dsa_peer_link* link, int32_t* ticket, int32_t* status,
                                                void* stream) {
  PeerLinkDev dev_link;
  if (!ticket || n_items < 1) {
    set_last_error("b200dsa_sparse_mla_decode_signal: ticket is required and n_items >= 1");
    return B200DSA_EINVAL;
  }
  // the flag words of the combine kernel itself are used: slot 0
  b200dsa_peer_link l = *link;
  if (l.slot != 0) {
    set_last_error("b200dsa_sparse_mla_decode_signal: the link must name slot 0, the combine kernel's 'ready' flags");
    return B200DSA_EINVAL;
  }
  l.slot = 1;   // validated as an ordinary slot, then set back
  if (!make_link(&l, &dev_link, "b200dsa_sparse_mla_decode_signal")) return B200DSA_EINVAL;
  dev_link.slot = 0;
  return mla_decode_launch(q_bf16, kv_bf16, kv_rows, kv_row_base, indices, idx_stride, n_idx, n_idx_item, q_pos,
                           q_pos_bias, pos_lo, pos_hi, n_items, n_heads, sm_scale, ctx, ctx_bf16, lse, status, &dev_link,
                           ticket, 0, stream);
}

static int mla_decode_launch(const void* q_bf16, const void* kv_bf16, int64_t kv_rows, const int64_t* kv_row_base,
                             const int32_t* indices, int64_t idx_stride, int32_t n_idx, const int32_t* n_idx_item,
                             const int32_t* q_pos, int32_t q_pos_bias, int32_t pos_lo, int32_t pos_hi, int32_t n_items,
                             int32_t n_heads, float sm_scale, void* ctx, int32_t ctx_bf16, float* lse, int32_t* status,
                             const PeerLinkDev* link, int32_t* ticket, int use_pair, void* stream) {
  if (n_items == 0) return B200DSA_OK;
  if (!q_bf16 || !kv_bf16 || !indices || !ctx || !lse || !status || n_items < 0 || n_heads < 1 ||
      n_heads > kMlaMaxHeads || n_idx < 0 || idx_stride < n_idx || kv_rows < 1 || pos_hi < pos_lo) {
    set_last_error("b200dsa_sparse_mla_decode: bad argument (1 <= n_heads <= 128, idx_stride >= n_idx)");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(q_bf16) & 15) || (reinterpret_cast<uintptr_t>(kv_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(ctx) & 15)) {
    set_last_error("b200dsa_sparse_mla_decode: q, kv and ctx must be 16-byte aligned");
    return B200DSA_EALIGN;
  }
  cudaError_t e = cudaFuncSetAttribute(sparse_mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kMlaSmemBytes);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  MlaParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q_bf16);
  p.kv = static_cast<const __nv_bfloat16*>(kv_bf16);
  p.kv_rows = kv_rows;
  p.kv_row_base = kv_row_base;
  p.indices = indices;
  p.idx_stride = idx_stride;
  p.n_idx = n_idx;
  p.n_idx_item = n_idx_item;
  p.q_pos = q_pos;
  p.q_pos_bias = q_pos_bias;
  p.pos_lo = pos_lo;
  p.pos_hi = pos_hi;
  p.n_items = n_items;
  p.n_heads = n_heads;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.ctx = ctx;
  p.ctx_bf16 = ctx_bf16;
  p.lse = lse;
  p.status = status;
  if (link) {
    p.signal_on = 1;
    p.link = *link;
    p.ticket = ticket;
  }
  if (use_pair) {
    // the cluster-of-two kernel that keeps all heads of an item in one M = 128 tile
    e = static_cast<cudaError_t>(mla_pair_launch(p, static_cast<cudaStream_t>(stream)));
  } else {
    e = launch_chained(sparse_mla_decode_kernel, dim3(n_items * 2), dim3(kMlaThreads), kMlaSmemBytes,
                       static_cast<cudaStream_t>(stream), p);
    if (e == cudaSuccess) e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
