// Sparse MLA attention in the absorbed latent space, cluster-of-two form: all 128 heads of an item are the
// UMMA M dimension (the tensor pipe runs M = 64 at half rate), and the two CTAs of a cluster split the
// latent dimensions instead of the heads.  An alternative to sparse_mla_decode_kernel with the same results,
// reached through b200dsa_sparse_mla_decode_pair only: at 64 items x 128 heads x 2048 keys it takes 86 us
// where the head-split kernel takes 63 us, because what crosses the cluster (24 KB per tile and CTA) moves at
// about 10 bytes per cycle, whether as bulk copies (about 1 200 cycles from issue to the receiver's barrier
// for 9 KB) or as stores with barrier completion (st.async: slower still), and because the exchange buffers
// leave shared memory for three gather stages only.
//
// CTA c of the pair owns value dims [256c, 256c + 256) and rope dims [512 + 32c, 512 + 32c + 32): it gathers
// only those 576 bytes of every selected row (so a row crosses the memory system once per item, not twice),
// holds the matching half of Q (value part in tensor memory, rope part in shared memory) and computes
//   S_c[h, j] = <q[h, dims_c], kv[idx_j, dims_c]>            M = 128 heads, N = 64 keys, K = 288
//   O_c[h, :] += P[h, j] * kv[idx_j, 256c : 256c + 256]      M = 128, N = 256, K = 64 keys
// The scores need both halves: S = S_0 + S_1.  CTA c runs the softmax of heads [64c, 64c + 64): the other CTA
// sends its partial scores of those heads into this CTA's shared memory, this CTA adds them, exponentiates,
// and puts the bf16 probabilities of its heads into the P tile of BOTH CTAs, together with the factor by
// which a grown row maximum rescales O.  The transfers are bulk copies from local shared memory into the
// partner's (one destination CTA each, no multicast) that complete on a barrier of the receiver.
//
// Buffer reuse needs no extra signals: the MMA warp issues S(0), S(1), PV(0), S(2), PV(1), ... and the tensor
// pipe retires in issue order, so "S(t) of a CTA has completed" (which the receipt of its partial scores
// proves) implies that its PV(t-2) has completed and its P tile / factor row / receive buffer of parity t&1
// are free again.
//
// Tensor memory (512 columns, lane = head): O 0..255, two score buffers 256..383, Q value half 384..511.
// Roles (416 threads): warps 0-3 gather; warps 4-11 by lane quadrant (= warp % 4): in the two quadrants whose
// heads this CTA owns, two softmax warps (one per 32 keys of the tile); in the other two, a sender of the
// partial scores and a rescaler of O; warp 12 issues the MMAs.  Every wait is bounded; a CTA that gives up
// also raises the abort flag of its partner, and both reach the closing cluster barrier.
#include "sparse_mla.cuh"

namespace b200dsa {

constexpr int kPairThreads = 416;
constexpr int kPairHeads = 128;
constexpr int kPairStages = 3;
constexpr int kPairVChunks = 4;                                // 64-dim value chunks per CTA
constexpr int kPairRopeBytes = kMlaTile * 64;                  // 32 rope dims per key, K-major core matrices
constexpr int kPairStageBytes = kPairVChunks * kMlaChunkBytesK + kPairRopeBytes;
constexpr int kPairRingBytes = kPairStages * kPairStageBytes;
constexpr int kPairPBytes = kPairHeads * kMlaTile * 2;         // bf16 P tile, 128 heads x 64 keys
// partial scores of 64 heads x 64 keys in fp32: [head half][key half][32 heads][32 keys + 4 words of padding], so that
// a thread reads and writes its head's 32 keys as eight conflict-free 16-byte vectors
constexpr int kPairRecvRow = 32 * 4 + 16;
constexpr int kPairRecvBlock = 32 * kPairRecvRow;              // one key half of 32 heads
constexpr int kPairRecvBytes = 4 * kPairRecvBlock;
constexpr int kPairQrBytes = kPairHeads * 32 * 2;              // rope half of Q, K-major core matrices
constexpr int kPairOffP = kPairRingBytes;
constexpr int kPairOffRecv = kPairOffP + 2 * kPairPBytes;
constexpr int kPairOffSend = kPairOffRecv + 2 * kPairRecvBytes;   // partial scores on their way to the partner
constexpr int kPairOffQr = kPairOffSend + 2 * kPairRecvBytes;
constexpr int kPairOffFac = kPairOffQr + kPairQrBytes;         // [2][128] fp32
constexpr int kPairOffFin = kPairOffFac + 2 * kPairHeads * 4;  // l[2][128], m[128] fp32
constexpr int kPairOffBars = kPairOffFin + 3 * kPairHeads * 4;
constexpr int kPairSmemBytes = kPairOffBars + 256 + 1024;
// Q staging in the tail of the ring (exactly the last two stages): per head row 512 value bytes + 64 rope bytes
constexpr int kPairQRowBytes = 512 + 64;
constexpr int kPairQStageOff = kPairRingBytes - kPairHeads * kPairQRowBytes;
static_assert(kPairQStageOff >= 0 && kPairQStageOff % 16 == 0, "Q staging must lie inside the ring");
constexpr uint32_t kPairTmemO = 0, kPairTmemS = 256, kPairTmemQ = 384;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_b32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// Bulk copy from this CTA's shared memory into another CTA of the cluster (one destination); the bytes are
// counted on a barrier of the destination CTA.  Addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes,
                                                 uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   dst_cluster),
               "r"(src_cta), "r"(bytes), "r"(bar_cluster)
               : "memory");
}


// Bounded wait of the pair kernel: as mbar_wait, and a timeout also raises the partner's abort flag (a
// shared::cluster address).  Every lane waits for itself: with one polling lane per warp and a shuffle the
// kernel ran 1.6 times slower.
__device__ __forceinline__ bool pair_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t partner_abort) {
  long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_test(bar, parity)) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitCycles) {
        *abort_flag = 1;
        st_cluster_b32(partner_abort, 1u);
        return false;
      }
    }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
sparse_mla_pair_kernel(const MlaParams p) {
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ uint32_t s_mask[kPairStages][2];  // validity bit per key of the stage

  const int item = blockIdx.x >> 1;
  const uint32_t c = cluster_ctarank();        // which half of the latent dims
  const uint32_t peer = c ^ 1u;

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const uint32_t kv_addr = smem_base;
  const uint32_t p_addr = smem_base + kPairOffP;
  const uint32_t recv_addr = smem_base + kPairOffRecv;
  const uint32_t send_addr = smem_base + kPairOffSend;
  const uint32_t qr_addr = smem_base + kPairOffQr;
  float* fac = reinterpret_cast<float*>(smem_al + kPairOffFac);     // [2][128]
  float* fin = reinterpret_cast<float*>(smem_al + kPairOffFin);     // l[2][128], m[128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + kPairOffBars);
  uint64_t* q_full = bars;                        // [1] 8 exchange warps: Q sits in TMEM / shared memory
  uint64_t* q_land = bars + 1;                    // [1] bytes of the staged Q rows
  uint64_t* s_full = bars + 2;                    // [2] score MMA retired
  uint64_t* s_empty = bars + 4;                   // [2] 8 exchange warps have read the partial scores
  uint64_t* recv_full = bars + 6;                 // [2] the partner's partial scores landed (16 KB)
  uint64_t* p_full = bars + 8;                    // [2] 4 local warps + the partner's P rows and factors (8448 B)
  uint64_t* o_ready = bars + 10;                  // [2] 8 exchange warps: O rescaled where needed
  uint64_t* pv_done = bars + 12;                  // [1] value MMA retired
  uint64_t* fin_bar = bars + 13;                  // [1] 4 local warps + the partner's row sums and maxima (768 B)
  uint64_t* kv_full = bars + 14;                  // [stages] 128 gather threads (arrivals of their copies)
  uint64_t* kv_empty = bars + 14 + kPairStages;   // [stages] value MMA retired

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_idx = p.n_idx_item ? max(0, min(p.n_idx, p.n_idx_item[item])) : p.n_idx;
  const int n_tiles = (n_idx + kMlaTile - 1) / kMlaTile;
  volatile int* abort_flag = &s_abort;
  const uint32_t partner_abort = map_to_cta(smem_u32(&s_abort), peer);

  if (tid == 0) {
    s_abort = 0;
    mbar_init(q_full, 8);
    mbar_init(q_land, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 6);     // four softmax warps, two senders
      mbar_init(&recv_full[s], 1);   // one arrival that states the bytes; the partner's copies bring them
      mbar_init(&p_full[s], 4);      // the local softmax warps; one of them states the partner's bytes
      mbar_init(&o_ready[s], 6);     // four softmax warps, two rescalers
    }
    mbar_init(pv_done, 1);
    mbar_init(fin_bar, 4);
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&kv_full[s], 128);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_fence_init();
  }
  if (warp == 12) {
    tmem_alloc(&s_tmem_base, kMlaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  const int qpos = p.q_pos ? p.q_pos[item] + p.q_pos_bias : 0x7fffffff;
  const int64_t row_base = (p.kv_row_base ? p.kv_row_base[item] : 0) - p.pos_lo;

  if (warp < 4) {
    // ------------------------------------------------------------------ gather producers
    // Warp w gathers rows 16w..16w+15 of every tile: per row one instruction for the 512 value bytes of this
    // CTA's half (32 lanes x 16 B), and one instruction per eight rows for their 64 rope bytes.
    const int32_t* idx_row = p.indices + static_cast<int64_t>(item) * p.idx_stride;
    const int r0 = warp * 16;
    auto load_idx = [&](int t) {
      const int j = t * kMlaTile + r0 + lane;
      return (lane < 16 && j < n_idx) ? __ldg(idx_row + j) : -1;
    };
    int idx_next = load_idx(0);
    const uint8_t* kv_bytes = reinterpret_cast<const uint8_t*>(p.kv);
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % kPairStages;
      const int idx = idx_next;
      if (t + 1 < n_tiles) idx_next = load_idx(t + 1);
      bool valid = idx >= 0 && idx <= qpos && idx >= p.pos_lo && idx < p.pos_hi;
      const int64_t grow = row_base + idx;
      if (valid && (grow < 0 || grow >= p.kv_rows)) {
        valid = false;
        atomicMax(p.status, kDevBadIndex);
      }
      bool ok = pair_wait(&kv_empty[s], ((t / kPairStages) & 1) ^ 1, abort_flag, partner_abort);
      // the tail of the ring holds the staged Q rows until the exchange threads have moved them
      if (t < kPairStages && (t + 1) * kPairStageBytes > kPairQStageOff)
        ok = ok && pair_wait(q_full, 0, abort_flag, partner_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      const unsigned vmask = __ballot_sync(0xffffffffu, valid) & 0xffffu;
      const uint32_t stage_addr = kv_addr + s * kPairStageBytes;
#pragma unroll
      for (int rr = 0; rr < 16; ++rr) {
        const int64_t g = __shfl_sync(0xffffffffu, grow, rr);
        const bool v = (vmask >> rr) & 1u;
        const uint8_t* src = kv_bytes + (v ? g : 0) * (kMlaD * 2) + c * 512 + lane * 16;
        const int r = r0 + rr;
        cp_async_16(stage_addr + (lane >> 3) * kMlaChunkBytesK + r * 128 + (((lane & 7) ^ (r & 7)) << 4), src, v);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int rr = 8 * i + (lane >> 2);
        const int64_t g = __shfl_sync(0xffffffffu, grow, rr);
        const bool v = (vmask >> rr) & 1u;
        const uint8_t* src = kv_bytes + (v ? g : 0) * (kMlaD * 2) + 1024 + c * 64 + (lane & 3) * 16;
        const int r = r0 + rr;
        cp_async_16(stage_addr + kPairVChunks * kMlaChunkBytesK + (r >> 3) * 512 + (lane & 3) * 128 + (r & 7) * 16, src, v);
      }
      if (lane == 0) reinterpret_cast<volatile uint16_t*>(&s_mask[s][0])[warp] = static_cast<uint16_t>(vmask);
      __threadfence_block();
      __syncwarp();
      cp_async_mbar_arrive(&kv_full[s]);
    }
    cp_async_wait_all();
  } else if (warp < 12) {
    // ------------------------------------------------------------------ exchange + softmax
    const int xw = warp - 4;
    const int q = xw & 3, hf = xw >> 2;                // lane quadrant (= warp % 4), column half
    const int row = q * 32 + lane;                     // head
    const bool own = static_cast<uint32_t>(q >> 1) == c;   // this CTA runs the softmax of the row
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool aborted = false;
    {
      // Q: one bulk copy per head row and part into the ring tail, then thread (row, hf) stores 128 bf16
      // of the value half into tensor memory (two per cell); hf = 1 also lays the 32 rope dims out as
      // K-major core matrices (8 rows x 16 bytes) for the two rope MMAs.
      const int rows_have = min(kPairHeads, p.n_heads);
      if (warp == 4) {
        if (lane == 0) mbar_arrive_expect_tx(q_land, static_cast<uint32_t>(rows_have) * 576u);
        __syncwarp();
        const uint8_t* q0 = reinterpret_cast<const uint8_t*>(p.q) + static_cast<int64_t>(item) * p.n_heads * (kMlaD * 2);
        for (int r = lane; r < rows_have; r += 32) {
          uint8_t* dst = smem_al + kPairQStageOff + r * kPairQRowBytes;
          bulk_load_1d(dst, q0 + static_cast<int64_t>(r) * (kMlaD * 2) + c * 512, 512, q_land);
          bulk_load_1d(dst + 512, q0 + static_cast<int64_t>(r) * (kMlaD * 2) + 1024 + c * 64, 64, q_land);
        }
      }
      const bool okq = pair_wait(q_land, 0, abort_flag, partner_abort);
      aborted = !__all_sync(0xffffffffu, okq);
      const bool have = row < p.n_heads;
      const uint32_t qrow = smem_base + kPairQStageOff + row * kPairQRowBytes;
#pragma unroll 1
      for (int cc = 0; cc < 2 && !aborted; ++cc) {
        uint32_t qv[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (have) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(qv[4 * j]), "=r"(qv[4 * j + 1]), "=r"(qv[4 * j + 2]), "=r"(qv[4 * j + 3])
                         : "r"(qrow + hf * 256 + cc * 128 + j * 16));
          } else {
            qv[4 * j] = qv[4 * j + 1] = qv[4 * j + 2] = qv[4 * j + 3] = 0u;
          }
        }
        tmem_st_32x32(tmem_base + lane_addr + kPairTmemQ + hf * 64 + cc * 32, qv);
      }
      if (hf == 1 && !aborted) {
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) {
          uint32_t a = 0, b = 0, cc2 = 0, d = 0;
          if (have) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(a), "=r"(b), "=r"(cc2), "=r"(d)
                         : "r"(qrow + 512 + kc * 16));
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(qr_addr + (row >> 3) * 512 + kc * 128 + (row & 7) * 16),
                       "r"(a), "r"(b), "r"(cc2), "r"(d)
                       : "memory");
        }
      }
      tc_wait_st();
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
    }
    // one lane of the softmax warps states, per tile, the bytes the partner will deliver to the two
    // barriers that receive bulk copies (that lane has seen the previous phase of each complete)
    const bool poster = own && hf == 0 && (q & 1) == 0 && lane == 0;
    const uint32_t half_off = (q & 1) * (2 * kPairRecvBlock);   // head half inside the owner's 64
    if (own) {
      // ---------------------------------------------------------------- softmax of this CTA's 64 heads
      for (int t = 0; t < n_tiles && !aborted; ++t) {
        const int sb = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (poster) mbar_arrive_expect_tx(&recv_full[sb], kPairRecvBytes);
        bool ok = pair_wait(&s_full[sb], ph, abort_flag, partner_abort);
        if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
        tc_fence_after();
        const int ks = t % kPairStages;
        // partial scores of this row: the other column half (only its maximum is needed), then ours
        uint32_t vo[32], v[32];
        tmem_ld_32x32(tmem_base + lane_addr + kPairTmemS + sb * kMlaTile + 32 * (hf ^ 1), vo);
        tmem_ld_32x32(tmem_base + lane_addr + kPairTmemS + sb * kMlaTile + 32 * hf, v);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[sb]);
        ok = pair_wait(&recv_full[sb], ph, abort_flag, partner_abort);
        if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
        const uint32_t rbase = recv_addr + sb * kPairRecvBytes + half_off + lane * kPairRecvRow;
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains
        {
          const uint32_t mk = s_mask[ks][hf ^ 1];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float r0, r1, r2, r3;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(r0), "=f"(r1), "=f"(r2), "=f"(r3)
                         : "r"(rbase + (hf ^ 1) * kPairRecvBlock + i * 16));
            const float a0 = __uint_as_float(vo[4 * i]) + r0, a1 = __uint_as_float(vo[4 * i + 1]) + r1;
            const float a2 = __uint_as_float(vo[4 * i + 2]) + r2, a3 = __uint_as_float(vo[4 * i + 3]) + r3;
            if (mk == 0xffffffffu) {
              mx[0] = fmaxf(mx[0], a0); mx[1] = fmaxf(mx[1], a1); mx[2] = fmaxf(mx[2], a2); mx[3] = fmaxf(mx[3], a3);
            } else {
              mx[0] = fmaxf(mx[0], ((mk >> (4 * i)) & 1u) ? a0 : -INFINITY);
              mx[1] = fmaxf(mx[1], ((mk >> (4 * i + 1)) & 1u) ? a1 : -INFINITY);
              mx[2] = fmaxf(mx[2], ((mk >> (4 * i + 2)) & 1u) ? a2 : -INFINITY);
              mx[3] = fmaxf(mx[3], ((mk >> (4 * i + 3)) & 1u) ? a3 : -INFINITY);
            }
          }
        }
        {
          const uint32_t mk = s_mask[ks][hf];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float r[4];
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3])
                         : "r"(rbase + hf * kPairRecvBlock + i * 16));
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float a = __uint_as_float(v[4 * i + e]) + r[e];
              if (mk != 0xffffffffu) a = ((mk >> (4 * i + e)) & 1u) ? a : -INFINITY;
              v[4 * i + e] = __float_as_uint(a);
              mx[e] = fmaxf(mx[e], a);
            }
          }
        }
        const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;   // the scale is positive
        // lazy rescale: only when the running maximum grows by more than 2^8
        float f = 1.0f;
        if (mt > m_ref + 8.0f) {
          const float g = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mt);
          l *= g;
          if (t > 0) f = g;   // O holds nothing before the first value MMA
          m_ref = mt;
        }
        const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
        uint32_t pk[16];
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[j]), p.scale_log2, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(v[j + 1]), p.scale_log2, neg_m));
          ls[(j >> 1) & 3] += p0 + p1;
          pk[j >> 1] = pack_bf16x2(p0, p1);
        }
        l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        // P tile: [key half][16 groups of 8 heads][4 core matrices of 8 keys][8 heads x 16 bytes]; the warp's
        // 32 heads x 32 keys are 2 KB in one piece, which lane 0 then copies into the partner's tile
        const uint32_t pwarp = p_addr + sb * kPairPBytes + hf * 8192 + q * 2048;
        const uint32_t prow = pwarp + (lane >> 3) * 512 + (lane & 7) * 16;
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + kc * 128), "r"(pk[4 * kc]),
                       "r"(pk[4 * kc + 1]), "r"(pk[4 * kc + 2]), "r"(pk[4 * kc + 3])
                       : "memory");
        }
        if (hf == 0) fac[sb * kPairHeads + row] = f;
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          const uint32_t bar_r = map_to_cta(smem_u32(&p_full[sb]), peer);
          bulk_copy_to_cta(map_to_cta(pwarp, peer), pwarp, 2048, bar_r);
          if (hf == 0) {
            const uint32_t fa = smem_u32(&fac[sb * kPairHeads + 32 * q]);
            bulk_copy_to_cta(map_to_cta(fa, peer), fa, 128, bar_r);
          }
          if (poster) mbar_arrive_expect_tx(&p_full[sb], 4 * 2048 + 2 * 128);
          else mbar_arrive(&p_full[sb]);
        }
        if (__any_sync(0xffffffffu, f != 1.0f)) {
          // PV(t-1) must have retired before O is rescaled (f != 1 only for t > 0)
          ok = pair_wait(pv_done, (t - 1) & 1, abort_flag, partner_abort);
          if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
          tc_fence_after();
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_base + lane_addr + kPairTmemO + hf * 128 + cc * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
            tmem_st_32x32(tmem_base + lane_addr + kPairTmemO + hf * 128 + cc * 32, o);
          }
          tc_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_ready[sb]);
      }
    } else if (hf == 0) {
      // ---------------------------------------------------------------- sender: the partner runs the softmax of
      // these 32 heads.  Our partial scores of a tile go out as soon as its score MMA has retired: staged in
      // local shared memory in the layout of the receive buffer, moved by one 9 KB bulk copy that counts on
      // the partner's barrier.  Staging and receive buffer of parity t&1 are free once p_full(t-2) has
      // completed here: the partner sent those probabilities after reading what it had received.
      for (int t = 0; t < n_tiles && !aborted; ++t) {
        const int sb = t & 1;
        bool ok = pair_wait(&s_full[sb], (t >> 1) & 1, abort_flag, partner_abort);
        if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
        tc_fence_after();
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(tmem_base + lane_addr + kPairTmemS + sb * kMlaTile, v0);
        tmem_ld_32x32(tmem_base + lane_addr + kPairTmemS + sb * kMlaTile + 32, v1);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[sb]);
        if (t >= 2) {
          ok = pair_wait(&p_full[sb], ((t - 2) >> 1) & 1, abort_flag, partner_abort);
          if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
        }
        const uint32_t src = send_addr + sb * kPairRecvBytes + half_off;
        const uint32_t mine = src + lane * kPairRecvRow;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(mine + i * 16), "r"(v0[4 * i]), "r"(v0[4 * i + 1]),
                       "r"(v0[4 * i + 2]), "r"(v0[4 * i + 3])
                       : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(mine + kPairRecvBlock + i * 16), "r"(v1[4 * i]),
                       "r"(v1[4 * i + 1]), "r"(v1[4 * i + 2]), "r"(v1[4 * i + 3])
                       : "memory");
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0)
          bulk_copy_to_cta(map_to_cta(recv_addr + sb * kPairRecvBytes + half_off, peer), src, 2 * kPairRecvBlock,
                           map_to_cta(smem_u32(&recv_full[sb]), peer));
      }
    } else {
      // ---------------------------------------------------------------- rescaler: the partner's softmax says by
      // which factor (if any) the rows of these 32 heads shrink before the value MMA of the tile
      for (int t = 0; t < n_tiles && !aborted; ++t) {
        const int sb = t & 1;
        bool ok = pair_wait(&p_full[sb], (t >> 1) & 1, abort_flag, partner_abort);
        if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
        const float f = fac[sb * kPairHeads + row];
        if (__any_sync(0xffffffffu, f != 1.0f)) {
          ok = pair_wait(pv_done, (t - 1) & 1, abort_flag, partner_abort);
          if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
          tc_fence_after();
#pragma unroll 1
          for (int cc = 0; cc < 8; ++cc) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_base + lane_addr + kPairTmemO + cc * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
            tmem_st_32x32(tmem_base + lane_addr + kPairTmemO + cc * 32, o);
          }
          tc_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_ready[sb]);
      }
    }
    // ---- output: thread (row, hf) writes 128 of this CTA's 256 value dims of its head
    const bool write = row < p.n_heads;
    const int64_t ctx_off = (static_cast<int64_t>(item) * p.n_heads + row) * kMlaDv + c * 256 + hf * 128;
    float* ctx_row = static_cast<float*>(p.ctx) + ctx_off;
    __nv_bfloat16* ctx_row_h = static_cast<__nv_bfloat16*>(p.ctx) + ctx_off;
    if (n_tiles == 0) {
      if (write && !aborted) {
        if (p.ctx_bf16) {
          for (int j = 0; j < 128; j += 8) *reinterpret_cast<uint4*>(ctx_row_h + j) = make_uint4(0, 0, 0, 0);
        } else {
          for (int j = 0; j < 128; j += 4) *reinterpret_cast<float4*>(ctx_row + j) = make_float4(0, 0, 0, 0);
        }
        if (own && hf == 0) p.lse[static_cast<int64_t>(item) * p.n_heads + row] = -INFINITY;
      }
    } else if (!aborted) {
      // the row sums (one per column half) and the row maximum go to both CTAs
      if (own) {
        fin[hf * kPairHeads + row] = l;
        if (hf == 0) fin[2 * kPairHeads + row] = m_ref;
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          const uint32_t bar_r = map_to_cta(smem_u32(fin_bar), peer);
          const uint32_t la = smem_u32(&fin[hf * kPairHeads + 32 * q]);
          bulk_copy_to_cta(map_to_cta(la, peer), la, 128, bar_r);
          if (hf == 0) {
            const uint32_t ma = smem_u32(&fin[2 * kPairHeads + 32 * q]);
            bulk_copy_to_cta(map_to_cta(ma, peer), ma, 128, bar_r);
          }
          if (poster) mbar_arrive_expect_tx(fin_bar, 6 * 128);
          else mbar_arrive(fin_bar);
        }
      }
      bool ok = pair_wait(fin_bar, 0, abort_flag, partner_abort);
      ok = ok && pair_wait(pv_done, (n_tiles - 1) & 1, abort_flag, partner_abort);
      if (__all_sync(0xffffffffu, ok)) {
        tc_fence_after();
        const float l_o = fin[row] + fin[kPairHeads + row];
        const float m_o = fin[2 * kPairHeads + row];
        const float inv = (l_o > 0.f) ? 1.0f / l_o : 0.f;
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + lane_addr + kPairTmemO + hf * 128 + cc * 32, o);
          tc_wait_ld();
          if (write && p.ctx_bf16) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
              *reinterpret_cast<uint4*>(ctx_row_h + cc * 32 + j) = v;
            }
          } else if (write) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              *reinterpret_cast<float4*>(ctx_row + cc * 32 + j) =
                  make_float4(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv,
                              __uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
            }
          }
        }
        tc_fence_before();
        if (write && own && hf == 0)
          p.lse[static_cast<int64_t>(item) * p.n_heads + row] =
              (l_o > 0.f) ? (m_o + log2f(l_o)) * 0.6931471805599453f : -INFINITY;
      }
    }
  } else {
    // ------------------------------------------------------------------ MMA issuer (warp 12)
    // Issue order S(0), S(1), PV(0), S(2), PV(1), ...: the scores of the next tile keep the tensor pipe busy
    // while the exchange and the softmax of the current one run.
    constexpr uint32_t idesc_s = make_idesc(kFmtBF16, kFmtBF16, kPairHeads, kMlaTile);
    constexpr uint32_t idesc_pv = make_idesc(kFmtBF16, kFmtBF16, kPairHeads, 256, 0, 1);
    auto issue_scores = [&](int t) -> bool {
      const int s = t % kPairStages, sb = t & 1;
      const bool w = pair_wait(&kv_full[s], (t / kPairStages) & 1, abort_flag, partner_abort) &&
                     pair_wait(&s_empty[sb], ((t >> 1) & 1) ^ 1, abort_flag, partner_abort);
      if (!__all_sync(0xffffffffu, w)) return false;
      fence_proxy_async();  // gathered rows were written through the generic proxy
      tc_fence_after();
      if (elect_one()) {
        const uint32_t d = tmem_base + kPairTmemS + sb * kMlaTile;
        const uint64_t b0 = make_desc_k_sw128(kv_addr + s * kPairStageBytes);
#pragma unroll
        for (int j = 0; j < kPairVChunks; ++j) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            mma_f16_ts(d, tmem_base + kPairTmemQ + j * 32 + kk * 8, b0 + ((j * kMlaChunkBytesK + kk * 32) >> 4),
                       idesc_s, (j | kk) != 0);
          }
        }
        const uint64_t qa0 = make_desc_k_noswz(qr_addr, 128, 512);
        const uint64_t rb0 = make_desc_k_noswz(kv_addr + s * kPairStageBytes + kPairVChunks * kMlaChunkBytesK, 128, 512);
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          mma_f16_ss(d, qa0 + ((kk * 256) >> 4), rb0 + ((kk * 256) >> 4), idesc_s, 1);
        }
        tc_commit(&s_full[sb]);
      }
      __syncwarp();
      return true;
    };
    bool ok = pair_wait(q_full, 0, abort_flag, partner_abort);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_tiles > 0) ok = issue_scores(0);
    for (int t = 0; ok && t < n_tiles; ++t) {
      if (t + 1 < n_tiles && !issue_scores(t + 1)) break;
      const int s = t % kPairStages, sb = t & 1;
      const bool w = pair_wait(&p_full[sb], (t >> 1) & 1, abort_flag, partner_abort) &&
                     pair_wait(&o_ready[sb], (t >> 1) & 1, abort_flag, partner_abort);
      if (!__all_sync(0xffffffffu, w)) break;
      fence_proxy_async();
      tc_fence_after();
      if (elect_one()) {
        const uint64_t vb0 = make_desc_mn_sw128(kv_addr + s * kPairStageBytes, kMlaChunkBytesK, 1024);
#pragma unroll
        for (int j = 0; j < kMlaTile / 16; ++j) {  // 16 keys per MMA
          // P tile: [key half][16 groups of 8 heads][4 core matrices of 8 keys]
          const uint64_t pa = make_desc_k_noswz(p_addr + sb * kPairPBytes + (j >> 1) * 8192 + (j & 1) * 256, 128, 512);
          mma_f16_ss(tmem_base + kPairTmemO, pa, vb0 + ((j * 2048) >> 4), idesc_pv, (t | j) != 0);
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
  cluster_sync_all();   // the partner no longer writes into this CTA's shared memory
  tc_fence_after();
  if (warp == 12) tmem_dealloc(tmem_base, kMlaTmemCols);
  if (tid == 0 && s_abort) atomicMax(p.status, kDevWaitTimeout);
  mla_signal_peers(p);
}

int mla_pair_launch(const MlaParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(sparse_mla_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kPairSmemBytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = launch_chained(sparse_mla_pair_kernel, dim3(p.n_items * 2), dim3(kPairThreads), kPairSmemBytes, stream, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  return static_cast<int>(e);
}

}  // namespace b200dsa
