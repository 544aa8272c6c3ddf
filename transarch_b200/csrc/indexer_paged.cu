// Lightning-indexer token logits over a block table, one tcgen05 contraction per 128 keys.
//
//   logit[r, c] = out_scale * key_scale(c) * sum_h w[r,h] * relu( <q[r,h,:], key(c)> )
//
// Two key sources share the kernel:
//   FP8 paged cache (decode): pages of P tokens, P*128 e4m3 bytes followed by P fp32 scales;
//     row r walks its block-table row, column c is the logical key index.
//   bf16 flat keys addressed by a per-row list of 128-key blocks (HISA stage 2): column c is
//     (list slot, offset); its position is list[slot]*128 + offset, masked to [pos_lo, pos_hi).
//
// Orientation: the 128 keys of a tile are the UMMA M dimension (one TMEM lane per key), the
// 64 index heads are N, d=128 is K.  Per-head scores exist only in TMEM and registers: each
// epilogue thread owns one key and reduces the 64 heads locally.
//
// Roles (192 threads): warp 0 lane 0 issues TMA loads into an mbarrier ring, warp 1 lane 0
// issues the MMAs into a double-buffered TMEM accumulator, warps 2-5 run the epilogue.  The
// grid is persistent: the list of all (row, tile) pairs is split evenly over the CTAs, so
// ragged context lengths stay balanced.  Every wait is bounded; on a timeout the CTA raises
// the status word, drains its loads, frees TMEM and returns.
#include <stdio.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kTileKeys = 128;
constexpr int kHeads = 64;
constexpr int kDim = 128;
constexpr int kMaxRows = 1024;  // rows per launch (host loops beyond that)
constexpr int kThreads = 192;

// Fused selection (kEmit): the epilogue also appends every score at or above a per-segment floor to
// the row's candidate list in global memory, so that the top-k kernel never reads the logits.
//   segment  = the run of consecutive tiles of one row inside a CTA's share of the tile list
//   floor    = taken from the scores of the segment's first kSampleTiles tiles (buffered in shared
//              memory): the want-th largest sampled score, found with a 4096-bin histogram of the top 12
//              key bits and an exact rank inside the bin that holds it.  With m sampled keys of a row of n,
//              jk = k m / n of them are expected among the row's top k; want = jk + z sqrt(want), z = 5.5,
//              so that fewer than k of the row's scores reach the floor with probability about 1e-8 per
//              segment, while the list is expected to hold n want / m entries (5 200 of 8 388 608... per
//              row at n = 131072, 11 500 at n = 524288, under the 16384-entry capacity)
//   row_floor[row] = max of the floors of the row's segments: the list is complete above it
constexpr int kSampleTiles = 16;
constexpr int kSampleMax = kSampleTiles * kTileKeys;   // 2048 buffered scores
constexpr int kEmitHistWords = 2048;                   // 4096 bins, two 16-bit counters per word
constexpr int kWarpBuf = 128;                          // private candidate buffer of an epilogue warp
constexpr int kEmitCap = 16384;                        // entries per row of the global candidate lists
constexpr int kEmitEqMax = 256;                        // samples ranked exactly inside the threshold bin

template <bool kFp8, bool kEmit = false>
struct PagedCfg {
  static constexpr int kElem = kFp8 ? 1 : 2;
  static constexpr int kStageBytes = kTileKeys * kDim * kElem;  // 16 KB / 32 KB
  static constexpr int kQBytes = kHeads * kDim * kElem;         // 8 KB / 16 KB
  // bf16 keys (HISA stages, routed prefill) come out of L2 and the kernel is bound by its epilogue: two
  // stages leave room for a second CTA per SM, which doubles the epilogue warps per scheduler
  // What bounds the FP8 decode form, measured: the copy operations are back-pressured at issue (about 190
  // cycles each, 2 x 8 KB keys + 2 x 256 B scales per tile at page size 64), so the producer runs at the memory
  // rate and its ring is never the limit: a sixth stage, four accumulators, a 256-byte L2 promotion, a prefetched
  // table window, scales fetched by per-lane cp.async, or one lane per tile preparing its own copies each
  // left the time unchanged or made it worse.  A bare copy loop over the same pages needs the same 1450 cycles
  // per tile and CTA; it runs at 1965 MHz, this kernel under the power cap at 1640-1780 MHz.
  static constexpr int kStages = kFp8 ? (kEmit ? 4 : 5) : 2;
  static constexpr int kEmitBytes = kEmit ? (kSampleMax * 4 + kEmitHistWords * 4 + 4 * kWarpBuf * 8 + 64) : 0;
  static constexpr int kCtasPerSm = 2;
  static constexpr int kKSteps = kFp8 ? 4 : 8;                  // MMAs per tile (32 B of K each)
  // Per-tile key scales travel through their own ring.  A slot is reused kScaleSlots tiles
  // later; by then the MMA of tile (it + 2) has retired, which needed the epilogue of tile
  // `it` to release its accumulator, and the epilogue reads the scale before that release.
  static constexpr int kScaleSlots = kStages + 2;
  static constexpr int kScaleBytes = kFp8 ? kScaleSlots * kTileKeys * 4 : 0;
  static constexpr int kSmemBytes =
      kStages * kStageBytes + 2 * kQBytes + kScaleBytes + 1024 /*align*/ + 512 /*barriers*/ + kEmitBytes;
};

struct PagedIndexerParams {
  const uint8_t* cache;         // fp8 mode: base of the paged cache (for the scales)
  int64_t page_bytes;           // fp8 mode: P*(128+4)
  int32_t page_size;            // fp8 mode: P (32, 64 or 128); bf16 mode: 128
  int32_t num_pages;            // valid page / block ids are [0, num_pages)
  const float* weights;         // [n_rows, 64]
  const int32_t* row_cols;      // [n_rows] number of columns of each row
  const int32_t* table;         // block table / block list
  int64_t table_stride;
  int32_t table_cols;           // entries that may be read per table row
  int32_t table_row_div;        // table row of row r is r / table_row_div (next_n > 1 shares tables)
  const int32_t* row_table;     // nullable: explicit table row per row (overrides the division)
  const int32_t* pos_lo;        // bf16 mode, nullable: keep only pos_lo[r] <= position < pos_hi[r]
  const int32_t* pos_hi;
  int32_t n_rows;
  float out_scale;
  float* logits;                // [n_rows, logits_stride]
  int64_t logits_stride;
  int32_t logits_cols;          // columns that may be written per row
  const uint64_t* head_mask;    // nullable [n_rows]: bit h set = head h counts towards logits_gated
  float* logits_gated;          // nullable [n_rows, logits_stride]: the same sum over the masked heads only
  int32_t* status;
  // fp8 mode over per-row lists of 128-key logical blocks (HISA stage 2 on the paged cache): tile t of
  // row r scores keys [128 b, 128 b + 128) of the row's request, b = klist[r * klist_stride + t], found
  // through the block table; keys at or beyond pos_hi[r] (the context length) are masked
  const int32_t* klist;
  int64_t klist_stride;
  // fused selection (kEmit kernels only)
  uint64_t* cand;               // [n_rows, kEmitCap] composites (ordered score << 32 | ~position)
  int32_t* cand_count;          // [n_rows] entries appended (may exceed kEmitCap: list unusable)
  uint32_t* row_floor;          // [n_rows] largest floor any segment of the row used (ordered-float bits; 0 = none)
  const int32_t* row_pos_offset;  // nullable [n_rows]: added to the column to give the output position
  int32_t cand_target;          // k: how many of a row's scores the selection after this kernel wants
};

// kList (fp8 only): rows address the cache through per-row lists of logical 128-key blocks.  A template
// parameter, not a run-time test: the plain decode kernel is bound by HBM closely enough that two extra
// branches per tile in its producer and epilogue cost 4 % of its time.
// kGather (bf16 only): the "table" row of a query is a list of arbitrary key positions (MISA stage 2: the
// stage-1 candidates); a tile's 128 rows are gathered with 16-byte asynchronous copies into the swizzled
// layout, column c of the row is candidate c.
template <bool kFp8, bool kEmit = false, bool kList = false, bool kGather = false>
__global__ void __launch_bounds__(kThreads, PagedCfg<kFp8, kEmit>::kCtasPerSm)
indexer_paged_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_q,
                     const PagedIndexerParams p) {
  using Cfg = PagedCfg<kFp8, kEmit>;
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ uint8_t smem_dyn[];
  __shared__ int s_prefix[kMaxRows + 1];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
  uint8_t* stage_mem = smem_al;
  uint8_t* q_mem = smem_al + Cfg::kStages * Cfg::kStageBytes;
  float* sc_mem = reinterpret_cast<float*>(q_mem + 2 * Cfg::kQBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(q_mem + 2 * Cfg::kQBytes + Cfg::kScaleBytes);
  uint64_t* full = bars;                       // [kStages]
  uint64_t* empty = bars + Cfg::kStages;       // [kStages]
  uint64_t* q_full = empty + Cfg::kStages;     // [2]
  uint64_t* q_empty = q_full + 2;              // [2]
  uint64_t* acc_full = q_empty + 2;            // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2]
  uint64_t* sc_full = acc_empty + 2;           // [kScaleSlots]
  uint64_t* rv_bar = sc_full + Cfg::kScaleSlots;  // [1] rendezvous of the 128 epilogue threads (kEmit)
  uint8_t* emit_mem = reinterpret_cast<uint8_t*>(bars) + 512;
  float* s_samp = reinterpret_cast<float*>(emit_mem);                                  // [kSampleMax]
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(emit_mem + kSampleMax * 4);           // [kEmitHistWords]
  uint64_t* s_wbuf = reinterpret_cast<uint64_t*>(emit_mem + kSampleMax * 4 + kEmitHistWords * 4);  // [4][kWarpBuf]
  float* s_floor = reinterpret_cast<float*>(emit_mem + kSampleMax * 4 + kEmitHistWords * 4 + 4 * kWarpBuf * 8);
  int* s_wtot = reinterpret_cast<int*>(s_floor + 1);                                   // [4] warp totals
  int* s_eqn = s_wtot + 4;                                                             // [3] entries, bin, rank wanted
  float* s_eq = reinterpret_cast<float*>(s_hist);                                      // reuses the histogram

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // tiles per row -> exclusive prefix (rows <= kMaxRows)
  if (tid == 0) s_abort = 0;
  for (int r = tid; r < p.n_rows; r += kThreads) {
    int c = p.row_cols[r];
    c = max(0, min(c, p.logits_cols));
    s_prefix[r + 1] = (c + kTileKeys - 1) / kTileKeys;
  }
  if (tid == 0) s_prefix[0] = 0;
  __syncthreads();
  if (warp == 0) warp_prefix_inplace(s_prefix, p.n_rows);
  if (tid == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full[s], kGather ? 32 : 1);   // gather: the producer warp's 32 lanes, each after its copies
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 128);
    }
    for (int s = 0; s < Cfg::kScaleSlots; ++s) mbar_init(&sc_full[s], 1);
    mbar_init(rv_bar, 128);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&s_tmem_base, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = s_tmem_base;
  const int total_tiles = s_prefix[p.n_rows];
  const int g0 = static_cast<int>((static_cast<int64_t>(total_tiles) * blockIdx.x) / gridDim.x);
  const int g1 = static_cast<int>((static_cast<int64_t>(total_tiles) * (blockIdx.x + 1)) / gridDim.x);
  volatile int* abort_flag = &s_abort;

  // first row of this CTA's range
  int row0 = 0;
  if (g0 < g1) {
    int lo = 0, hi = p.n_rows;  // find row with prefix[row] <= g0 < prefix[row+1]
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= g0) lo = mid; else hi = mid;
    }
    row0 = lo;
  }

  int issued = 0;  // producer: loads issued (for the drain on abort)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the tile list with identical (uniform) values in every lane; the
    // lanes fetch 32 table entries at a time and one elected lane issues the copies.
    if (elect_one()) {
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_q);
    }
    int row = row0, prev_row = -1;
    int it = 0, qit = 0;
    int tbl_base = -1, tbl_entry = -1, tbl_len = 0, cols = 0, ident0 = 0;
    const int32_t* trow = p.table;
    const int P = kFp8 ? p.page_size : kTileKeys;
    const int p_shift = 31 - __clz(P);  // P is a power of two
    for (int g = g0; g < g1; ++g) {
      while (g >= s_prefix[row + 1]) ++row;
      const int t = g - s_prefix[row];
      if (row != prev_row) {
        const int qs = qit & 1;
        const bool okq = mbar_wait(&q_empty[qs], ((qit >> 1) & 1) ^ 1, abort_flag);
        if (!__all_sync(0xffffffffu, okq)) break;
        if (elect_one()) {
          mbar_arrive_expect_tx(&q_full[qs], Cfg::kQBytes);
          tma_load_2d(q_mem + qs * Cfg::kQBytes, &tmap_q, &q_full[qs], 0, row * kHeads);
          if constexpr (!kFp8)
            tma_load_2d(q_mem + qs * Cfg::kQBytes + Cfg::kQBytes / 2, &tmap_q, &q_full[qs], 64, row * kHeads);
        }
        ++qit;
        prev_row = row;
        cols = max(0, min(p.row_cols[row], p.logits_cols));
        if (p.table) {
          trow = p.table + static_cast<int64_t>(p.row_table ? p.row_table[row] : row / p.table_row_div) * p.table_stride;
        } else {
          ident0 = p.pos_lo[row] >> 7;    // no list: consecutive blocks from the one holding pos_lo
        }
        tbl_len = min(p.table_cols, (cols + P - 1) >> p_shift);
        tbl_base = -1;
      }
      const int s = it % Cfg::kStages;
      const bool oke = mbar_wait(&empty[s], ((it / Cfg::kStages) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, oke)) break;
      uint8_t* dst = stage_mem + s * Cfg::kStageBytes;
      const int key0 = t * kTileKeys;
      int nkeys = min(kTileKeys, cols - key0);
      int first = key0 >> p_shift;
      constexpr bool listed = kFp8 && kList;
      if constexpr (listed) {
        // the tile is logical block b of the request: its pages, as far as the context reaches
        const int b = p.klist[static_cast<int64_t>(row) * p.klist_stride + t];
        const int hi = p.pos_hi[row];
        nkeys = (b < 0) ? 0 : max(0, min(kTileKeys, hi - b * kTileKeys));
        first = (b < 0 ? 0 : b) * (kTileKeys >> p_shift);
        tbl_base = first;
        const int e = first + lane;
        tbl_entry = (lane < 4 && e < p.table_cols) ? trow[e] : -1;
      }
      const int npages = (nkeys + P - 1) >> p_shift;
      if (!listed && !kGather && (tbl_base < 0 || first < tbl_base || first + npages > tbl_base + 32)) {
        tbl_base = first;
        const int e = tbl_base + lane;
        tbl_entry = (e < tbl_len) ? (p.table ? trow[e] : ident0 + e) : -1;
      }
      if constexpr (kFp8) {
        int pg[4];  // statically indexed below so that it stays in registers
        int nvalid = 0;
        float* sc = sc_mem + (it % Cfg::kScaleSlots) * kTileKeys;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          pg[j] = -1;
          if (j < npages) {
            const int e = __shfl_sync(0xffffffffu, tbl_entry, (first + j - tbl_base) & 31);
            if (e >= 0 && e < p.num_pages) {
              pg[j] = e;
              ++nvalid;
            } else {
              for (int i = lane; i < P; i += 32) sc[j * P + i] = -1.0f;  // marks the keys as masked
            }
          }
        }
        __syncwarp();
        if (elect_one()) {
          uint64_t* scb = &sc_full[it % Cfg::kScaleSlots];
          mbar_arrive_expect_tx(scb, nvalid * P * 4);
          mbar_arrive_expect_tx(&full[s], nvalid * P * kDim);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (pg[j] < 0) continue;
            tma_load_3d(dst + j * P * kDim, &tmap_k, &full[s], 0, 0, pg[j]);
            bulk_load_1d(sc + j * P, p.cache + static_cast<int64_t>(pg[j]) * p.page_bytes + static_cast<int64_t>(P) * kDim,
                         P * 4, scb);
          }
          if (nvalid != npages) atomicMax(p.status, kDevBadIndex);
        }
      } else if constexpr (kGather) {
        // candidate positions of the tile: four per lane; a row is 16 copies of 16 bytes, two rows per instruction
        int idx4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = key0 + u * 32 + lane;
          const int v = (i < cols) ? __ldg(trow + i) : -1;
          idx4[u] = (v >= 0 && v < p.num_pages) ? v : -1;
        }
        const int c16 = lane & 15, half = lane >> 4;
        const uint32_t dst0 = smem_u32(dst) + (c16 >> 3) * (Cfg::kStageBytes / 2);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int h = 0; h < 16; ++h) {
            const int r = u * 32 + 2 * h + half;
            const int idx = __shfl_sync(0xffffffffu, idx4[u], 2 * h + half);
            const uint8_t* src = p.cache + static_cast<int64_t>(idx < 0 ? 0 : idx) * (kDim * 2) + c16 * 16;
            cp_async_16(dst0 + r * 128 + (((c16 & 7) ^ (r & 7)) << 4), src, idx >= 0);   // missing rows are zero-filled
          }
        }
        cp_async_mbar_arrive(&full[s]);
      } else {
        const int blk = __shfl_sync(0xffffffffu, tbl_entry, (first - tbl_base) & 31);
        if (elect_one()) {
          if (blk >= 0 && blk < p.num_pages) {
            mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
            tma_load_2d(dst, &tmap_k, &full[s], 0, blk * kTileKeys);
            tma_load_2d(dst + Cfg::kStageBytes / 2, &tmap_k, &full[s], 64, blk * kTileKeys);
          } else {
            mbar_arrive_expect_tx(&full[s], 0);
            atomicMax(p.status, kDevBadIndex);
          }
        }
      }
      ++it;
    }
    issued = it;
    if constexpr (kGather) cp_async_wait_all();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Whole warp in the loop; one elected lane issues the MMAs and their commits.
    constexpr uint32_t idesc = kFp8 ? make_idesc(kFmtE4M3, kFmtE4M3, 128, kHeads)
                                    : make_idesc(kFmtBF16, kFmtBF16, 128, kHeads);
    int row = row0, prev_row = -1;
    int it = 0, qit = 0, ait = 0, qs = 0;
    for (int g = g0; g < g1; ++g) {
      while (g >= s_prefix[row + 1]) ++row;
      if (row != prev_row) {
        qs = qit & 1;
        const bool okq = mbar_wait(&q_full[qs], (qit >> 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, okq)) break;
        ++qit;
        prev_row = row;
      }
      const bool last_of_row = (g + 1 == g1) || (g + 1 >= s_prefix[row + 1]);
      const int s = it % Cfg::kStages;
      const int as = ait & 1;
      const bool okf = mbar_wait(&full[s], (it / Cfg::kStages) & 1, abort_flag) &&
                       mbar_wait(&acc_empty[as], ((ait >> 1) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, okf)) break;
      if constexpr (kGather) fence_proxy_async();   // gathered rows were written through the generic proxy
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_addr = smem_base + s * Cfg::kStageBytes;
        const uint32_t b_addr = smem_base + Cfg::kStages * Cfg::kStageBytes + qs * Cfg::kQBytes;
        const uint32_t d_tmem = tmem_base + as * kHeads;
#pragma unroll
        for (int kk = 0; kk < Cfg::kKSteps; ++kk) {
          uint32_t a_off, b_off;
          if constexpr (kFp8) {
            a_off = kk * 32;
            b_off = kk * 32;
          } else {
            a_off = (kk >> 2) * (Cfg::kStageBytes / 2) + (kk & 3) * 32;
            b_off = (kk >> 2) * (Cfg::kQBytes / 2) + (kk & 3) * 32;
          }
          const uint64_t a_desc = make_desc_k_sw128(a_addr + a_off);
          const uint64_t b_desc = make_desc_k_sw128(b_addr + b_off);
          if constexpr (kFp8) mma_f8f6f4_ss(d_tmem, a_desc, b_desc, idesc, kk > 0);
          else mma_f16_ss(d_tmem, a_desc, b_desc, idesc, kk > 0);
        }
        tc_commit(&empty[s]);
        tc_commit(&acc_full[as]);
        if (last_of_row) tc_commit(&q_empty[qs]);  // q slot free once this row's MMAs retire
      }
      __syncwarp();
      ++it;
      ++ait;
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int lane_base = (warp & 3) * 32;  // TMEM lanes this warp may read
    float w[kHeads];
    int row = row0, prev_row = -1;
    int ait = 0;
    int cols = 0, lo = 0, hi = 0x7fffffff;
    uint32_t hm0 = 0, hm1 = 0;
    const bool dual = p.logits_gated != nullptr;
    const int32_t* trow = p.table;
    // fused selection state (identical in all 128 epilogue threads except wcnt, which is per warp)
    const int tix = lane_base + lane;                 // this thread's key inside a tile
    const bool emit = kEmit && p.cand != nullptr;
    uint64_t* wbuf = s_wbuf + (warp & 3) * kWarpBuf;
    int seg_g0 = 0, samp_tiles = 0, wcnt = 0, rv_phase = 0, posoff = 0;
    float floor_v = -3.402823466e38f;
    bool floor_ready = false, emit_abort = false;
    // append the warp's buffered candidates to the row's global list (one atomic per flush)
    auto flush_warp = [&](int r) {
      __syncwarp();
      if (wcnt > 0) {
        int base = 0;
        if (lane == 0) base = atomicAdd(p.cand_count + r, wcnt);
        base = __shfl_sync(0xffffffffu, base, 0);
        if (base + wcnt <= kEmitCap) {
          uint64_t* dst = p.cand + static_cast<int64_t>(r) * kEmitCap + base;
          for (int i = lane; i < wcnt; i += 32) dst[i] = wbuf[i];
        }
        wcnt = 0;
      }
      __syncwarp();
    };
    auto emit_one = [&](float v, int32_t pos, int r) {
      const bool take = v >= floor_v && v <= 3.402823466e38f;   // NaN, -inf and +inf never qualify
      const unsigned act = __ballot_sync(0xffffffffu, take);
      if (take)
        wbuf[wcnt + __popc(act & ((1u << lane) - 1))] =
            (static_cast<uint64_t>(float_to_ordered(v)) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(pos));
      wcnt += __popc(act);
      if (wcnt > kWarpBuf - 32) flush_warp(r);
    };
    // bounded rendezvous of the 128 epilogue threads (shared-memory writes before it are visible after it)
    auto rendezvous = [&]() {
      mbar_arrive(rv_bar);
      const bool ok = mbar_wait(rv_bar, rv_phase & 1, abort_flag);
      ++rv_phase;
      return __all_sync(0xffffffffu, ok);
    };
    for (int g = g0; g < g1; ++g) {
      while (g >= s_prefix[row + 1]) ++row;
      const int t = g - s_prefix[row];
      if (row != prev_row) {
        const float4* wr = reinterpret_cast<const float4*>(p.weights + static_cast<int64_t>(row) * kHeads);
#pragma unroll
        for (int j = 0; j < kHeads / 4; ++j) {
          float4 x = __ldg(wr + j);
          w[4 * j + 0] = x.x; w[4 * j + 1] = x.y; w[4 * j + 2] = x.z; w[4 * j + 3] = x.w;
        }
        cols = max(0, min(p.row_cols[row], p.logits_cols));
        if (p.table)
          trow = p.table + static_cast<int64_t>(p.row_table ? p.row_table[row] : row / p.table_row_div) * p.table_stride;
        if (p.pos_lo) lo = p.pos_lo[row];
        if (p.pos_hi) hi = p.pos_hi[row];
        if (dual) {
          const uint64_t hm = p.head_mask[row];
          hm0 = static_cast<uint32_t>(hm);
          hm1 = static_cast<uint32_t>(hm >> 32);
        }
        prev_row = row;
        if (emit) {   // a new segment: sample its first tiles before anything is appended
          seg_g0 = g;
          samp_tiles = min(kSampleTiles, min(g1, s_prefix[row + 1]) - g);
          floor_ready = false;
          posoff = p.row_pos_offset ? p.row_pos_offset[row] : 0;
        }
      }
      const int key = t * kTileKeys + lane_base + lane;  // column of this thread
      float kscale = 1.0f;
      bool keep = key < cols;
      if constexpr (kFp8) {
        const int slot = ait % Cfg::kScaleSlots;
        const bool sc_ready = mbar_wait(&sc_full[slot], (ait / Cfg::kScaleSlots) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, sc_ready)) break;
        kscale = sc_mem[slot * kTileKeys + lane_base + lane];
        keep = keep && (kscale >= 0.0f);
        if constexpr (kList) {
          const int b = p.klist[static_cast<int64_t>(row) * p.klist_stride + t];
          const int pos = b * kTileKeys + lane_base + lane;
          keep = keep && b >= 0 && pos >= lo && pos < hi;
        }
      } else if constexpr (kGather) {
        if (keep) {
          const int pos = __ldg(trow + key);
          keep = pos >= 0 && pos < p.num_pages && pos >= lo && pos < hi;
        }
      } else {
        if (keep) {
          const int blk = p.table ? trow[t] : (lo >> 7) + t;
          const int pos = blk * kTileKeys + lane_base + lane;
          keep = (blk >= 0 && blk < p.num_pages) && pos >= lo && pos < hi;
        }
      }
      const int as = ait & 1;
      const bool ready = mbar_wait(&acc_full[as], (ait >> 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) break;  // warp-uniform: tcgen05.ld needs the whole warp
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + as * kHeads;
      uint32_t v0[32], v1[32];
      tmem_ld_32x32(taddr, v0);
      tmem_ld_32x32(taddr + 32, v1);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
      float acc0 = 0.f, acc1 = 0.f;
      const int tile_cols = min(p.logits_cols, (t + 1) * kTileKeys);
      if (dual) {
        // one pass, two sums: all heads, and the routed heads only (a zero weight elsewhere); the same four
        // chains as the single-sum path, so that either sum equals a separate pass bit for bit
        float gat0 = 0.f, gat1 = 0.f, acc2 = 0.f, acc3 = 0.f, gat2 = 0.f, gat3 = 0.f;
        if constexpr (kFp8) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float r0 = fmaxf(__uint_as_float(v0[j]), 0.f), r1 = fmaxf(__uint_as_float(v1[j]), 0.f);
            acc0 = fmaf(r0, w[j], acc0);
            acc1 = fmaf(r1, w[32 + j], acc1);
            gat0 = fmaf(r0, ((hm0 >> j) & 1u) ? w[j] : 0.f, gat0);
            gat1 = fmaf(r1, ((hm1 >> j) & 1u) ? w[32 + j] : 0.f, gat1);
          }
        } else {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float r0 = fmaxf(__uint_as_float(v0[j]), 0.f), r1 = fmaxf(__uint_as_float(v1[j]), 0.f);
          const float r2 = fmaxf(__uint_as_float(v0[j + 1]), 0.f), r3 = fmaxf(__uint_as_float(v1[j + 1]), 0.f);
          acc0 = fmaf(r0, w[j], acc0);
          acc2 = fmaf(r2, w[j + 1], acc2);
          acc1 = fmaf(r1, w[32 + j], acc1);
          acc3 = fmaf(r3, w[33 + j], acc3);
          gat0 = fmaf(r0, ((hm0 >> j) & 1u) ? w[j] : 0.f, gat0);
          gat2 = fmaf(r2, ((hm0 >> (j + 1)) & 1u) ? w[j + 1] : 0.f, gat2);
          gat1 = fmaf(r1, ((hm1 >> j) & 1u) ? w[32 + j] : 0.f, gat1);
          gat3 = fmaf(r3, ((hm1 >> (j + 1)) & 1u) ? w[33 + j] : 0.f, gat3);
        }
        }
        acc0 += acc2;
        acc1 += acc3;
        gat0 += gat2;
        gat1 += gat3;
        if (key < tile_cols)
          p.logits_gated[static_cast<int64_t>(row) * p.logits_stride + key] =
              keep ? (gat0 + gat1) * kscale * p.out_scale : -INFINITY;
      } else if constexpr (kFp8) {
        // two chains of 32: the decode kernel is bound by HBM, and the shorter instruction stream is faster there
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          acc0 = fmaf(fmaxf(__uint_as_float(v0[j]), 0.f), w[j], acc0);
          acc1 = fmaf(fmaxf(__uint_as_float(v1[j]), 0.f), w[32 + j], acc1);
        }
      } else {
        float acc2 = 0.f, acc3 = 0.f;   // four independent chains of 16: the bf16 modes are bound by this loop
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          acc0 = fmaf(fmaxf(__uint_as_float(v0[j]), 0.f), w[j], acc0);
          acc2 = fmaf(fmaxf(__uint_as_float(v0[j + 1]), 0.f), w[j + 1], acc2);
          acc1 = fmaf(fmaxf(__uint_as_float(v1[j]), 0.f), w[32 + j], acc1);
          acc3 = fmaf(fmaxf(__uint_as_float(v1[j + 1]), 0.f), w[33 + j], acc3);
        }
        acc0 += acc2;
        acc1 += acc3;
      }
      const float out = keep ? (acc0 + acc1) * kscale * p.out_scale : -INFINITY;
      if (key < tile_cols && p.logits) p.logits[static_cast<int64_t>(row) * p.logits_stride + key] = out;
      if constexpr (kEmit) {
        if (emit) {
          const int seg_tile = g - seg_g0;
          if (!floor_ready) {
            s_samp[seg_tile * kTileKeys + tix] = out;
            if (seg_tile == samp_tiles - 1) {
              // ---- floor of this segment from its buffered head
              const int n_samp = samp_tiles * kTileKeys;
              const int key0 = (t - seg_tile) * kTileKeys;                      // first key of the segment
              const int m_valid = max(0, min(n_samp, cols - key0));
              // samples expected among the row's top k, and the sample rank that leaves a 5.5-sigma margin
              const float jk = static_cast<float>(p.cand_target) * static_cast<float>(m_valid) /
                               static_cast<float>(max(cols, 1));
              const int want = static_cast<int>(ceilf(jk + 15.125f + 5.5f * sqrtf(jk + 7.5625f)));
              floor_v = -3.402823466e38f;
              if (want < (m_valid * 9) / 10) {                                  // uniform over the 128 threads
                for (int i = tix; i < kEmitHistWords; i += 128) s_hist[i] = 0;
                if (!rendezvous()) { emit_abort = true; break; }              // histogram clear
                for (int i = 0; i < samp_tiles; ++i) {
                  const float v = s_samp[i * kTileKeys + tix];
                  if (v >= -3.402823466e38f && v <= 3.402823466e38f) {
                    const uint32_t bin = float_to_ordered(v) >> 20;
                    atomicAdd(&s_hist[bin >> 1], 1u << (16 * (bin & 1)));
                  }
                }
                if (!rendezvous()) { emit_abort = true; break; }
                // thread tix owns bins [32 tix, 32 tix + 32); higher threads hold higher bins
                int chunk = 0;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const uint32_t wv = s_hist[16 * tix + i];
                  chunk += static_cast<int>(wv & 0xffffu) + static_cast<int>(wv >> 16);
                }
                int suf = chunk;                       // inclusive suffix over the lanes of this warp
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                  const int u = __shfl_down_sync(0xffffffffu, suf, o);
                  if (lane + o < 32) suf += u;
                }
                if (lane == 0) s_wtot[warp & 3] = suf;
                if (tix == 0) {
                  *s_floor = -3.402823466e38f;         // fewer valid samples than wanted: everything is taken
                  s_eqn[0] = 0;
                  s_eqn[1] = -1;
                }
                if (!rendezvous()) { emit_abort = true; break; }
                int above = suf - chunk;               // samples in the bins above this thread's
                for (int wq = (warp & 3) + 1; wq < 4; ++wq) above += s_wtot[wq];
                if (above < want && above + chunk >= want) {
                  for (int b = 31; b >= 0; --b) {
                    const uint32_t wv = s_hist[16 * tix + (b >> 1)];
                    const int c = static_cast<int>((b & 1) ? (wv >> 16) : (wv & 0xffffu));
                    if (above + c >= want) {
                      *s_floor = fmaxf(ordered_to_float(static_cast<uint32_t>(32 * tix + b) << 20), -3.402823466e38f);
                      s_eqn[1] = 32 * tix + b;         // the bin that holds the want-th largest sample ...
                      s_eqn[2] = want - above;         // ... which is the s_eqn[2]-th largest inside it
                      break;
                    }
                    above += c;
                  }
                }
                if (!rendezvous()) { emit_abort = true; break; }              // histogram no longer read
                const int tbin = s_eqn[1];
                if (tbin >= 0) {
                  for (int i = 0; i < samp_tiles; ++i) {
                    const float v = s_samp[i * kTileKeys + tix];
                    if (v >= -3.402823466e38f && v <= 3.402823466e38f &&
                        static_cast<int>(float_to_ordered(v) >> 20) == tbin) {
                      const int slot = atomicAdd(&s_eqn[0], 1);
                      if (slot < kEmitEqMax) s_eq[slot] = v;
                    }
                  }
                }
                if (!rendezvous()) { emit_abort = true; break; }
                const int n_eq = s_eqn[0];
                if (tbin >= 0 && n_eq <= kEmitEqMax) {
                  // exact rank inside the bin (a crowded bin keeps its lower edge as the floor)
                  for (int i = tix; i < n_eq; i += 128) {
                    const float v = s_eq[i];
                    int rank = 0;
                    for (int j = 0; j < n_eq; ++j) {
                      const float u = s_eq[j];
                      rank += (u > v) || (u == v && j < i);
                    }
                    if (rank == s_eqn[2] - 1) *s_floor = v;
                  }
                }
                if (!rendezvous()) { emit_abort = true; break; }
                floor_v = *s_floor;
              }
              floor_ready = true;
              for (int i = 0; i < samp_tiles; ++i)                              // replay the buffered head
                emit_one(s_samp[i * kTileKeys + tix], (t - seg_tile + i) * kTileKeys + tix + posoff, row);
              if (!rendezvous()) { emit_abort = true; break; }                // buffer free for the next segment
            }
          } else {
            emit_one(out, key + posoff, row);
          }
          if ((g + 1 == g1) || (g + 1 >= s_prefix[row + 1])) {                 // end of the segment
            flush_warp(row);
            if (tix == 0) atomicMax(p.row_floor + row, float_to_ordered(floor_v));
          }
        }
      }
      ++ait;
    }
    if (emit_abort) *abort_flag = 1;
  }

  // ---------------------------------------------------------------------- common tail
  if (s_abort && warp == 0 && lane == 0) {
    // give loads already in flight a bounded chance to land before shared memory is released
    const int n = min(issued, Cfg::kStages);
    for (int j = 0; j < n; ++j) {
      const int it = issued - 1 - j;
      const int s = it % Cfg::kStages;
      const long long t0 = clock64();
      while (!mbar_test(&full[s], (it / Cfg::kStages) & 1)) {
        if (clock64() - t0 > (1ll << 22)) break;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 128);
  if (tid == 0 && s_abort) atomicMax(p.status, kDevWaitTimeout);
}

void set_last_error(const char* msg);

static int encode_map(CUtensorMap* m, CUtensorMapDataType dt, uint32_t rank, const void* base, const cuuint64_t* dims,
                      const cuuint64_t* strides, const cuuint32_t* box) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return B200DSA_ECUDA;
  cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(m, dt, rank, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled rejected the tensor layout");
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

static int sm_count() {
  static int n = 0;
  if (n) return n;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (n <= 0) n = 148;
  return n;
}

template <bool kFp8, bool kEmit = false, bool kList = false, bool kGather = false>
static int launch_paged(const CUtensorMap& mk, const CUtensorMap& mq, PagedIndexerParams p, int64_t est_tiles,
                        cudaStream_t stream) {
  using Cfg = PagedCfg<kFp8, kEmit>;
  cudaError_t e = cudaFuncSetAttribute(indexer_paged_kernel<kFp8, kEmit, kList, kGather>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  int grid = sm_count() * Cfg::kCtasPerSm;
  if (est_tiles > 0 && est_tiles < grid) grid = static_cast<int>(est_tiles);
  e = launch_chained(indexer_paged_kernel<kFp8, kEmit, kList, kGather>, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, mk,
                     mq, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

}  // namespace b200dsa

using namespace b200dsa;

namespace b200dsa {

struct ListArgs {            // per-row lists of 128-key logical blocks (fp8 paged mode)
  const int32_t* klist = nullptr;
  int64_t klist_stride = 0;
  const int32_t* list_cols = nullptr;   // [n_rows] 128 * (number of listed blocks)
};

struct EmitArgs {
  uint64_t* cand = nullptr;
  int32_t* cand_count = nullptr;
  uint32_t* row_floor = nullptr;
  const int32_t* row_pos_offset = nullptr;
  int32_t cand_target = 0;
};

// Validation, tensor maps and launches shared by the logits entry point and the fused selection.
int paged_fp8_launch(const char* who, const void* q_fp8, const float* weights, const void* cache, int32_t num_pages,
                     int32_t page_size, const int32_t* context_lens, const int32_t* block_table,
                     int64_t block_table_stride, const int32_t* row_table, int32_t n_rows, int32_t next_n,
                     int32_t max_cols, float out_scale, float* logits, int64_t logits_stride,
                     const uint64_t* head_mask, float* logits_gated, int32_t* status, const EmitArgs& em,
                     cudaStream_t stream, const ListArgs& ls = ListArgs{}) {
  char msg[160];
  if (!q_fp8 || !weights || !cache || !context_lens || !block_table || !status || n_rows < 0 || next_n < 1 ||
      num_pages < 1 || max_cols < 0 || (logits && logits_stride < max_cols) || (!logits && !em.cand) ||
      ((head_mask == nullptr) != (logits_gated == nullptr)) || (logits_gated && !logits)) {
    snprintf(msg, sizeof(msg), "%s: bad argument", who);
    set_last_error(msg);
    return B200DSA_EINVAL;
  }
  if (page_size != 32 && page_size != 64 && page_size != 128) {
    snprintf(msg, sizeof(msg), "%s: page_size must be 32, 64 or 128", who);
    set_last_error(msg);
    return B200DSA_EUNSUPPORTED;
  }
  if ((reinterpret_cast<uintptr_t>(q_fp8) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(weights) & 15)) {
    snprintf(msg, sizeof(msg), "%s: q, weights and cache must be 16-byte aligned", who);
    set_last_error(msg);
    return B200DSA_EALIGN;
  }
  const int64_t page_bytes = static_cast<int64_t>(page_size) * (kDim + 4);
  CUtensorMap mk, mq;
  {
    cuuint64_t dims[3] = {kDim, static_cast<cuuint64_t>(page_size), static_cast<cuuint64_t>(num_pages)};
    cuuint64_t strides[2] = {kDim, static_cast<cuuint64_t>(page_bytes)};
    cuuint32_t box[3] = {kDim, static_cast<cuuint32_t>(page_size), 1};
    int rc = encode_map(&mk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, cache, dims, strides, box);
    if (rc) return rc;
  }
  for (int r0 = 0; r0 < n_rows; r0 += kMaxRows) {
    const int nr = n_rows - r0 < kMaxRows ? n_rows - r0 : kMaxRows;
    // chunk boundaries must not split the next_n rows of one request
    if (!row_table && r0 % next_n != 0) {
      snprintf(msg, sizeof(msg), "%s: next_n must divide 1024 when n_rows > 1024", who);
      set_last_error(msg);
      return B200DSA_EUNSUPPORTED;
    }
    const uint8_t* qbase = static_cast<const uint8_t*>(q_fp8) + static_cast<int64_t>(r0) * kHeads * kDim;
    cuuint64_t dims[2] = {kDim, static_cast<cuuint64_t>(nr) * kHeads};
    cuuint64_t strides[1] = {kDim};
    cuuint32_t box[2] = {kDim, kHeads};
    int rc = encode_map(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, qbase, dims, strides, box);
    if (rc) return rc;
    PagedIndexerParams p{};
    p.cache = static_cast<const uint8_t*>(cache);
    p.page_bytes = page_bytes;
    p.page_size = page_size;
    p.num_pages = num_pages;
    p.weights = weights + static_cast<int64_t>(r0) * kHeads;
    p.row_cols = context_lens + r0;
    if (ls.klist) {
      p.row_cols = ls.list_cols + r0;
      p.klist = ls.klist + static_cast<int64_t>(r0) * ls.klist_stride;
      p.klist_stride = ls.klist_stride;
    }
    p.table = row_table ? block_table : block_table + static_cast<int64_t>(r0 / next_n) * block_table_stride;
    p.row_table = row_table ? row_table + r0 : nullptr;
    p.table_stride = block_table_stride;
    p.table_cols = static_cast<int32_t>(block_table_stride);
    p.table_row_div = next_n;
    p.pos_lo = nullptr;
    p.pos_hi = ls.klist ? context_lens + r0 : nullptr;
    p.n_rows = nr;
    p.out_scale = out_scale;
    p.logits = logits ? logits + static_cast<int64_t>(r0) * logits_stride : nullptr;
    p.logits_stride = logits_stride;
    p.logits_cols = max_cols;
    p.head_mask = head_mask ? head_mask + r0 : nullptr;
    p.logits_gated = logits_gated ? logits_gated + static_cast<int64_t>(r0) * logits_stride : nullptr;
    p.status = status;
    if (em.cand) {
      p.cand = em.cand + static_cast<int64_t>(r0) * kEmitCap;
      p.cand_count = em.cand_count + r0;
      p.row_floor = em.row_floor + r0;
      p.row_pos_offset = em.row_pos_offset ? em.row_pos_offset + r0 : nullptr;
      p.cand_target = em.cand_target;
      rc = launch_paged<true, true>(mk, mq, p, 0, stream);
    } else if (ls.klist) {
      rc = launch_paged<true, false, true>(mk, mq, p, 0, stream);
    } else {
      rc = launch_paged<true, false, false>(mk, mq, p, 0, stream);
    }
    if (rc) return rc;
  }
  return B200DSA_OK;
}

}  // namespace b200dsa

extern "C" int b200dsa_indexer_paged_fp8_logits(const void* q_fp8, const float* weights, const void* cache,
                                                int32_t num_pages, int32_t page_size, const int32_t* context_lens,
                                                const int32_t* block_table, int64_t block_table_stride,
                                                const int32_t* row_table, int32_t n_rows, int32_t next_n,
                                                int32_t max_cols, float out_scale,
                                                float* logits, int64_t logits_stride, const uint64_t* head_mask,
                                                float* logits_gated, int32_t* status, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!logits) {
    set_last_error("b200dsa_indexer_paged_fp8_logits: bad argument");
    return B200DSA_EINVAL;
  }
  return paged_fp8_launch("b200dsa_indexer_paged_fp8_logits", q_fp8, weights, cache, num_pages, page_size, context_lens,
                          block_table, block_table_stride, row_table, n_rows, next_n, max_cols, out_scale, logits,
                          logits_stride, head_mask, logits_gated, status, EmitArgs{}, static_cast<cudaStream_t>(stream));
}

namespace b200dsa {
int topk_select_from_lists(const float* scores, int64_t row_stride, int32_t n_rows, int32_t n_cols,
                           const int32_t* col_end, int32_t k, int32_t sorted, const int32_t* row_pos_offset,
                           uint64_t* cand, int32_t* count, uint32_t* floor_bits, int32_t* out_idx, float* out_val,
                           int64_t out_stride, int32_t* status, const PeerLinkDev* push, int64_t push_off,
                           cudaStream_t stream);
}

extern "C" int b200dsa_indexer_paged_blocklist_fp8_logits(const void* q_fp8, const float* weights, const void* cache,
                                                          int32_t num_pages, int32_t page_size,
                                                          const int32_t* context_lens, const int32_t* block_table,
                                                          int64_t block_table_stride, const int32_t* row_table,
                                                          int32_t n_rows, int32_t next_n, const int32_t* block_list,
                                                          int64_t block_list_stride, const int32_t* row_cols,
                                                          int32_t max_cols, float out_scale, float* logits,
                                                          int64_t logits_stride, int32_t* status, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!logits || !block_list || !row_cols || block_list_stride < 0 || (max_cols & 127) ||
      block_list_stride * 128 < max_cols) {
    set_last_error("b200dsa_indexer_paged_blocklist_fp8_logits: bad argument (max_cols a multiple of 128, at most "
                   "128 * block_list_stride)");
    return B200DSA_EINVAL;
  }
  ListArgs ls;
  ls.klist = block_list;
  ls.klist_stride = block_list_stride;
  ls.list_cols = row_cols;
  return paged_fp8_launch("b200dsa_indexer_paged_blocklist_fp8_logits", q_fp8, weights, cache, num_pages, page_size,
                          context_lens, block_table, block_table_stride, row_table, n_rows, next_n, max_cols, out_scale,
                          logits, logits_stride, nullptr, nullptr, status, EmitArgs{}, static_cast<cudaStream_t>(stream),
                          ls);
}

static int fused_topk(const char* who, const void* q_fp8, const float* weights, const void* cache, int32_t num_pages,
                      int32_t page_size, const int32_t* context_lens, const int32_t* block_table,
                      int64_t block_table_stride, const int32_t* row_table, int32_t n_rows, int32_t next_n,
                      int32_t max_cols, float out_scale, float* logits, int64_t logits_stride, int32_t k,
                      int32_t sorted, const int32_t* row_pos_offset, void* scratch_cand, int32_t* scratch_count,
                      int32_t* out_idx, float* out_val, int64_t out_stride, const PeerLinkDev* push, int64_t push_off,
                      int32_t* status, void* stream) {
  if (!scratch_cand || !scratch_count || !out_idx || k < 1 || k > 2048 || out_stride < k ||
      (reinterpret_cast<uintptr_t>(scratch_cand) & 7)) {
    char msg[200];
    snprintf(msg, sizeof(msg), "%s: bad argument (1 <= k <= 2048, out_stride >= k, 8-byte aligned scratch)", who);
    set_last_error(msg);
    return B200DSA_EINVAL;
  }
  EmitArgs em;
  em.cand = static_cast<uint64_t*>(scratch_cand);
  em.cand_count = scratch_count;
  em.row_floor = reinterpret_cast<uint32_t*>(scratch_count + n_rows);
  em.row_pos_offset = row_pos_offset;
  em.cand_target = k;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = paged_fp8_launch(who, q_fp8, weights, cache, num_pages, page_size, context_lens, block_table,
                            block_table_stride, row_table, n_rows, next_n, max_cols, out_scale, logits, logits_stride,
                            nullptr, nullptr, status, em, st);
  if (rc) return rc;
  return topk_select_from_lists(logits, logits_stride, n_rows, max_cols, context_lens, k, sorted, row_pos_offset,
                                em.cand, em.cand_count, em.row_floor, out_idx, out_val, out_stride, status, push,
                                push_off, st);
}

extern "C" int b200dsa_indexer_paged_fp8_topk(const void* q_fp8, const float* weights, const void* cache,
                                              int32_t num_pages, int32_t page_size, const int32_t* context_lens,
                                              const int32_t* block_table, int64_t block_table_stride,
                                              const int32_t* row_table, int32_t n_rows, int32_t next_n,
                                              int32_t max_cols, float out_scale, float* logits, int64_t logits_stride,
                                              int32_t k, int32_t sorted, const int32_t* row_pos_offset,
                                              void* scratch_cand, int32_t* scratch_count, int32_t* out_idx,
                                              float* out_val, int64_t out_stride, int32_t* status, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  return fused_topk("b200dsa_indexer_paged_fp8_topk", q_fp8, weights, cache, num_pages, page_size, context_lens,
                    block_table, block_table_stride, row_table, n_rows, next_n, max_cols, out_scale, logits,
                    logits_stride, k, sorted, row_pos_offset, scratch_cand, scratch_count, out_idx, out_val,
                    out_stride, nullptr, 0, status, stream);
}

extern "C" int b200dsa_indexer_paged_fp8_topk_push(const void* q_fp8, const float* weights, const void* cache,
                                                   int32_t num_pages, int32_t page_size, const int32_t* context_lens,
                                                   const int32_t* block_table, int64_t block_table_stride,
                                                   const int32_t* row_table, int32_t n_rows, int32_t next_n,
                                                   int32_t max_cols, float out_scale, float* logits,
                                                   int64_t logits_stride, int32_t k, int32_t sorted,
                                                   const int32_t* row_pos_offset, void* scratch_cand,
                                                   int32_t* scratch_count, int32_t* out_idx, float* out_val,
                                                   int64_t out_stride, const b200dsa_peer_link* link, int64_t off_recv,
                                                   int32_t* status, void* stream) {
  PeerLinkDev dev_link;
  if (!make_link(link, &dev_link, "b200dsa_indexer_paged_fp8_topk_push")) return B200DSA_EINVAL;
  if (off_recv < 0 || (off_recv & 15) || n_rows < 1) {
    set_last_error("b200dsa_indexer_paged_fp8_topk_push: off_recv must be 16-byte aligned and n_rows >= 1");
    return B200DSA_EINVAL;
  }
  return fused_topk("b200dsa_indexer_paged_fp8_topk_push", q_fp8, weights, cache, num_pages, page_size, context_lens,
                    block_table, block_table_stride, row_table, n_rows, next_n, max_cols, out_scale, logits,
                    logits_stride, k, sorted, row_pos_offset, scratch_cand, scratch_count, out_idx, out_val,
                    out_stride, &dev_link, off_recv, status, stream);
}

extern "C" int b200dsa_indexer_blocklist_bf16_logits(const void* q_bf16, const float* weights, const void* keys_bf16,
                                                     int32_t n_keys, const int32_t* block_list,
                                                     int64_t block_list_stride, const int32_t* row_cols,
                                                     const int32_t* pos_lo, const int32_t* pos_hi, int32_t n_rows,
                                                     int32_t max_cols, float out_scale, float* logits,
                                                     int64_t logits_stride, const uint64_t* head_mask,
                                                     float* logits_gated, int32_t* status, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!q_bf16 || !weights || !keys_bf16 || (!block_list && !pos_lo) || !row_cols || !logits || !status || n_rows < 0 ||
      n_keys < 1 || max_cols < 0 || logits_stride < max_cols || ((pos_lo == nullptr) != (pos_hi == nullptr)) ||
      ((head_mask == nullptr) != (logits_gated == nullptr))) {
    set_last_error("b200dsa_indexer_blocklist_bf16_logits: bad argument");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(q_bf16) & 15) || (reinterpret_cast<uintptr_t>(keys_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(weights) & 15)) {
    set_last_error("b200dsa_indexer_blocklist_bf16_logits: q, weights and keys must be 16-byte aligned");
    return B200DSA_EALIGN;
  }
  CUtensorMap mk, mq;
  {
    cuuint64_t dims[2] = {kDim, static_cast<cuuint64_t>(n_keys)};
    cuuint64_t strides[1] = {kDim * 2};
    cuuint32_t box[2] = {64, kTileKeys};
    int rc = encode_map(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, keys_bf16, dims, strides, box);
    if (rc) return rc;
  }
  const int n_blocks = (n_keys + kTileKeys - 1) / kTileKeys;
  for (int r0 = 0; r0 < n_rows; r0 += kMaxRows) {
    const int nr = n_rows - r0 < kMaxRows ? n_rows - r0 : kMaxRows;
    const uint8_t* qbase = static_cast<const uint8_t*>(q_bf16) + static_cast<int64_t>(r0) * kHeads * kDim * 2;
    cuuint64_t dims[2] = {kDim, static_cast<cuuint64_t>(nr) * kHeads};
    cuuint64_t strides[1] = {kDim * 2};
    cuuint32_t box[2] = {64, kHeads};
    int rc = encode_map(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, qbase, dims, strides, box);
    if (rc) return rc;
    PagedIndexerParams p{};
    p.cache = nullptr;
    p.page_bytes = 0;
    p.page_size = kTileKeys;
    p.num_pages = n_blocks;
    p.weights = weights + static_cast<int64_t>(r0) * kHeads;
    p.row_cols = row_cols + r0;
    p.table = block_list ? block_list + static_cast<int64_t>(r0) * block_list_stride : nullptr;
    p.table_stride = block_list_stride;
    p.table_cols = block_list ? static_cast<int32_t>(block_list_stride) : 0x7fffffff;
    p.table_row_div = 1;
    p.pos_lo = pos_lo ? pos_lo + r0 : nullptr;
    p.pos_hi = pos_hi ? pos_hi + r0 : nullptr;
    p.n_rows = nr;
    p.out_scale = out_scale;
    p.logits = logits + static_cast<int64_t>(r0) * logits_stride;
    p.logits_stride = logits_stride;
    p.logits_cols = max_cols;
    p.head_mask = head_mask ? head_mask + r0 : nullptr;
    p.logits_gated = logits_gated ? logits_gated + static_cast<int64_t>(r0) * logits_stride : nullptr;
    p.status = status;
    rc = launch_paged<false, false>(mk, mq, p, 0, static_cast<cudaStream_t>(stream));
    if (rc) return rc;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_indexer_gather_bf16_logits(const void* q_bf16, const float* weights, const void* keys_bf16,
                                                  int32_t n_keys, const int32_t* cand, int64_t cand_stride,
                                                  const int32_t* row_cols, const int32_t* pos_lo,
                                                  const int32_t* pos_hi, int32_t n_rows, int32_t max_cols,
                                                  float out_scale, float* logits, int64_t logits_stride,
                                                  int32_t* status, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!q_bf16 || !weights || !keys_bf16 || !cand || !row_cols || !logits || !status || n_rows < 0 || n_keys < 1 ||
      max_cols < 0 || logits_stride < max_cols || cand_stride < max_cols ||
      ((pos_lo == nullptr) != (pos_hi == nullptr))) {
    set_last_error("b200dsa_indexer_gather_bf16_logits: bad argument (cand_stride and logits_stride >= max_cols)");
    return B200DSA_EINVAL;
  }
  if ((reinterpret_cast<uintptr_t>(q_bf16) & 15) || (reinterpret_cast<uintptr_t>(keys_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(weights) & 15)) {
    set_last_error("b200dsa_indexer_gather_bf16_logits: q, weights and keys must be 16-byte aligned");
    return B200DSA_EALIGN;
  }
  CUtensorMap mk, mq;
  {
    cuuint64_t dims[2] = {kDim, static_cast<cuuint64_t>(n_keys)};
    cuuint64_t strides[1] = {kDim * 2};
    cuuint32_t box[2] = {64, kTileKeys};
    int rc = encode_map(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, keys_bf16, dims, strides, box);   // not loaded through
    if (rc) return rc;
  }
  for (int r0 = 0; r0 < n_rows; r0 += kMaxRows) {
    const int nr = n_rows - r0 < kMaxRows ? n_rows - r0 : kMaxRows;
    const uint8_t* qbase = static_cast<const uint8_t*>(q_bf16) + static_cast<int64_t>(r0) * kHeads * kDim * 2;
    cuuint64_t dims[2] = {kDim, static_cast<cuuint64_t>(nr) * kHeads};
    cuuint64_t strides[1] = {kDim * 2};
    cuuint32_t box[2] = {64, kHeads};
    int rc = encode_map(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, qbase, dims, strides, box);
    if (rc) return rc;
    PagedIndexerParams p{};
    p.cache = static_cast<const uint8_t*>(keys_bf16);   // gather source
    p.page_bytes = 0;
    p.page_size = kTileKeys;
    p.num_pages = n_keys;                               // valid positions are [0, n_keys)
    p.weights = weights + static_cast<int64_t>(r0) * kHeads;
    p.row_cols = row_cols + r0;
    p.table = cand + static_cast<int64_t>(r0) * cand_stride;
    p.table_stride = cand_stride;
    p.table_cols = static_cast<int32_t>(cand_stride < 0x7fffffff ? cand_stride : 0x7fffffff);
    p.table_row_div = 1;
    p.pos_lo = pos_lo ? pos_lo + r0 : nullptr;
    p.pos_hi = pos_hi ? pos_hi + r0 : nullptr;
    p.n_rows = nr;
    p.out_scale = out_scale;
    p.logits = logits + static_cast<int64_t>(r0) * logits_stride;
    p.logits_stride = logits_stride;
    p.logits_cols = max_cols;
    p.status = status;
    rc = launch_paged<false, false, false, true>(mk, mq, p, 0, static_cast<cudaStream_t>(stream));
    if (rc) return rc;
  }
  return B200DSA_OK;
}
