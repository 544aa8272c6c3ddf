// Row-wise top-k over fp32 scores, one CTA per row.
//
// Scores are mapped to order-preserving 32-bit keys and paired with the bit-inverted output
// position into a unique 64-bit composite, so "k largest composites" is a total order:
// descending score, ties towards the lowest position.
//
// topk_select_kernel (few rows; 256 to 1024 threads per row), by where the candidates of a row come from:
//   * a list collected by an earlier kernel (the indexer's epilogue, or topk_collect_kernel), a row of at most
//     sixteen columns per thread, or the merged candidates of the ranks: the candidates stay in REGISTERS; the
//     score keys are taken relative to the smallest one, an exact most-significant-digit radix select with 12-bit
//     digits runs over them with two alternating histograms until the threshold bin holds exactly the keys still
//     wanted, and the winners are placed by a scan of per-thread counts;
//   * a long row: contiguous chunks spread over the row are sampled into a 4096-bin histogram of the top 12 key
//     bits and a bin is chosen so that, with a 6-sigma margin, at least k row elements lie at or above it; one
//     streaming pass appends every element at or above that bin to a shared-memory candidate list; the same
//     radix select then runs on the list in shared memory;
//   * exact fallback (any distribution, massive ties, overflowing lists): the radix select (12/12/8-bit digits)
//     with the row in global memory as its source, re-reading it once per digit; the undecided bin, once small,
//     is sorted to pick the last few winners.
// topk_rows_kernel (many rows of at most 8192 columns): a 256-thread CTA per row, the row in shared memory as
// 32-bit keys, positions computed for tied keys and winners only.
// The k winners are optionally ordered (descending score, ascending position) by a counting sort into buckets that
// are linear in the score, with a bitonic sort as the fallback for rows whose scores crowd into one bucket.
#include <type_traits>

#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kHistBins = 4096;
constexpr int kCandCap = 8192;   // candidate list entries (64 KB)
constexpr int kEqCap = 1024;     // undecided-bin list (8 KB)
constexpr int kListCap = 16384;  // entries per row of the lists the indexer's epilogue collects (128 KB)
constexpr int kMaxSelectSmem = kHistBins * 4 + (kListCap + kEqCap + kCandCap) * 8;   // largest configuration
constexpr int kSampleChunk = 128;
constexpr int kSampleMax = 8192;

struct TopkParams {
  const float* scores;
  int64_t row_stride;
  int32_t n_rows, n_cols;
  const int32_t* col_begin;
  const int32_t* col_end;
  int32_t k;
  int32_t keep_pos_inf;
  const int32_t* pos_map;
  int64_t pos_map_stride;
  const int32_t* page_table;
  int64_t page_table_stride;
  int32_t page_size;
  const int32_t* row_pos_offset;
  int32_t* out_idx;
  float* out_val;
  int64_t out_stride;
  int32_t sorted;
  int32_t seg_cols;     // > 0: column c lives at (c / seg_cols) * seg_stride + c % seg_cols of its row
  int64_t seg_stride;
  // split mode: candidates pre-collected by topk_collect_kernel into global scratch
  uint64_t* pre_cand;   // [n_rows, kCandCap]
  int32_t* pre_count;   // [n_rows]; > kCandCap means "no usable list, select from the row itself"
  // segmented rows whose segments are separate buffers (peer GPUs): element offset of segment r
  // from `scores` / `pos_map` instead of r * seg_stride
  int32_t seg_off_n;
  int64_t seg_off[8];
  // lists collected by the indexer's own epilogue (fused selection): pre_floor[row] is the largest
  // score floor any part of the row was collected with (ordered-float bits), so the list holds EVERY
  // score of the row at or above it; the selection from the list is exact iff at least k entries
  // reach that floor.  `scores` may then be NULL (no fallback: *status gets kDevSelectIncomplete).
  uint32_t* pre_floor;
  int32_t* status;
  // key-sharded decode, first exchange folded into the two selections:
  //  push (local selection): row r's k positions and k score bit patterns are also stored as
  //    [2k] int32 at push_off + (push.rank * n_rows + r) * 2k * 4 of EVERY rank's exchange buffer;
  //    when the last CTA has fenced its stores it raises this rank's flag word on every rank
  //  wait (merge of the pushed lists): the kernel starts by waiting, bounded, until every rank's flag
  //    reached the step this rank's own push recorded in wait.state[0]
  //  owned: the winners inside [own_lo, own_hi) are also written, compacted and -1 padded, to `owned`
  int32_t push_on, wait_on;
  PeerLinkDev link;
  int64_t push_off;
  int32_t own_lo, own_hi;
  int32_t* owned;
  int64_t owned_stride;
  int32_t* owned_count;
};

__device__ __forceinline__ bool score_valid(float v, int keep_pos_inf) {
  // -inf, NaN never; +inf on request
  if (v != v) return false;
  if (v == -INFINITY) return false;
  if (v == INFINITY) return keep_pos_inf != 0;
  return true;
}

__device__ __forceinline__ int64_t col_offset(const TopkParams& p, int col) {
  if (p.seg_cols <= 0) return col;
  const int r = col / p.seg_cols;
  return (p.seg_off_n > 0 ? p.seg_off[r] : r * p.seg_stride) + (col - r * p.seg_cols);
}

__device__ __forceinline__ int32_t out_position(const TopkParams& p, int row, int col) {
  int32_t pos;
  if (p.pos_map) {
    pos = p.pos_map[row * p.pos_map_stride + col_offset(p, col)];
  } else if (p.page_table) {
    int pg = col / p.page_size;
    pos = p.page_table[row * p.page_table_stride + pg] * p.page_size + (col - pg * p.page_size);
  } else {
    pos = col;
  }
  if (p.row_pos_offset) pos += p.row_pos_offset[row];
  return pos;
}

__device__ __forceinline__ uint64_t make_composite(float v, int32_t pos) {
  return (static_cast<uint64_t>(float_to_ordered(v)) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(pos));
}

// histogram increment (shared-memory atomic without a return value)
__device__ __forceinline__ void hist_add(uint32_t* hist, uint32_t bin, bool active) {
  if (active) atomicAdd(&hist[bin], 1u);
}

// warp-aggregated append; entries beyond cap are counted but not stored
__device__ __forceinline__ void list_append(uint64_t* list, int* counter, int cap, uint64_t key, bool active) {
  unsigned act = __ballot_sync(0xffffffffu, active);
  if (act == 0) return;
  int lane = threadIdx.x & 31;
  int leader = __ffs(act) - 1;
  int base = 0;
  if (lane == leader) base = atomicAdd(counter, __popc(act));
  base = __shfl_sync(0xffffffffu, base, leader);
  if (active) {
    int slot = base + __popc(act & ((1u << lane) - 1));
    if (slot < cap) list[slot] = key;
  }
}

// Totals of the warps of a block (at most 32, in shared memory) -> sum of the totals of the warps before `warp`,
// and the sum of all of them.  One load and a shuffle scan per thread instead of a dependent chain of up to 32
// shared-memory loads.
template <class T>
__device__ __forceinline__ void warp_totals_scan(const T* totals, int nwarps, int warp, int& before, int& total) {
  const int lane = threadIdx.x & 31;
  const int mine = lane < nwarps ? static_cast<int>(totals[lane]) : 0;
  int incl = mine;
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  before = __shfl_sync(0xffffffffu, incl - mine, warp);
  total = __shfl_sync(0xffffffffu, incl, 31);
}

// Stream row elements [begin, begin+n) through f(value, column, in_range) with many loads in
// flight per thread.  Every thread calls f the same number of times (f may use warp votes).
// The 16-byte path needs src 16-byte aligned.
template <class F, class Off>
__device__ __forceinline__ void stream_row(const float* __restrict__ src, int begin, int n, bool vec_ok, Off&& off, F&& f) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  if (vec_ok) {
    const int a0 = begin & ~3;
    const int n4 = (begin + n - a0 + 3) >> 2;
    for (int base = 0; base < n4; base += nthr * 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i4 = base + u * nthr + tid;
        // off() maps a column to its element offset (segmented rows: four aligned columns never
        // straddle a segment, the caller checked that segment sizes and offsets are multiples of 4)
        v[u] = (i4 < n4) ? __ldg(reinterpret_cast<const float4*>(src + off(a0 + 4 * i4)))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = a0 + 4 * (base + u * nthr + tid);
        f(v[u].x, c + 0, c + 0 >= begin && c + 0 < begin + n);
        f(v[u].y, c + 1, c + 1 >= begin && c + 1 < begin + n);
        f(v[u].z, c + 2, c + 2 >= begin && c + 2 < begin + n);
        f(v[u].w, c + 3, c + 3 >= begin && c + 3 < begin + n);
      }
    }
  } else {
    for (int base = 0; base < n; base += nthr * 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * nthr + tid;
        v[u] = (i < n) ? __ldg(src + off(begin + i)) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * nthr + tid;
        f(v[u], begin + i, i < n);
      }
    }
  }
}

// In-place descending bitonic sort of n (power of two, >= 64) keys in shared memory.  Pair index t
// is handled by thread t % blockDim, so a warp works on contiguous 64-key chunks and keeps the same
// chunks in every stage: stages whose stride is at most 32 exchange keys inside a chunk only and need
// a warp barrier, not a block barrier (51 of the 66 stages of a 2048-key sort).
__device__ void bitonic_sort_desc(uint64_t* a, int n) {
  bool prev_wide = true;  // keys were written by other warps before the sort
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const bool wide = stride > 32;
      if (wide || prev_wide) __syncthreads(); else __syncwarp();
      prev_wide = wide;
      for (int t = threadIdx.x; t < (n >> 1); t += blockDim.x) {
        int lo = 2 * t - (t & (stride - 1));
        int hi = lo + stride;
        bool desc = ((lo & size) == 0);
        uint64_t x = a[lo], y = a[hi];
        if ((x < y) == desc) {
          a[lo] = y;
          a[hi] = x;
        }
      }
    }
  }
  __syncthreads();
}

// The same sort with the keys in registers: thread t holds keys [E*t, E*t + E).  Strides below E
// are compare-exchanges inside the thread, strides below 32*E go through warp shuffles, and only the
// widest strides pass through shared memory (10 of the 66 stages of a 2048-key sort with 512
// threads).  n must equal E * blockDim.x.
template <int E>
__device__ void bitonic_sort_desc_reg(uint64_t* a, int n) {
  const int base = threadIdx.x * E;
  uint64_t v[E];
  __syncthreads();
#pragma unroll
  for (int e = 0; e < E; ++e) v[e] = a[base + e];
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (stride >= 32 * E) {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < E; ++e) a[base + e] = v[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int idx = base + e;
          const uint64_t other = a[idx ^ stride];
          const bool want_max = ((idx & stride) != 0) != ((idx & size) == 0);
          v[e] = (want_max == (v[e] > other)) ? v[e] : other;
        }
      } else if (stride >= E) {
        const int lane_mask = stride / E;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int idx = base + e;
          const uint64_t other = __shfl_xor_sync(0xffffffffu, v[e], lane_mask);
          const bool want_max = ((idx & stride) != 0) != ((idx & size) == 0);
          v[e] = (want_max == (v[e] > other)) ? v[e] : other;
        }
      } else {
#pragma unroll
        for (int s = E >> 1; s > 0; s >>= 1) {
          if (stride == s) {
#pragma unroll
            for (int e = 0; e < E; ++e) {
              if ((e & s) == 0) {
                const bool desc = ((base + e) & size) == 0;
                const uint64_t x = v[e], y = v[e + s];
                if ((x < y) == desc) {
                  v[e] = y;
                  v[e + s] = x;
                }
              }
            }
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int e = 0; e < E; ++e) a[base + e] = v[e];
  __syncthreads();
}

// Sort dispatcher: registers when the key count is 2, 4 or 8 times the thread count.
__device__ void sort_desc(uint64_t* a, int n) {
  const int per = n / static_cast<int>(blockDim.x);
  if (per * static_cast<int>(blockDim.x) == n && per == 2) bitonic_sort_desc_reg<2>(a, n);
  else if (per * static_cast<int>(blockDim.x) == n && per == 4) bitonic_sort_desc_reg<4>(a, n);
  else if (per * static_cast<int>(blockDim.x) == n && per == 8) bitonic_sort_desc_reg<8>(a, n);
  else bitonic_sort_desc(a, n);
}

// Descending sort of the n winners in `a` by counting: 4096 buckets that are linear in the score between the
// smallest and the largest finite winner (monotone in the key, so buckets never interleave), an exclusive
// scan of the bucket sizes from the top, a scatter into `tmp`, and an exact rank inside each bucket by
// comparing the full 64-bit keys.  Five passes over the keys instead of the 66 compare-exchange stages of a
// 2048-key bitonic sort.  Returns false, with `a` untouched, when a bucket would hold more than kBucketMax keys
// (long runs of equal scores): the caller then sorts by compare-exchange.  All threads call it.
constexpr int kBucketMax = 48;
__device__ bool bucket_sort_desc(uint64_t* a, int n, uint64_t* tmp, uint32_t* hist, uint32_t* s_seg) {
  const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
  __shared__ uint32_t s_lo, s_hi, s_big;
  if (tid == 0) {
    s_lo = 0xffffffffu;
    s_hi = 0u;
    s_big = 0u;
  }
  for (int i = tid; i < kHistBins; i += nthr) hist[i] = 0;
  __syncthreads();
  // range of the finite scores (ordered bits compare like the floats)
  constexpr uint32_t kPosInf = 0xff800000u;   // float_to_ordered(+inf)
  uint32_t lo = 0xffffffffu, hi = 0u;
  for (int i = tid; i < n; i += nthr) {
    const uint32_t o = static_cast<uint32_t>(a[i] >> 32);
    lo = min(lo, o);
    if (o < kPosInf) hi = max(hi, o);
  }
  for (int o = 16; o > 0; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if (lane == 0) {
    atomicMin(&s_lo, lo);
    atomicMax(&s_hi, hi);
  }
  __syncthreads();
  const float vmin = ordered_to_float(s_lo);
  const float vmax = ordered_to_float(max(s_hi, s_lo));
  const float span = vmax - vmin;
  const float scale = (span > 0.f && span <= 3.0e38f) ? 4094.0f / span : 0.f;
  auto bucket = [&](uint64_t key) -> int {
    const uint32_t o = static_cast<uint32_t>(key >> 32);
    if (o >= kPosInf) return kHistBins - 1;
    const float x = (ordered_to_float(o) - vmin) * scale;      // monotone in the score
    return min(kHistBins - 2, max(0, static_cast<int>(x)));
  };
  for (int i = tid; i < n; i += nthr) atomicAdd(&hist[bucket(a[i])], 1u);
  __syncthreads();
  // exclusive scan from the top: thread t owns the kHistBins / nthr bins below bin (kHistBins - t * per)
  const int per = kHistBins / nthr;           // 4, 8 or 16
  uint32_t sum = 0, big = 0;
  const int top = kHistBins - 1 - tid * per;  // highest bin of this thread
  for (int j = 0; j < per; ++j) {
    const uint32_t c = hist[top - j];
    sum += c;
    big = max(big, c);
  }
  uint32_t incl = sum;
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  for (int o = 16; o > 0; o >>= 1) big = max(big, __shfl_xor_sync(0xffffffffu, big, o));
  if (lane == 31) s_seg[warp] = incl;
  if (lane == 0 && big > static_cast<uint32_t>(kBucketMax)) atomicMax(&s_big, big);
  __syncthreads();
  if (s_big != 0u) return false;   // uniform: every thread reads the same word
  int before_w, total_w;
  warp_totals_scan(s_seg, nwarps, warp, before_w, total_w);
  (void)total_w;
  uint32_t before = incl - sum + static_cast<uint32_t>(before_w);
  // hist[b] <- first output slot of bucket b
  for (int j = 0; j < per; ++j) {
    const uint32_t c = hist[top - j];
    hist[top - j] = before;
    before += c;
  }
  __syncthreads();
  for (int i = tid; i < n; i += nthr) {
    const uint64_t key = a[i];
    tmp[atomicAdd(&hist[bucket(key)], 1u)] = key;   // afterwards hist[b] = one past the last slot of bucket b
  }
  __syncthreads();
  for (int i = tid; i < n; i += nthr) {
    const uint64_t key = tmp[i];
    const int b = bucket(key);
    const int end = static_cast<int>(hist[b]);
    const int start = (b == kHistBins - 1) ? 0 : static_cast<int>(hist[b + 1]);
    int rank = 0;
    for (int j = start; j < end; ++j) rank += tmp[j] > key;
    a[start + rank] = key;
  }
  __syncthreads();
  (void)nwarps;
  return true;
}

// Find the highest bin d such that (#elements in bins >= d) >= need.  All threads call it
// (it contains block barriers).  Writes res[0]=d (or -1 when the whole histogram holds fewer
// than need), res[1]=count in bins above d, res[2]=hist[d].  Segment s (128 bins) covers bins
// [4096-128(s+1), 4096-128s): segment 0 is the highest.
__device__ void find_threshold_bin(const uint32_t* hist, int need, int* res, uint32_t* seg_sum) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int sgm = warp; sgm < 32; sgm += nwarps) {
    const uint4 v = reinterpret_cast<const uint4*>(hist + kHistBins - 128 * (sgm + 1))[lane];
    uint32_t t = v.x + v.y + v.z + v.w;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) seg_sum[sgm] = t;
  }
  __syncthreads();
  if (warp == 0) {
    const uint32_t mine = seg_sum[lane];
    uint32_t incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
    const bool owner = (incl - mine < static_cast<uint32_t>(need)) && (incl >= static_cast<uint32_t>(need));
    const unsigned who = __ballot_sync(0xffffffffu, owner);
    if (who == 0) {
      if (lane == 0) {
        res[0] = -1;
        res[1] = static_cast<int>(total);
        res[2] = 0;
      }
    } else {
      const int sgm = __ffs(who) - 1;
      const uint32_t above_seg = __shfl_sync(0xffffffffu, incl - mine, sgm);
      // lane l takes bins base+4l..base+4l+3; higher lanes hold higher bins
      const int base = kHistBins - 128 * (sgm + 1);
      const uint4 v = reinterpret_cast<const uint4*>(hist + base)[lane];
      const uint32_t t = v.x + v.y + v.z + v.w;
      uint32_t suf = t;  // inclusive suffix over lanes (lane 31 first)
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t u = __shfl_down_sync(0xffffffffu, suf, o);
        if (lane + o < 32) suf += u;
      }
      const uint32_t above_lane = above_seg + suf - t;  // elements in bins above this lane's four
      const bool own = (above_lane < static_cast<uint32_t>(need)) && (above_lane + t >= static_cast<uint32_t>(need));
      if (own) {
        uint32_t above = above_lane;
        const uint32_t h[4] = {v.w, v.z, v.y, v.x};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (above + h[j] >= static_cast<uint32_t>(need)) {
            res[0] = base + 4 * lane + 3 - j;
            res[1] = static_cast<int>(above);
            res[2] = static_cast<int>(h[j]);
            break;
          }
          above += h[j];
        }
      }
    }
  }
  __syncthreads();
}

// find_threshold_bin with one barrier: every warp repeats the search over the 32 segment sums and the
// owning segment itself, so the answer sits in registers of every thread and nothing goes through shared memory
// a second time.  d = -1 when the histogram holds fewer than `need`.
__device__ __forceinline__ void find_threshold_bin_bcast(const uint32_t* hist, int need, uint32_t* seg_sum, int& d,
                                                         int& above, int& in_bin) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int sgm = warp; sgm < 32; sgm += nwarps) {
    const uint4 v = reinterpret_cast<const uint4*>(hist + kHistBins - 128 * (sgm + 1))[lane];
    uint32_t t = v.x + v.y + v.z + v.w;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) seg_sum[sgm] = t;
  }
  __syncthreads();
  const uint32_t mine = seg_sum[lane];
  uint32_t incl = mine;
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  const bool owner = (incl - mine < static_cast<uint32_t>(need)) && (incl >= static_cast<uint32_t>(need));
  const unsigned who = __ballot_sync(0xffffffffu, owner);
  d = -1;
  above = 0;
  in_bin = 0;
  if (who == 0) return;
  const int sgm = __ffs(who) - 1;
  const uint32_t above_seg = __shfl_sync(0xffffffffu, incl - mine, sgm);
  const int base = kHistBins - 128 * (sgm + 1);
  const uint4 v = reinterpret_cast<const uint4*>(hist + base)[lane];   // lane l: bins base+4l .. base+4l+3
  const uint32_t t = v.x + v.y + v.z + v.w;
  uint32_t suf = t;  // inclusive suffix over lanes (lane 31 first)
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t u = __shfl_down_sync(0xffffffffu, suf, o);
    if (lane + o < 32) suf += u;
  }
  const uint32_t above_lane = above_seg + suf - t;
  const bool own = (above_lane < static_cast<uint32_t>(need)) && (above_lane + t >= static_cast<uint32_t>(need));
  int dd = 0, aa = 0, ib = 0;
  if (own) {
    uint32_t a = above_lane;
    const uint32_t h[4] = {v.w, v.z, v.y, v.x};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (a < static_cast<uint32_t>(need) && a + h[j] >= static_cast<uint32_t>(need)) {
        dd = base + 4 * lane + 3 - j;
        aa = static_cast<int>(a);
        ib = static_cast<int>(h[j]);
      }
      a += h[j];
    }
  }
  const int src = __ffs(__ballot_sync(0xffffffffu, own)) - 1;
  d = __shfl_sync(0xffffffffu, dd, src);
  above = __shfl_sync(0xffffffffu, aa, src);
  in_bin = __shfl_sync(0xffffffffu, ib, src);
}

// Sample the row into the 4096-bin histogram and choose the bin floor: with a 6-sigma margin at
// least k elements of the row lie at or above it.  Returns false when the fast path does not
// apply (margin too wide for the candidate list, or a sample with too few valid scores).  All
// threads of the CTA call it.  Rows up to kSampleMax are histogrammed completely (exact bin).
//
// Shared-memory atomics on the few bins around the mode of the scores serialise badly, and those
// bins are irrelevant for a top-k: a first pass over 1024 samples finds a bin well below the
// wanted quantile (4x the wanted tail mass), and the main pass only counts scores at or above it.
template <class Off>
__device__ bool sample_bin_floor(const TopkParams& p, const float* __restrict__ src, int begin, int n, int k,
                                 Off&& coff, uint32_t* hist, int* s_res, uint32_t* s_seg, uint32_t* bin_floor,
                                 int list_cap = kCandCap) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const bool exact = n <= kSampleMax;
  const int m = exact ? n : kSampleMax;
  const int n_chunks = kSampleMax / kSampleChunk;  // 128
  const int64_t step = exact ? kSampleChunk : n / n_chunks;
  const float ratio = static_cast<float>(n) / static_cast<float>(m);
  const float want_full = exact ? static_cast<float>(k) : k + 6.0f * sqrtf(2.0f * k * ratio) + 32.0f;
  if (want_full > 0.8f * list_cap) return false;
  const int want_sample = static_cast<int>(ceilf(want_full / ratio));

  // pass 1: 8 samples from the head of every chunk
  for (int i = tid; i < kHistBins; i += nthr) hist[i] = 0;
  __syncthreads();
  const int m1 = min(m, n_chunks * 8);
  for (int i = tid; i < ((m1 + 31) & ~31); i += nthr) {
    const int c = i >> 3;
    const int col = exact ? i : begin * 0 + static_cast<int>(c * step) + (i & 7);
    float v = 0.f;
    if (i < m1) v = __ldg(src + coff(begin + col));
    hist_add(hist, float_to_ordered(v) >> 20, (i < m1) && score_valid(v, p.keep_pos_inf));
  }
  __syncthreads();
  const int want1 = min(m1, 4 * static_cast<int>(ceilf(static_cast<float>(want_sample) * m1 / m)) + 8);
  find_threshold_bin(hist, want1, s_res, s_seg);
  const uint32_t bin_lo = s_res[0] < 0 ? 0u : static_cast<uint32_t>(s_res[0]);
  __syncthreads();

  // pass 2: the full sample, counting only scores at or above bin_lo
  for (int i = tid; i < kHistBins; i += nthr) hist[i] = 0;
  __syncthreads();
  for (int base = 0; base < m; base += nthr * 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * nthr + tid;
      const int c = i / kSampleChunk;
      v[u] = (i < m) ? __ldg(src + coff(begin + static_cast<int>(c * step) + (i - c * kSampleChunk))) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * nthr + tid;
      const uint32_t bin = float_to_ordered(v[u]) >> 20;
      hist_add(hist, bin, (i < m) && bin >= bin_lo && score_valid(v[u], p.keep_pos_inf));
    }
  }
  __syncthreads();
  find_threshold_bin(hist, want_sample, s_res, s_seg);
  const bool ok = s_res[0] >= 0;   // fewer counted samples than wanted: bin_lo was too high, or too few valid scores
  if (ok) *bin_floor = static_cast<uint32_t>(s_res[0]);
  __syncthreads();
  return ok;
}

struct SelectResult {
  bool take_all;     // fewer valid keys than wanted: every valid key wins
  uint64_t full;     // decided leading bits of the threshold composite
  int full_bits;
  int need_eq;       // winners still to be taken from the keys whose leading bits equal `full`
  bool eq_all_win;   // exactly need_eq keys have those leading bits: they all win, nothing is left to order
};

// Most-significant-digit radix select.  for_each(need_pos, f) must call f(key, active) the same
// number of times on every thread of a warp; keys are 64-bit composites (position bits may be
// zero while need_pos is false).
// to_the_end: keep refining until the threshold bin holds exactly the keys still wanted (cheap passes over keys
// in shared memory: two or three levels for distinct scores) instead of stopping at a bin of up to kEqCap keys
// that the caller then has to sort.
// In that mode the caller may pass the leading bits that all keys share (lead_bits of them, value `lead`): the
// first digit then starts right below them and spreads the keys over the whole histogram (candidates above a
// floor share sign, exponent and often more: the top 12 bits alone put them into a handful of bins, on which the
// shared-memory atomics serialise).
template <class ForEach>
__device__ SelectResult radix_select(ForEach&& for_each, int need, uint32_t* hist, int* s_res, uint32_t* s_seg,
                                     bool to_the_end = false, uint64_t lead = 0, int lead_bits = 0) {
  SelectResult r{false, 0, 0, 0, false};
  uint64_t prefix = lead;
  int prefix_bits = lead_bits;
  for (int level = 0; level < 6; ++level) {
    const int digit_bits = to_the_end ? min(12, 64 - prefix_bits) : ((level % 3 == 2) ? 8 : 12);
    const int shift = 64 - prefix_bits - digit_bits;
    const bool need_pos = (prefix_bits + digit_bits) > 32;
    for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for_each(need_pos, [&](uint64_t key, bool active) {
      const bool ok = active && (prefix_bits == 0 || (key >> (64 - prefix_bits)) == prefix);
      const uint32_t bin = static_cast<uint32_t>(key >> shift) & ((1u << digit_bits) - 1);
      hist_add(hist, bin, ok);
    });
    __syncthreads();
    find_threshold_bin(hist, need, s_res, s_seg);
    const int d = s_res[0];
    if (d < 0) {  // level 0 only
      r.take_all = true;
      return r;
    }
    const int above = s_res[1];
    const int in_bin = s_res[2];
    r.full = (prefix << digit_bits) | static_cast<uint64_t>(d);
    r.full_bits = prefix_bits + digit_bits;
    r.need_eq = need - above;
    r.eq_all_win = in_bin == r.need_eq;
    if (r.eq_all_win || level == 5 || r.full_bits == 64 || (!to_the_end && in_bin <= kEqCap)) return r;
    prefix = r.full;
    prefix_bits = r.full_bits;
    need = r.need_eq;
  }
  return r;
}

__global__ void __launch_bounds__(1024, 1) topk_select_kernel(const TopkParams p, int k_pow2, int cand_cap) {
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem_raw);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw + kHistBins * sizeof(uint32_t));
  uint64_t* eq = cand + cand_cap;   // cand_cap <= kCandCap: rows that fit entirely get a smaller list
  uint64_t* sel = eq + kEqCap;  // k_pow2 entries
  __shared__ int s_eq_cnt, s_sel_cnt, s_res[3], s_warp_cnt[32], s_overflow, s_own_cnt, s_last;
  __shared__ uint32_t s_kmin, s_kmax;   // range of the score keys of the candidates in shared memory
  __shared__ uint32_t s_seg[32];

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  int begin = p.col_begin ? p.col_begin[row] : 0;
  int end = p.col_end ? p.col_end[row] : p.n_cols;
  begin = max(begin, 0);
  end = min(end, p.n_cols);
  const int n = end - begin;
  const float* src = p.scores + row * p.row_stride;
  bool vec_ok = ((reinterpret_cast<uintptr_t>(p.scores) & 15) == 0) && ((p.row_stride & 3) == 0);
  if (p.seg_cols > 0) {
    vec_ok = vec_ok && ((p.seg_cols & 3) == 0) && ((p.seg_stride & 3) == 0);
    for (int r = 0; r < p.seg_off_n; ++r) vec_ok = vec_ok && ((p.seg_off[r] & 3) == 0);
  }
  auto coff = [&](int col) { return col_offset(p, col); };
  int32_t* out_idx = p.out_idx + row * p.out_stride;
  float* out_val = p.out_val ? p.out_val + row * p.out_stride : nullptr;
  const int k = p.k;

  if (tid == 0) {
    s_overflow = 0;
    s_eq_cnt = 0;
    s_sel_cnt = 0;
    s_own_cnt = 0;
    s_res[0] = 0;
    s_kmin = 0xffffffffu;
    s_kmax = 0u;
  }
  if (p.wait_on) {
    // the rows of this launch were pushed by the peers' selections: wait for every rank's flag
    const uint32_t step = static_cast<uint32_t>(*reinterpret_cast<volatile int32_t*>(p.link.state));
    if (tid < p.link.world && !wait_step(link_flag(p.link, p.link.rank, tid), step, p.link.wait_cycles))
      atomicMax(p.status, kDevWaitTimeout);
  }
  __syncthreads();

  // Writes the first n_out composites of `src_keys` (or nothing) as the row's result, -1 / -inf padded:
  // locally, into every peer's receive slot when pushing, and compacted into the owned list.
  auto write_row = [&](const uint64_t* src_keys, int n_out) {
    int32_t* own_row = p.owned ? p.owned + row * p.owned_stride : nullptr;
    const int64_t push_row = (static_cast<int64_t>(p.link.rank) * p.n_rows + row) * 2 * k;
    for (int j = tid; j < k; j += nthr) {
      int32_t pos = -1;
      float val = -INFINITY;
      if (j < n_out) {
        const uint64_t key = src_keys[j];
        pos = static_cast<int32_t>(~static_cast<uint32_t>(key & 0xffffffffu));
        val = ordered_to_float(static_cast<uint32_t>(key >> 32));
      }
      out_idx[j] = pos;
      if (out_val) out_val[j] = val;
      if (p.push_on) {
        for (int r = 0; r < p.link.world; ++r) {
          int32_t* dst = reinterpret_cast<int32_t*>(p.link.buf[r] + p.push_off) + push_row;
          dst[j] = pos;
          dst[k + j] = __float_as_int(val);
        }
      }
      if (own_row && pos >= p.own_lo && pos < p.own_hi) own_row[atomicAdd(&s_own_cnt, 1)] = pos;
    }
    if (own_row) {
      __syncthreads();
      const int n_own = s_own_cnt;
      for (int j = n_own + tid; j < k; j += nthr) own_row[j] = -1;
      if (tid == 0) p.owned_count[row] = n_own;
    }
    if (p.push_on) {
      // every CTA of the grid takes a ticket after fencing its peer stores; the last one raises the flags
      __syncthreads();
      if (tid == 0) {
        __threadfence_system();
        s_last = (atomicAdd(p.link.state + 1, 1) == static_cast<int>(gridDim.x) - 1);
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
        const uint32_t step = static_cast<uint32_t>(*reinterpret_cast<volatile int32_t*>(p.link.state)) + 1u;
        if (tid < p.link.world) st_release_sys(link_flag(p.link, tid, p.link.rank), step);
        if (tid == 0) {
          p.link.state[1] = 0;
          p.link.state[0] = static_cast<int32_t>(step);
        }
      }
    }
  };

  if (n <= 0) {
    write_row(nullptr, 0);
    return;
  }

  // ---- selection from at most eight candidates per thread held in registers (composites; bit j of `pres` says
  // that t[j] holds one; n_present of them in the block; s_kmin / s_kmax hold the range of their score keys and
  // both histograms are clear).  The score keys are taken relative to the smallest one, so that the first digit
  // starts at the highest bit in which the candidates differ and spreads them over the whole histogram (above a
  // floor they share sign, exponent and more: the top key bits alone would put them into a handful of bins, on
  // which the shared-memory atomics serialise); two histograms alternate, so a level costs two barriers; the
  // winners are placed by a scan of per-thread counts.  Writes the row's result.
  constexpr int kFastPer = 8;
  const int warp_id = tid >> 5, lane_id = tid & 31, n_warps = nthr >> 5;
  uint32_t* hist2 = reinterpret_cast<uint32_t*>(cand);   // the candidate area is not used on these paths
  auto pres_of_count = [&](int c) {
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < kFastPer; ++j) m |= (tid + j * nthr < c) ? (1u << j) : 0u;
    return m;
  };
  auto select_from_registers = [&](auto& t, uint32_t pres, int n_present) {
    constexpr int kPer = static_cast<int>(sizeof(t) / sizeof(t[0]));
    const uint32_t kmin = s_kmin, kmax = s_kmax;
    const int score_bits = kmax > kmin ? 32 - __clz(kmax - kmin) : 0;
    const int width = score_bits + 32;
    const uint64_t sub = static_cast<uint64_t>(kmin) << 32;
#pragma unroll
    for (int j = 0; j < kPer; ++j) t[j] -= sub;   // absent entries are never looked at
    uint64_t prefix = 0;
    int pbits = 0, need = k;
    const int max_levels = n_present > k ? 6 : 0;   // no more candidates than wanted: all of them win
    uint32_t* cur = hist;
    uint32_t* other = hist2;
#pragma unroll 1
    for (int level = 0; level < max_levels; ++level) {
      const int dbits = min(12, width - pbits);
      const int shift = width - pbits - dbits;
      const uint32_t mask = (1u << dbits) - 1u;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        if (((pres >> j) & 1u) && (pbits == 0 || (t[j] >> (width - pbits)) == prefix))
          atomicAdd(&cur[static_cast<uint32_t>(t[j] >> shift) & mask], 1u);
      }
      __syncthreads();
      if (level > 0) {   // the histogram of the previous level has been read by every warp: clear it for the next
        for (int i = tid; i < kHistBins; i += nthr) other[i] = 0;
      }
      int d, above, in_bin;
      find_threshold_bin_bcast(cur, need, s_seg, d, above, in_bin);
      if (d < 0) break;      // cannot happen: more candidates than wanted share the prefix
      prefix = (prefix << dbits) | static_cast<uint64_t>(d);
      pbits += dbits;
      need -= above;
      if (in_bin == need || pbits == width) break;
      uint32_t* sw = cur;
      cur = other;
      other = sw;
    }
    // winners: everything at or above the decided prefix
    auto wins = [&](uint64_t x) { return pbits == 0 || (x >> (width - pbits)) >= prefix; };
    int mine = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) mine += (((pres >> j) & 1u) && wins(t[j])) ? 1 : 0;
    int incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane_id >= o) incl += v;
    }
    if (lane_id == 31) s_warp_cnt[warp_id] = incl;
    __syncthreads();
    int before, total;
    warp_totals_scan(s_warp_cnt, n_warps, warp_id, before, total);
    before += incl - mine;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      if (((pres >> j) & 1u) && wins(t[j])) {
        if (before < k_pow2) sel[before] = t[j] + sub;
        ++before;
      }
    }
    __syncthreads();
    const int n_fast = min(total, k);
    if (p.sorted && (n_fast <= 64 || !bucket_sort_desc(sel, n_fast, cand, hist, s_seg))) {
      int n_pow2 = 32;
      while (n_pow2 < n_fast) n_pow2 <<= 1;
      for (int i = n_fast + tid; i < n_pow2; i += nthr) sel[i] = 0;
      sort_desc(sel, n_pow2);
    }
    write_row(sel, n_fast);
  };

  // ------------------------------------------------------------------ candidate collection
  const int seg_cap = cand_cap / n_warps;
  uint64_t* my_seg = cand + warp_id * seg_cap;
  bool from_smem = false;
  int cnt = 0;  // total candidates
  bool have_pre = false;
  if (p.pre_cand) {
    // split / fused mode: the candidates of this row were collected by an earlier kernel
    // the first eight entries per thread of the row's list are fetched before its length is known (the slots
    // exist whatever the length; what lies beyond it is dropped below): one memory round trip instead of two
    uint64_t t[kFastPer];
    {
      const uint64_t* g = p.pre_cand + static_cast<int64_t>(row) * cand_cap;
#pragma unroll
      for (int j = 0; j < kFastPer; ++j) t[j] = (tid + j * nthr < cand_cap) ? g[tid + j * nthr] : 0ull;
    }
    const int c = p.pre_count[row];
    const uint32_t fl = p.pre_floor ? p.pre_floor[row] : 0u;
    // ---- fast path: a list of at most eight candidates per thread stays in registers.  The score keys are
    // taken relative to the smallest one, so that the first digit starts at the highest bit in which the
    // candidates differ and spreads them over the whole histogram (above a floor they share sign, exponent
    // and more, and the top key bits alone would put them into a handful of bins); two histograms alternate,
    // so a level costs two barriers; winners are placed by a scan of per-thread counts.
    if (c > k && c <= kFastPer * nthr && c <= cand_cap) {
      for (int i = tid; i < kHistBins; i += nthr) {
        hist[i] = 0;
        hist2[i] = 0;
      }
#pragma unroll
      for (int j = 0; j < kFastPer; ++j) {
        if (tid + j * nthr >= c) t[j] = 0ull;
      }
      int n_ge = 0;
      uint32_t lo = 0xffffffffu, hi = 0u;
#pragma unroll
      for (int j = 0; j < kFastPer; ++j) {
        if (tid + j * nthr < c) {
          const uint32_t sk = static_cast<uint32_t>(t[j] >> 32);
          n_ge += sk >= fl;
          lo = min(lo, sk);
          hi = max(hi, sk);
        }
      }
      for (int o = 16; o > 0; o >>= 1) {
        n_ge += __shfl_xor_sync(0xffffffffu, n_ge, o);
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
      }
      if (lane_id == 0 && lo <= hi) {
        atomicAdd(&s_res[0], n_ge);
        atomicMin(&s_kmin, lo);
        atomicMax(&s_kmax, hi);
      }
      __syncthreads();
      const bool fast_ok = !p.pre_floor || s_res[0] >= k || fl == 0x00800000u;
      if (fast_ok) {
        if (tid == 0) {          // re-arm for the next call (every thread has read the count by now)
          p.pre_count[row] = 0;
          if (p.pre_floor) p.pre_floor[row] = 0u;
        }
        select_from_registers(t, c <= 0 ? 0u : pres_of_count(c), c);
        return;
      }
    }
    __syncthreads();
    if (tid == 0) {          // re-arm for the next call
      p.pre_count[row] = 0;
      if (p.pre_floor) p.pre_floor[row] = 0u;
    }
    // lists are cand_cap entries apart (8192 in the split form, 16384 when the indexer collected them)
    bool usable = c <= cand_cap && (p.pre_floor || c >= k);
    if (usable) {
      const uint64_t* g = p.pre_cand + static_cast<int64_t>(row) * cand_cap;
      int n_ge = 0;
      uint32_t lo = 0xffffffffu, hi = 0u;
      for (int i = tid; i < c; i += nthr) {
        const uint64_t e = g[i];
        cand[i] = e;
        const uint32_t sk = static_cast<uint32_t>(e >> 32);
        n_ge += sk >= fl;
        lo = min(lo, sk);
        hi = max(hi, sk);
      }
      for (int o = 16; o > 0; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
      }
      if (lane_id == 0 && lo <= hi) {
        atomicMin(&s_kmin, lo);
        atomicMax(&s_kmax, hi);
      }
      if (p.pre_floor) {
        // the list is complete at and above the floor; a floor of -FLT_MAX means the whole row is in it
        if (tid == 0) s_res[0] = 0;
        __syncthreads();
        if (n_ge) atomicAdd(&s_res[0], n_ge);
        __syncthreads();
        usable = (s_res[0] >= k) || (fl == 0x00800000u);
        __syncthreads();
      }
    }
    if (!usable && p.pre_floor && p.scores == nullptr) {
      // no logits to fall back to: report, and return the best of what the list holds
      if (tid == 0 && p.status) atomicMax(p.status, kDevSelectIncomplete);
      usable = c <= cand_cap;
      if (!usable) {
        write_row(nullptr, 0);
        return;
      }
    }
    if (usable) {
      if (tid < n_warps) s_warp_cnt[tid] = max(0, min(seg_cap, c - tid * seg_cap));
      __syncthreads();
      have_pre = true;
      from_smem = true;
      cnt = c;
    }
  }
  // short rows, and the merge of the ranks' candidates: straight from global memory into registers, eight
  // columns per thread (sixteen for the 16384 candidates of an eight-rank merge)
  auto direct_from_global = [&](auto per_tag) {
    constexpr int kPer = decltype(per_tag)::value;
    // short rows, and the merge of the ranks' candidates: straight from global memory into registers
    for (int i = tid; i < kHistBins; i += nthr) {
      hist[i] = 0;
      hist2[i] = 0;
    }
    float v[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = tid + j * nthr;
      v[j] = i < n ? __ldg(src + coff(begin + i)) : 0.f;
    }
    uint64_t t[kPer];
    uint32_t pres = 0, lo = 0xffffffffu, hi = 0u;
    int n_pres = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = tid + j * nthr;
      t[j] = 0ull;
      if (i < n && score_valid(v[j], p.keep_pos_inf)) {
        t[j] = make_composite(v[j], out_position(p, row, begin + i));
        pres |= 1u << j;
        const uint32_t sk = static_cast<uint32_t>(t[j] >> 32);
        lo = min(lo, sk);
        hi = max(hi, sk);
        ++n_pres;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      n_pres += __shfl_xor_sync(0xffffffffu, n_pres, o);
      lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (lane_id == 0 && lo <= hi) {
      atomicAdd(&s_res[0], n_pres);
      atomicMin(&s_kmin, lo);
      atomicMax(&s_kmax, hi);
    }
    __syncthreads();
    select_from_registers(t, pres, s_res[0]);
  };
  if (!p.pre_cand && cand_cap >= 2048) {
    if (n <= kFastPer * nthr) {
      direct_from_global(std::integral_constant<int, kFastPer>{});
      return;
    }
    if (n <= 2 * kFastPer * nthr) {
      direct_from_global(std::integral_constant<int, 2 * kFastPer>{});
      return;
    }
  }
  uint32_t bin_floor = 0;
  bool try_fast = !have_pre;
  if (try_fast && n > cand_cap)
    try_fast = sample_bin_floor(p, src, begin, n, k, coff, hist, s_res, s_seg, &bin_floor, cand_cap);

  // Each warp compacts its takes into its own segment of the candidate list with votes
  // only (no atomics); a full segment raises the overflow flag and the row falls back.
  if (try_fast) {
    int wcnt = 0;  // warp-uniform
    uint32_t lo = 0xffffffffu, hi = 0u;
    stream_row(src, begin, n, vec_ok, coff, [&](float v, int col, bool in_range) {
      const uint32_t sk = float_to_ordered(v);
      const bool take = in_range && score_valid(v, p.keep_pos_inf) && (sk >> 20) >= bin_floor;
      const unsigned act = __ballot_sync(0xffffffffu, take);
      if (take) {
        const int slot = wcnt + __popc(act & ((1u << lane_id) - 1));
        if (slot < seg_cap) my_seg[slot] = make_composite(v, out_position(p, row, col));
        lo = min(lo, sk);
        hi = max(hi, sk);
      }
      wcnt += __popc(act);
    });
    for (int o = 16; o > 0; o >>= 1) {
      lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (lane_id == 0) {
      s_warp_cnt[warp_id] = min(wcnt, seg_cap);
      if (wcnt > seg_cap) s_overflow = 1;
      if (lo <= hi) {
        atomicMin(&s_kmin, lo);
        atomicMax(&s_kmax, hi);
      }
    }
    __syncthreads();
    {
      int before_unused, total;
      warp_totals_scan(s_warp_cnt, n_warps, warp_id, before_unused, total);
      cnt += total;
    }
    from_smem = (s_overflow == 0) && (cnt >= k || n <= cand_cap);
  }

  // ------------------------------------------------------------------ exact selection
  auto each_cand = [&](bool /*need_pos*/, auto&& f) {
    if (have_pre) {  // contiguous list
      for (int base = 0; base < cnt; base += nthr) {
        const int i = base + tid;
        const bool active = i < cnt;
        f(active ? cand[i] : 0ull, active);
      }
      return;
    }
    for (int base = 0; base < cand_cap; base += nthr) {
      const int i = base + tid;
      const int w = i / seg_cap;
      const bool active = (i - w * seg_cap) < s_warp_cnt[w];
      f(active ? cand[i] : 0ull, active);
    }
  };
  auto each_row = [&](bool need_pos, auto&& f) {
    stream_row(src, begin, n, vec_ok, coff, [&](float v, int col, bool in_range) {
      const bool active = in_range && score_valid(v, p.keep_pos_inf);
      uint64_t key = 0;
      if (active)
        key = need_pos ? make_composite(v, out_position(p, row, col))
                       : (static_cast<uint64_t>(float_to_ordered(v)) << 32);
      f(key, active);
    });
  };
  auto emit = [&](const SelectResult& r) {
    return [&, r](uint64_t key, bool active) {
      bool direct = false, tie = false;
      if (active) {
        if (r.take_all) {
          direct = true;
        } else {
          const uint64_t top = key >> (64 - r.full_bits);
          direct = top > r.full || (r.eq_all_win && top == r.full);
          tie = !r.eq_all_win && top == r.full;
        }
      }
      list_append(sel, &s_sel_cnt, k_pow2, key, direct);
      list_append(eq, &s_eq_cnt, kEqCap, key, tie);
    };
  };

  SelectResult r;
  if (from_smem) {
    if (cnt <= k) {
      r = SelectResult{true, 0, 0, 0, false};
    } else {
      // leading bits that every candidate's score key shares
      const uint32_t kmin = s_kmin, kmax = s_kmax;
      const int lead_bits = kmin > kmax ? 0 : ((kmin ^ kmax) ? __clz(kmin ^ kmax) : 32);
      const uint64_t lead = lead_bits ? static_cast<uint64_t>(kmax >> (32 - lead_bits)) : 0ull;
      r = radix_select(each_cand, k, hist, s_res, s_seg, /*to_the_end=*/true, lead, lead_bits);
    }
    if (have_pre && (r.take_all || r.eq_all_win)) {
      // contiguous list, exact threshold: count this thread's winners, scan the counts over the block, place
      // them (one pass of votes and an atomic per warp and 32 candidates costs more than both passes here)
      auto wins = [&](uint64_t key) {
        if (r.take_all) return true;
        return (key >> (64 - r.full_bits)) >= r.full;
      };
      int mine = 0;
      for (int i = tid; i < cnt; i += nthr) mine += wins(cand[i]) ? 1 : 0;
      int incl = mine;
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane_id >= o) incl += v;
      }
      if (lane_id == 31) s_seg[warp_id] = static_cast<uint32_t>(incl);
      __syncthreads();
      int before, total;
      warp_totals_scan(s_seg, n_warps, warp_id, before, total);
      before += incl - mine;
      if (tid == 0) s_sel_cnt = total;
      for (int i = tid; i < cnt; i += nthr) {
        const uint64_t key = cand[i];
        if (wins(key)) {
          if (before < k_pow2) sel[before] = key;
          ++before;
        }
      }
    } else {
      each_cand(true, emit(r));
    }
  } else {
    r = radix_select(each_row, k, hist, s_res, s_seg);
    each_row(true, emit(r));
  }
  __syncthreads();
  int n_sel = min(s_sel_cnt, k_pow2);
  if (!r.take_all && !r.eq_all_win) {
    const int n_eq = min(s_eq_cnt, kEqCap);
    int n_eq_pow2 = 32;
    while (n_eq_pow2 < n_eq) n_eq_pow2 <<= 1;
    if (n_eq <= 32) {
      // the usual case (a handful of undecided keys): one warp sorts them in registers
      if (tid < 32) {
        uint64_t key = tid < n_eq ? eq[tid] : 0ull;
#pragma unroll
        for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
          for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const uint64_t other = __shfl_xor_sync(0xffffffffu, key, stride);
            const bool upper = (tid & stride) != 0;           // holds the later slot of the pair
            const bool desc = (tid & size) == 0;
            const bool want_max = (upper != desc);             // descending run: earlier slot keeps the larger key
            key = (want_max == (key > other)) ? key : other;
          }
        }
        eq[tid] = key;
      }
      __syncthreads();
    } else {
      for (int i = n_eq + tid; i < n_eq_pow2; i += nthr) eq[i] = 0;
      bitonic_sort_desc(eq, n_eq_pow2);
    }
    const int take = min(min(r.need_eq, n_eq), k_pow2 - n_sel);
    for (int i = tid; i < take; i += nthr) sel[n_sel + i] = eq[i];
    n_sel += take;
    __syncthreads();
  }

  // ------------------------------------------------------------------ order + write
  if (p.sorted) {
    // counting sort into score buckets; compare-exchange only for short lists and for rows whose scores
    // crowd into a few buckets (the candidate list is free to serve as the scratch array by now)
    if (n_sel <= 64 || !bucket_sort_desc(sel, n_sel, cand, hist, s_seg)) {
      int n_pow2 = 32;
      while (n_pow2 < n_sel) n_pow2 <<= 1;
      for (int i = n_sel + tid; i < n_pow2; i += nthr) sel[i] = 0;
      sort_desc(sel, n_pow2);
    }
  }
  write_row(sel, min(n_sel, k));
}


// Split mode.  Kernel 1 (one CTA per row) samples the row and stores the bin floor (or -1 when
// the fast path does not apply: short rows, rows dominated by ties or invalid scores).
__global__ void __launch_bounds__(1024, 1) topk_floor_kernel(const TopkParams p, int32_t* __restrict__ floor_out) {
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem_raw);
  __shared__ int s_res[3];
  __shared__ uint32_t s_seg[32];
  const int row = blockIdx.x;
  int begin = p.col_begin ? p.col_begin[row] : 0;
  int end = p.col_end ? p.col_end[row] : p.n_cols;
  begin = max(begin, 0);
  end = min(end, p.n_cols);
  const int n = end - begin;
  const float* src = p.scores + row * p.row_stride;
  auto coff = [](int col) { return col; };
  uint32_t bin_floor = 0;
  bool ok = n > kCandCap;  // short rows are cheaper in the last kernel alone
  if (ok) ok = sample_bin_floor(p, src, begin, n, p.k, coff, hist, s_res, s_seg, &bin_floor);
  if (threadIdx.x == 0) floor_out[row] = ok ? static_cast<int32_t>(bin_floor) : -1;
}

// Kernel 2: CTA (split, row) streams its slice of the row; every thread keeps the scores at or
// above the floor in a private list (interleaved in shared memory, no votes, no atomics); the
// lists are then compacted into the row's candidate list in global scratch.  A count above
// kCandCap tells the last kernel that no usable list exists for the row.
constexpr int kCollectThreads = 512;
constexpr int kCollectSlots = kCandCap / kCollectThreads;  // 16 private entries per thread

__global__ void __launch_bounds__(kCollectThreads, 2)
topk_collect_kernel(const TopkParams p, int splits, const int32_t* __restrict__ floor_in) {
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw);  // [slot][thread]
  __shared__ int s_warp_tot[kCollectThreads / 32], s_base, s_overflow;

  const int row = blockIdx.y, split = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int begin = p.col_begin ? p.col_begin[row] : 0;
  int end = p.col_end ? p.col_end[row] : p.n_cols;
  begin = max(begin, 0);
  end = min(end, p.n_cols);
  const int n = end - begin;
  if (n <= 0) return;
  const int fl = floor_in[row];
  if (fl < 0) {
    if (split == 0 && tid == 0) atomicAdd(&p.pre_count[row], kCandCap + 1);
    return;
  }
  const float* src = p.scores + row * p.row_stride;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.scores) & 15) == 0) && ((p.row_stride & 3) == 0);
  auto coff = [](int col) { return col; };
  // smallest float of the floor bin; comparing floats directly is equivalent to comparing bins
  const float thr = fmaxf(ordered_to_float(static_cast<uint32_t>(fl) << 20), -3.402823466e38f);
  const float vmax = p.keep_pos_inf ? INFINITY : 3.402823466e38f;
  if (tid == 0) s_overflow = 0;
  __syncthreads();  // the flag is raised by any thread below; every return above is taken by the whole block
  const int slice = (((n + splits - 1) / splits) + 3) & ~3;
  const int my_begin = begin + split * slice;
  const int my_n = min(slice, end - my_begin);
  int cnt = 0;
  if (my_n > 0) {
    stream_row(src, my_begin, my_n, vec_ok, coff, [&](float v, int col, bool in_range) {
      if (in_range && v >= thr && v <= vmax) {
        if (cnt < kCollectSlots) cand[cnt * kCollectThreads + tid] = make_composite(v, out_position(p, row, col));
        ++cnt;
      }
    });
  }
  if (cnt > kCollectSlots) s_overflow = 1;
  cnt = min(cnt, kCollectSlots);
  // block-wide exclusive scan of the private counts
  int incl = cnt;
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) s_warp_tot[warp] = incl;
  __syncthreads();
  int warp_off = 0, total = 0;
  for (int w = 0; w < kCollectThreads / 32; ++w) {
    if (w == warp) warp_off = total;
    total += s_warp_tot[w];
  }
  if (tid == 0) s_base = atomicAdd(&p.pre_count[row], s_overflow ? kCandCap + 1 : total);
  __syncthreads();
  const int base = s_base;
  if (s_overflow || base + total > kCandCap) return;  // the count already marks the list unusable
  uint64_t* g = p.pre_cand + static_cast<int64_t>(row) * kCandCap + base + warp_off + (incl - cnt);
  for (int j = 0; j < cnt; ++j) g[j] = cand[j * kCollectThreads + tid];
}

// ---------------------------------------------------------------------------------------------
// Many rows of at most 8192 columns: a 256-thread CTA per row with the whole row in shared memory as
// 32-bit order-preserving keys (0 marks an invalid score), several CTAs per SM so that the block-wide
// steps of one row hide behind those of the others.  Exact most-significant-digit radix select with 12 /
// 12 / 8-bit digits over the score key; only when more keys tie at the k-th score than are still wanted
// does it go on over the bit-inverted positions of the tied keys (12 / 12 / 8 bits again), so positions
// are computed for tied keys and for winners only.  The level-0 histogram is filled while the row is
// loaded.  Winners leave in scan order, or through the counting sort when an ordered result is asked for.
// ---------------------------------------------------------------------------------------------
constexpr int kRowsThreads = 256;
constexpr int kRowsMaxCols = 8192;
constexpr int kRowsMinRows = 256;

__global__ void __launch_bounds__(kRowsThreads) topk_rows_kernel(const TopkParams p, int key_words, int k_pow2) {
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem_raw);                 // 4096 bins
  uint32_t* keys = hist + kHistBins;                                      // the row; later the sort's scratch
  uint64_t* sel = reinterpret_cast<uint64_t*>(keys + key_words);          // ordered result only: the winners
  __shared__ int s_res[3], s_cnt;
  __shared__ uint32_t s_seg[32], s_kmin, s_kmax, s_big;

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  int begin = p.col_begin ? p.col_begin[row] : 0;
  int end = p.col_end ? p.col_end[row] : p.n_cols;
  begin = max(begin, 0);
  end = min(end, p.n_cols);
  const int n = max(0, end - begin);
  const float* src = p.scores + row * p.row_stride + begin;
  int32_t* out_idx = p.out_idx + row * p.out_stride;
  float* out_val = p.out_val ? p.out_val + row * p.out_stride : nullptr;
  const int k = p.k;

  for (int i = tid; i < kHistBins; i += kRowsThreads) hist[i] = 0;
  if (tid == 0) {
    s_cnt = 0;
    s_kmin = 0xffffffffu;
    s_kmax = 0u;
    s_big = 0u;
  }
  __syncthreads();
  // ---- load: keys to shared memory, level-0 histogram (top 12 bits) on the way; for an ordered result also
  // the range of the valid keys
  uint32_t klo = 0xffffffffu, khi = 0u;
  for (int base = 0; base < n; base += kRowsThreads * 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * kRowsThreads + tid;
      v[u] = i < n ? __ldg(src + i) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * kRowsThreads + tid;
      if (i < n) {
        const bool ok = score_valid(v[u], p.keep_pos_inf);
        const uint32_t key = ok ? float_to_ordered(v[u]) : 0u;
        keys[i] = key;
        if (ok) {
          atomicAdd(&hist[key >> 20], 1u);
          klo = min(klo, key);
          khi = max(khi, key);
        }
      }
    }
  }
  if (p.sorted) {
    for (int o = 16; o > 0; o >>= 1) {
      klo = min(klo, __shfl_xor_sync(0xffffffffu, klo, o));
      khi = max(khi, __shfl_xor_sync(0xffffffffu, khi, o));
    }
    if ((tid & 31) == 0 && klo <= khi) {
      atomicMin(&s_kmin, klo);
      atomicMax(&s_kmax, khi);
    }
  }
  __syncthreads();

  // ---- radix select.  Decided so far: the top kbits of the score key (tkey), then the top nbits of ~position
  uint32_t tkey = 0, tnpos = 0;
  int kbits = 0, nbits = 0, need = k;
  bool take_all = false;
  auto npos_of = [&](int i) { return ~static_cast<uint32_t>(out_position(p, row, begin + i)); };
#pragma unroll 1
  for (int level = 0; level < 6; ++level) {
    const int width = (level % 3 == 2) ? 8 : 12;
    if (level > 0) {
      for (int i = tid; i < kHistBins; i += kRowsThreads) hist[i] = 0;
      __syncthreads();
      for (int i = tid; i < n; i += kRowsThreads) {
        const uint32_t key = keys[i];
        if (key == 0u) continue;
        if (level < 3) {
          if ((key >> (32 - kbits)) != (tkey >> (32 - kbits))) continue;
          atomicAdd(&hist[(key >> (32 - kbits - width)) & ((1u << width) - 1u)], 1u);
        } else {
          if (key != tkey) continue;
          const uint32_t np = npos_of(i);
          if (nbits > 0 && (np >> (32 - nbits)) != (tnpos >> (32 - nbits))) continue;
          atomicAdd(&hist[(np >> (32 - nbits - width)) & ((1u << width) - 1u)], 1u);
        }
      }
      __syncthreads();
    }
    find_threshold_bin(hist, need, s_res, s_seg);
    const int d = s_res[0], above = s_res[1], in_bin = s_res[2];
    __syncthreads();   // s_res is rewritten by the next level
    if (d < 0) {       // fewer valid keys than wanted (level 0 only): all of them win
      take_all = true;
      break;
    }
    if (level < 3) {
      tkey |= static_cast<uint32_t>(d) << (32 - kbits - width);
      kbits += width;
    } else {
      tnpos |= static_cast<uint32_t>(d) << (32 - nbits - width);
      nbits += width;
    }
    need -= above;
    if (in_bin == need) break;   // everything with these leading bits wins
  }

  // ---- emit
  auto wins = [&](uint32_t key, int i) -> bool {
    if (key == 0u) return false;
    if (take_all) return true;
    if (kbits < 32) return (key >> (32 - kbits)) >= (tkey >> (32 - kbits));
    if (key != tkey) return key > tkey;
    if (nbits == 0) return true;
    return (npos_of(i) >> (32 - nbits)) >= (tnpos >> (32 - nbits));
  };
  const int lane = tid & 31;
  // Ordered result: the winners are counted into 4096 buckets of equal width in KEY space, bucket 0 holding the
  // largest keys (the smallest winner key is the decided threshold prefix, or the row minimum when everything
  // wins; integer arithmetic only), while they are emitted.
  uint32_t win_lo = s_kmin;
  if (!take_all) win_lo = max(win_lo, kbits >= 32 ? tkey : (tkey & ~((1u << (32 - kbits)) - 1u)));
  const uint32_t win_hi = max(s_kmax, win_lo);
  const int span_bits = win_hi > win_lo ? 32 - __clz(win_hi - win_lo) : 0;
  const int bshift = max(0, span_bits - 12);
  auto bucket_of = [&](uint32_t key) { return static_cast<int>((win_hi - key) >> bshift); };   // 0 .. 4095
  const bool use_buckets = p.sorted && k > 64;   // up to 64 winners are ordered by compare-exchange
  if (use_buckets) {
    for (int i = tid; i < kHistBins; i += kRowsThreads) hist[i] = 0;   // the radix levels are done with it
    __syncthreads();
  }
  for (int base = 0; base < n; base += kRowsThreads) {
    const int i = base + tid;
    const uint32_t key = i < n ? keys[i] : 0u;
    const bool win = i < n && wins(key, i);
    const unsigned m = __ballot_sync(0xffffffffu, win);
    if (m == 0) continue;
    const int leader = __ffs(m) - 1;
    int slot = 0;
    if (lane == leader) slot = atomicAdd(&s_cnt, __popc(m));
    slot = __shfl_sync(0xffffffffu, slot, leader) + __popc(m & ((1u << lane) - 1u));
    if (win && slot < k) {
      const int32_t pos = out_position(p, row, begin + i);
      if (p.sorted) {
        sel[slot] = (static_cast<uint64_t>(key) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(pos));
        if (use_buckets) atomicAdd(&hist[bucket_of(key)], 1u);
      } else {
        out_idx[slot] = pos;
        if (out_val) out_val[slot] = ordered_to_float(key);
      }
    }
  }
  __syncthreads();
  const int n_sel = min(s_cnt, k);
  if (p.sorted) {
    uint64_t* tmp = reinterpret_cast<uint64_t*>(keys);
    bool done = false;
    if (use_buckets && n_sel > 64) {
      // exclusive scan of the bucket counts (thread t owns buckets 16t .. 16t+15); hist[b] <- first slot of bucket b
      constexpr int kPer = kHistBins / kRowsThreads;
      uint32_t sum = 0, big = 0;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const uint32_t c = hist[tid * kPer + j];
        sum += c;
        big = max(big, c);
      }
      uint32_t incl = sum;
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      for (int o = 16; o > 0; o >>= 1) big = max(big, __shfl_xor_sync(0xffffffffu, big, o));
      if (lane == 31) s_seg[tid >> 5] = incl;
      if (lane == 0 && big > static_cast<uint32_t>(kBucketMax)) atomicMax(&s_big, big);
      __syncthreads();
      if (s_big == 0u) {     // uniform; otherwise long runs of equal-ish keys: the general sort below
        int before_w, total_w;
        warp_totals_scan(s_seg, kRowsThreads / 32, tid >> 5, before_w, total_w);
        uint32_t before = incl - sum + static_cast<uint32_t>(before_w);
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          const uint32_t c = hist[tid * kPer + j];
          hist[tid * kPer + j] = before;
          before += c;
        }
        __syncthreads();
        for (int i = tid; i < n_sel; i += kRowsThreads) {
          const uint64_t key = sel[i];
          tmp[atomicAdd(&hist[bucket_of(static_cast<uint32_t>(key >> 32))], 1u)] = key;   // hist[b] ends as one past bucket b
        }
        __syncthreads();
        // exact rank inside the bucket by the full composite, then straight to the result
        for (int i = tid; i < n_sel; i += kRowsThreads) {
          const uint64_t key = tmp[i];
          const int b = bucket_of(static_cast<uint32_t>(key >> 32));
          const int e = static_cast<int>(hist[b]);
          const int s0 = b == 0 ? 0 : static_cast<int>(hist[b - 1]);
          int rank = 0;
          for (int j = s0; j < e; ++j) rank += tmp[j] > key;
          out_idx[s0 + rank] = static_cast<int32_t>(~static_cast<uint32_t>(key & 0xffffffffu));
          if (out_val) out_val[s0 + rank] = ordered_to_float(static_cast<uint32_t>(key >> 32));
        }
        done = true;
      }
    }
    if (!done) {
      if (n_sel > 1 && (n_sel <= 64 || !bucket_sort_desc(sel, n_sel, tmp, hist, s_seg))) {
        int n_pow2 = 64;
        while (n_pow2 < n_sel) n_pow2 <<= 1;
        for (int i = n_sel + tid; i < n_pow2; i += kRowsThreads) sel[i] = 0;
        __syncthreads();
        sort_desc(sel, n_pow2);
      }
      for (int j = tid; j < n_sel; j += kRowsThreads) {
        const uint64_t key = sel[j];
        out_idx[j] = static_cast<int32_t>(~static_cast<uint32_t>(key & 0xffffffffu));
        if (out_val) out_val[j] = ordered_to_float(static_cast<uint32_t>(key >> 32));
      }
    }
  }
  for (int j = n_sel + tid; j < k; j += kRowsThreads) {
    out_idx[j] = -1;
    if (out_val) out_val[j] = -INFINITY;
  }
  (void)k_pow2;
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_topk_select(const float* scores, int64_t row_stride, int32_t n_rows, int32_t n_cols,
                                   const int32_t* col_begin, const int32_t* col_end, int32_t k,
                                   int32_t keep_pos_inf, int32_t sorted, const int32_t* pos_map,
                                   int64_t pos_map_stride, const int32_t* page_table, int64_t page_table_stride,
                                   int32_t page_size, const int32_t* row_pos_offset, int32_t seg_cols,
                                   int64_t seg_stride, const int64_t* seg_offsets, int32_t* out_idx,
                                   float* out_val, int64_t out_stride, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!scores || !out_idx || n_rows < 0 || n_cols < 0 || k < 1 || k > kCandCap || out_stride < k ||
      (seg_cols <= 0 && row_stride < n_cols) || seg_cols < 0) {
    set_last_error("b200dsa_topk_select: bad argument (need 1<=k<=8192, out_stride>=k, row_stride>=n_cols)");
    return B200DSA_EINVAL;
  }
  if (page_table && page_size <= 0) {
    set_last_error("b200dsa_topk_select: page_table given with page_size <= 0");
    return B200DSA_EINVAL;
  }
  TopkParams p{scores, row_stride, n_rows, n_cols, col_begin, col_end, k, keep_pos_inf, pos_map, pos_map_stride,
               page_table, page_table_stride, page_size, row_pos_offset, out_idx, out_val, out_stride, sorted,
               seg_cols, seg_stride};
  if (seg_offsets) {
    const int n_seg = seg_cols > 0 ? (n_cols + seg_cols - 1) / seg_cols : 0;
    if (n_seg < 1 || n_seg > 8) {
      set_last_error("b200dsa_topk_select: seg_offsets needs seg_cols > 0 and at most 8 segments");
      return B200DSA_EINVAL;
    }
    p.seg_off_n = n_seg;
    for (int r = 0; r < n_seg; ++r) p.seg_off[r] = seg_offsets[r];
  }
  int k_pow2 = 32;
  while (k_pow2 < k) k_pow2 <<= 1;
  // many rows that fit shared memory: a small CTA per row, several per SM
  if (n_rows >= kRowsMinRows && n_cols <= kRowsMaxCols && k <= 4096 && seg_cols == 0) {
    const int sel_entries = sorted ? max(k_pow2, 64) : 0;
    const int key_words = max((n_cols + 3) & ~3, 2 * sel_entries);
    const size_t smem_rows = kHistBins * sizeof(uint32_t) + static_cast<size_t>(key_words) * 4 +
                             static_cast<size_t>(sel_entries) * 8;
    cudaError_t e3 = cudaFuncSetAttribute(topk_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kHistBins * 4 + kRowsMaxCols * 4 + 4096 * 8);
    if (e3 == cudaSuccess)
      e3 = launch_chained(topk_rows_kernel, dim3(n_rows), dim3(kRowsThreads), smem_rows,
                          static_cast<cudaStream_t>(stream), p, key_words, k_pow2);
    if (e3 == cudaSuccess) e3 = cudaGetLastError();
    if (e3 != cudaSuccess) {
      set_last_error(cudaGetErrorString(e3));
      return B200DSA_ECUDA;
    }
    return B200DSA_OK;
  }
  // rows that fit the candidate list entirely need no larger list than the row: smaller CTAs, more of
  // them per SM (block top-m, causal prefill)
  int cand_cap = kCandCap;
  if (n_cols <= kCandCap) {
    cand_cap = 2048;   // at least 16 KB: the register path keeps its second histogram there
    while (cand_cap < n_cols) cand_cap <<= 1;
  } else if (k > kCandCap / 2) {
    // a large k (MISA's stage-1 top-8192) needs room for k plus the sampling margin: the long list, which
    // together with 8192 winners is the largest shared-memory configuration
    cand_cap = kListCap;
  }
  const size_t smem = kHistBins * sizeof(uint32_t) + (static_cast<size_t>(cand_cap) + kEqCap + k_pow2) * sizeof(uint64_t);
  cudaError_t e = cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kMaxSelectSmem);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  const int threads = n_cols > 4096 ? 1024 : (n_cols > 2048 ? 512 : 256);   // at most eight columns per thread up to 8192
  e = launch_chained(topk_select_kernel, dim3(n_rows), dim3(threads), smem, static_cast<cudaStream_t>(stream), p, k_pow2,
                     cand_cap);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_topk_select_split(const float* scores, int64_t row_stride, int32_t n_rows, int32_t n_cols,
                                         const int32_t* col_begin, const int32_t* col_end, int32_t k,
                                         int32_t keep_pos_inf, int32_t sorted, const int32_t* row_pos_offset,
                                         int32_t splits, void* scratch_cand, int32_t* scratch_count,
                                         int32_t* out_idx, float* out_val, int64_t out_stride, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!scores || !out_idx || !scratch_cand || !scratch_count || n_rows < 0 || n_cols < 0 || k < 1 ||
      k > kCandCap || out_stride < k || row_stride < n_cols || splits < 1 || splits > 64) {
    set_last_error("b200dsa_topk_select_split: bad argument (1<=k<=8192, 1<=splits<=64, scratch required)");
    return B200DSA_EINVAL;
  }
  if (reinterpret_cast<uintptr_t>(scratch_cand) & 7) {
    set_last_error("b200dsa_topk_select_split: scratch_cand must be 8-byte aligned");
    return B200DSA_EALIGN;
  }
  TopkParams p{scores, row_stride, n_rows, n_cols, col_begin, col_end, k, keep_pos_inf, nullptr, 0, nullptr, 0, 0,
               row_pos_offset, out_idx, out_val, out_stride, sorted, 0, 0,
               static_cast<uint64_t*>(scratch_cand), scratch_count};
  int k_pow2 = 32;
  while (k_pow2 < k) k_pow2 <<= 1;
  const size_t smem_f = kHistBins * sizeof(uint32_t);
  const size_t smem_a = kCandCap * sizeof(uint64_t);
  const size_t smem_b = kHistBins * sizeof(uint32_t) + (kCandCap + kEqCap + k_pow2) * sizeof(uint64_t);
  cudaError_t e = cudaFuncSetAttribute(topk_collect_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem_a));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMaxSelectSmem);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t* floor_bin = scratch_count + n_rows;  // second half of the int32 scratch
  e = launch_chained(topk_floor_kernel, dim3(n_rows), dim3(1024), smem_f, st, p, floor_bin);
  if (e == cudaSuccess)
    e = launch_chained(topk_collect_kernel, dim3(splits, n_rows), dim3(kCollectThreads), smem_a, st, p, splits,
                       static_cast<const int32_t*>(floor_bin));
  if (e == cudaSuccess) e = launch_chained(topk_select_kernel, dim3(n_rows), dim3(1024), smem_b, st, p, k_pow2,
                                             static_cast<int>(kCandCap));
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

// Last kernel of the fused selection: exact top-k of every row from the candidate list the indexer's
// epilogue collected (see indexer_paged.cu), falling back to the row's logits when a list cannot be
// proven complete (scores may be NULL: then *status reports it).
namespace b200dsa {
int topk_select_from_lists(const float* scores, int64_t row_stride, int32_t n_rows, int32_t n_cols,
                           const int32_t* col_end, int32_t k, int32_t sorted, const int32_t* row_pos_offset,
                           uint64_t* cand, int32_t* count, uint32_t* floor_bits, int32_t* out_idx, float* out_val,
                           int64_t out_stride, int32_t* status, const PeerLinkDev* push, int64_t push_off,
                           cudaStream_t stream) {
  TopkParams p{scores, row_stride, n_rows, n_cols, nullptr, col_end, k, 0, nullptr, 0, nullptr, 0, 0,
               row_pos_offset, out_idx, out_val, out_stride, sorted, 0, 0, cand, count};
  p.pre_floor = floor_bits;
  p.status = status;
  if (push) {
    p.push_on = 1;
    p.link = *push;
    p.push_off = push_off;
  }
  int k_pow2 = 32;
  while (k_pow2 < k) k_pow2 <<= 1;
  const size_t smem = kHistBins * sizeof(uint32_t) + (kListCap + kEqCap + k_pow2) * sizeof(uint64_t);
  cudaError_t e = cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSelectSmem);
  if (e == cudaSuccess)
    e = launch_chained(topk_select_kernel, dim3(n_rows), dim3(1024), smem, stream, p, k_pow2, static_cast<int>(kListCap));
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
}  // namespace b200dsa

extern "C" int b200dsa_topk_merge_owned(const int32_t* recv, int32_t world, int32_t n_rows, int32_t k, int32_t sorted,
                                        int32_t own_lo, int32_t own_hi, int32_t* out_idx, int64_t out_stride,
                                        int32_t* owned, int64_t owned_stride, int32_t* owned_count,
                                        const b200dsa_peer_link* link, int32_t* status, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!recv || !out_idx || !owned || !owned_count || !status || world < 1 || world > 8 || n_rows < 0 || k < 1 ||
      k > kCandCap || out_stride < k || owned_stride < k || (reinterpret_cast<uintptr_t>(recv) & 15) || (k & 3)) {
    set_last_error("b200dsa_topk_merge_owned: bad argument (1 <= world <= 8, k a multiple of 4, strides >= k)");
    return B200DSA_EINVAL;
  }
  // column c of row r = candidate c % k of rank c / k: scores at recv + rank*n_rows*2k + r*2k + k + c%k,
  // positions k ints before them
  const float* scores = reinterpret_cast<const float*>(recv) + k;
  TopkParams p{scores, 2 * static_cast<int64_t>(k), n_rows, world * k, nullptr, nullptr, k, 0, recv,
               2 * static_cast<int64_t>(k), nullptr, 0, 0, nullptr, out_idx, nullptr, out_stride, sorted, k,
               static_cast<int64_t>(n_rows) * 2 * k};
  p.status = status;
  p.own_lo = own_lo;
  p.own_hi = own_hi;
  p.owned = owned;
  p.owned_stride = owned_stride;
  p.owned_count = owned_count;
  if (link) {
    if (!make_link(link, &p.link, "b200dsa_topk_merge_owned")) return B200DSA_EINVAL;
    p.wait_on = 1;
  }
  int k_pow2 = 32;
  while (k_pow2 < k) k_pow2 <<= 1;
  int cand_cap = kCandCap;
  if (world * k <= kCandCap) {
    cand_cap = 2048;
    while (cand_cap < world * k) cand_cap <<= 1;
  }
  const size_t smem = kHistBins * sizeof(uint32_t) + (static_cast<size_t>(cand_cap) + kEqCap + k_pow2) * sizeof(uint64_t);
  cudaError_t e = cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kMaxSelectSmem);
  const int threads = world * k > 4096 ? 1024 : (world * k > 2048 ? 512 : 256);
  if (e == cudaSuccess)
    e = launch_chained(topk_select_kernel, dim3(n_rows), dim3(threads), smem, static_cast<cudaStream_t>(stream), p,
                       k_pow2, cand_cap);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

// ---------------------------------------------------------------------------------------------
// Split top-k without caller-provided scratch.
//
// Some hosts of this library cannot obtain device memory at call time: a serving engine that
// handed nearly all of the GPU to its own memory pool at start-up (a later cudaMalloc from a
// plug-in can simply fail there), or a plain C caller that owns no workspace and no allocator.
// For them the candidate lists and counters live in a fixed array inside the library image.
// The price: every device that loads the library carries the 4 MB until the process exits, the
// row count is capped, and all calls share the one array.
// ---------------------------------------------------------------------------------------------
namespace b200dsa {

constexpr int kStaticMaxRows = 64;
constexpr size_t kStaticCandBytes = static_cast<size_t>(kStaticMaxRows) * kCandCap * sizeof(uint64_t);  // 4 MiB
constexpr size_t kStaticIntBytes = 2 * kStaticMaxRows * sizeof(int32_t);

// candidate lists first, then 2*rows int32 (per-row counters, per-row bin floors)
static __device__ __align__(256) unsigned char g_topk_static_scratch[kStaticCandBytes + kStaticIntBytes];

}  // namespace b200dsa

#include <mutex>

extern "C" int b200dsa_topk_select_split_static(const float* scores, int64_t row_stride, int32_t n_rows,
                                                int32_t n_cols, const int32_t* col_begin, const int32_t* col_end,
                                                int32_t k, int32_t keep_pos_inf, int32_t sorted,
                                                const int32_t* row_pos_offset, int32_t splits, int32_t* out_idx,
                                                float* out_val, int64_t out_stride, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (n_rows < 0 || n_rows > kStaticMaxRows) {
    set_last_error("b200dsa_topk_select_split_static: n_rows exceeds the built-in scratch (at most 64 rows); "
                   "use b200dsa_topk_select_split with caller-provided scratch for larger batches");
    return B200DSA_EINVAL;
  }
  // The array's name is only a host-side handle; the device address has to be asked for, once
  // per device, while that device is current.
  constexpr int kMaxDevices = 64;
  static void* dev_ptr[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_last_error("b200dsa_topk_select_split_static: cannot identify the current device");
    return B200DSA_ECUDA;
  }
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!dev_ptr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_topk_static_scratch);
      if (e != cudaSuccess || !p) {
        set_last_error("b200dsa_topk_select_split_static: cudaGetSymbolAddress failed for the built-in scratch");
        return B200DSA_ECUDA;
      }
      dev_ptr[dev] = p;
    }
    base = dev_ptr[dev];
  }
  unsigned char* bytes = static_cast<unsigned char*>(base);
  int32_t* counters = reinterpret_cast<int32_t*>(bytes + kStaticCandBytes);
  // The array keeps whatever the previous call (possibly of another shape, possibly cut short)
  // left behind; the per-row counters are the only part that must start at zero.
  e = cudaMemsetAsync(counters, 0, kStaticIntBytes, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return b200dsa_topk_select_split(scores, row_stride, n_rows, n_cols, col_begin, col_end, k, keep_pos_inf, sorted,
                                   row_pos_offset, splits, bytes, counters, out_idx, out_val, out_stride, stream);
}
