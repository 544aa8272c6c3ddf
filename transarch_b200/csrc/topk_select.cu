// Row-wise top-k over fp32 scores, one CTA per row.
//
// Scores are mapped to order-preserving 32-bit keys and paired with the bit-inverted output
// position into a unique 64-bit composite, so "k largest composites" is a total order:
// descending score, ties towards the lowest position.
//
// Fast path (reads the row about once):
//   1. contiguous chunks spread over the row are sampled into a 4096-bin histogram of the
//      top 12 key bits (warp-aggregated shared-memory atomics) and a bin is chosen so that,
//      with a 6-sigma margin, at least k row elements lie at or above it;
//   2. one streaming pass appends every element at or above that bin to a shared-memory
//      candidate list (warp-aggregated append);
//   3. the candidates are bitonic-sorted in shared memory and the first k are written.
// Rows that fit the candidate list entirely skip step 1.
// Exact fallback (any distribution, massive ties): most-significant-digit radix select over
// the 64-bit composite, re-reading the row per digit until the undecided bin fits the list.
#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kHistBins = 4096;
constexpr int kCandCap = 8192;   // candidate list entries (64 KB)
constexpr int kEqCap = 4096;     // undecided-bin list of the fallback (32 KB)
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
};

__device__ __forceinline__ bool score_valid(float v, int keep_pos_inf) {
  // -inf, NaN never; +inf on request
  if (v != v) return false;
  if (v == -INFINITY) return false;
  if (v == INFINITY) return keep_pos_inf != 0;
  return true;
}

__device__ __forceinline__ int32_t out_position(const TopkParams& p, int row, int col) {
  int32_t pos;
  if (p.pos_map) {
    pos = p.pos_map[row * p.pos_map_stride + col];
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

// warp-aggregated histogram increment
__device__ __forceinline__ void hist_add(uint32_t* hist, uint32_t bin, bool active) {
  unsigned act = __ballot_sync(0xffffffffu, active);
  if (!active) return;
  unsigned peers = __match_any_sync(act, bin);
  int leader = __ffs(peers) - 1;
  if ((threadIdx.x & 31) == leader) atomicAdd(&hist[bin], __popc(peers));
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

// In-place descending bitonic sort of n (power of two) keys in shared memory.
__device__ void bitonic_sort_desc(uint64_t* a, int n) {
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
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

// Warp 0: find the highest bin d such that (#elements in bins >= d) >= need.
// Writes res[0]=d (or -1 when the whole histogram holds fewer than need), res[1]=count in
// bins above d, res[2]=hist[d].
__device__ void find_threshold_bin(const uint32_t* hist, int nbins, int need, int* res) {
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  const int per = nbins / 32;
  // lane 0 owns the highest bins
  const int hi = nbins - lane * per;  // exclusive
  uint32_t mine = 0;
  for (int b = hi - 1; b >= hi - per; --b) mine += hist[b];
  uint32_t incl = mine;  // inclusive prefix over lanes (= suffix over bins)
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  uint32_t excl = incl - mine;
  bool owner = (excl < static_cast<uint32_t>(need)) && (incl >= static_cast<uint32_t>(need));
  unsigned who = __ballot_sync(0xffffffffu, owner);
  const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
  if (who == 0) {
    if (lane == 0) {
      res[0] = -1;
      res[1] = static_cast<int>(total);
      res[2] = 0;
    }
    return;
  }
  if (owner) {
    uint32_t above = excl;
    for (int b = hi - 1; b >= hi - per; --b) {
      uint32_t h = hist[b];
      if (above + h >= static_cast<uint32_t>(need)) {
        res[0] = b;
        res[1] = static_cast<int>(above);
        res[2] = static_cast<int>(h);
        break;
      }
      above += h;
    }
  }
}

__global__ void __launch_bounds__(1024, 1) topk_select_kernel(const TopkParams p, int k_pow2) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem_raw);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw + kHistBins * sizeof(uint32_t));
  uint64_t* eq = cand + kCandCap;
  __shared__ int s_cnt, s_eq_cnt, s_res[3];

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  int begin = p.col_begin ? p.col_begin[row] : 0;
  int end = p.col_end ? p.col_end[row] : p.n_cols;
  begin = max(begin, 0);
  end = min(end, p.n_cols);
  const int n = end - begin;
  const float* src = p.scores + row * p.row_stride;
  int32_t* out_idx = p.out_idx + row * p.out_stride;
  float* out_val = p.out_val ? p.out_val + row * p.out_stride : nullptr;
  const int k = p.k;

  if (n <= 0) {
    for (int j = tid; j < k; j += nthr) {
      out_idx[j] = -1;
      if (out_val) out_val[j] = -INFINITY;
    }
    return;
  }

  if (tid == 0) {
    s_cnt = 0;
    s_eq_cnt = 0;
  }
  __syncthreads();
  bool done = false;
  int n_final = 0;  // entries in cand to be sorted

  // ------------------------------------------------------------------ fast paths
  uint32_t bin_floor = 0;
  bool try_fast = true;
  if (n > kCandCap) {
    // sample histogram
    for (int i = tid; i < kHistBins; i += nthr) hist[i] = 0;
    __syncthreads();
    const int n_chunks = kSampleMax / kSampleChunk;  // 64
    const int m = n_chunks * kSampleChunk;
    const int64_t step = n / n_chunks;               // >= 128 since n > 8192
    for (int i = tid; i < m; i += nthr) {
      int c = i / kSampleChunk;
      int col = begin + static_cast<int>(c * step) + (i - c * kSampleChunk);
      float v = src[col];
      bool ok = score_valid(v, p.keep_pos_inf);
      hist_add(hist, float_to_ordered(v) >> 20, ok);
    }
    __syncthreads();
    // elements wanted at or above the bin: k + 6 sigma of the scaled-up sample count
    const float ratio = static_cast<float>(n) / static_cast<float>(m);
    const float want_full = k + 6.0f * sqrtf(2.0f * k * ratio) + 32.0f;
    if (want_full > 0.8f * kCandCap) {
      try_fast = false;
    } else {
      int want_sample = static_cast<int>(ceilf(want_full / ratio));
      find_threshold_bin(hist, kHistBins, want_sample, s_res);
      __syncthreads();
      if (s_res[0] < 0) try_fast = false;  // sample too sparse (many invalid entries)
      else bin_floor = static_cast<uint32_t>(s_res[0]);
    }
    __syncthreads();
  }

  if (try_fast) {
    // streaming collect of everything at or above bin_floor
    const int n_round = (n + 31) & ~31;
    for (int i = tid; i < n_round; i += nthr) {
      bool take = false;
      uint64_t key = 0;
      if (i < n) {
        float v = src[begin + i];
        if (score_valid(v, p.keep_pos_inf) && (float_to_ordered(v) >> 20) >= bin_floor) {
          take = true;
          key = make_composite(v, out_position(p, row, begin + i));
        }
      }
      list_append(cand, &s_cnt, kCandCap, key, take);
    }
    __syncthreads();
    const int cnt = s_cnt;
    if (cnt <= kCandCap && (cnt >= k || n <= kCandCap)) {
      done = true;
      n_final = cnt;
    }
    __syncthreads();
  }

  // ------------------------------------------------------------------ exact fallback
  if (!done) {
    uint64_t prefix = 0;
    int prefix_bits = 0;
    int need = k;
    int digit_bits = 12;
    uint64_t full = 0;
    int full_bits = 0;
    int need_eq = 0;
    bool take_all = false;
    for (int level = 0; level < 6; ++level) {
      digit_bits = (level % 3 == 2) ? 8 : 12;
      const int shift = 64 - prefix_bits - digit_bits;
      const bool need_pos = (prefix_bits + digit_bits) > 32;
      for (int i = tid; i < kHistBins; i += nthr) hist[i] = 0;
      __syncthreads();
      const int n_round = (n + 31) & ~31;
      for (int i = tid; i < n_round; i += nthr) {
        bool ok = false;
        uint32_t bin = 0;
        if (i < n) {
          float v = src[begin + i];
          if (score_valid(v, p.keep_pos_inf)) {
            uint64_t key = need_pos ? make_composite(v, out_position(p, row, begin + i))
                                    : (static_cast<uint64_t>(float_to_ordered(v)) << 32);
            if (prefix_bits == 0 || (key >> (64 - prefix_bits)) == prefix) {
              ok = true;
              bin = static_cast<uint32_t>(key >> shift) & ((1u << digit_bits) - 1);
            }
          }
        }
        hist_add(hist, bin, ok);
      }
      __syncthreads();
      find_threshold_bin(hist, kHistBins, need, s_res);
      __syncthreads();
      const int d = s_res[0];
      if (d < 0) {  // fewer valid elements than k: everything valid is selected (level 0 only)
        take_all = true;
        break;
      }
      const int above = s_res[1];
      const int in_bin = s_res[2];
      full = (prefix << digit_bits) | static_cast<uint64_t>(d);
      full_bits = prefix_bits + digit_bits;
      need_eq = need - above;
      if (in_bin <= kEqCap || level == 5) break;
      prefix = full;
      prefix_bits = full_bits;
      need = need_eq;
      __syncthreads();
    }
    if (tid == 0) {
      s_cnt = 0;
      s_eq_cnt = 0;
    }
    __syncthreads();
    const int n_round = (n + 31) & ~31;
    for (int i = tid; i < n_round; i += nthr) {
      bool direct = false, tie = false;
      uint64_t key = 0;
      if (i < n) {
        float v = src[begin + i];
        if (score_valid(v, p.keep_pos_inf)) {
          key = make_composite(v, out_position(p, row, begin + i));
          if (take_all) {
            direct = true;
          } else {
            uint64_t top = key >> (64 - full_bits);
            direct = top > full;
            tie = top == full;
          }
        }
      }
      list_append(cand, &s_cnt, kCandCap, key, direct);
      list_append(eq, &s_eq_cnt, kEqCap, key, tie);
    }
    __syncthreads();
    int n_direct = s_cnt;
    if (!take_all) {
      int n_eq = min(s_eq_cnt, kEqCap);
      int n_eq_pow2 = 32;
      while (n_eq_pow2 < n_eq) n_eq_pow2 <<= 1;
      for (int i = n_eq + tid; i < n_eq_pow2; i += nthr) eq[i] = 0;
      bitonic_sort_desc(eq, n_eq_pow2);
      int take = min(need_eq, n_eq);
      for (int i = tid; i < take; i += nthr) cand[n_direct + i] = eq[i];
      n_direct += take;
    }
    n_final = n_direct;
    __syncthreads();
  }

  // ------------------------------------------------------------------ sort + write
  int n_pow2 = 32;
  while (n_pow2 < n_final) n_pow2 <<= 1;
  for (int i = n_final + tid; i < n_pow2; i += nthr) cand[i] = 0;
  bitonic_sort_desc(cand, n_pow2);
  const int n_out = min(n_final, k);
  for (int j = tid; j < k; j += nthr) {
    if (j < n_out) {
      uint64_t key = cand[j];
      out_idx[j] = static_cast<int32_t>(~static_cast<uint32_t>(key & 0xffffffffu));
      if (out_val) out_val[j] = ordered_to_float(static_cast<uint32_t>(key >> 32));
    } else {
      out_idx[j] = -1;
      if (out_val) out_val[j] = -INFINITY;
    }
  }
  (void)k_pow2;
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_topk_select(const float* scores, int64_t row_stride, int32_t n_rows, int32_t n_cols,
                                   const int32_t* col_begin, const int32_t* col_end, int32_t k,
                                   int32_t keep_pos_inf, const int32_t* pos_map, int64_t pos_map_stride,
                                   const int32_t* page_table, int64_t page_table_stride, int32_t page_size,
                                   const int32_t* row_pos_offset, int32_t* out_idx, float* out_val,
                                   int64_t out_stride, void* stream) {
  if (n_rows == 0) return B200DSA_OK;
  if (!scores || !out_idx || n_rows < 0 || n_cols < 0 || k < 1 || k > kCandCap || out_stride < k ||
      row_stride < n_cols) {
    set_last_error("b200dsa_topk_select: bad argument (need 1<=k<=8192, out_stride>=k, row_stride>=n_cols)");
    return B200DSA_EINVAL;
  }
  if (page_table && page_size <= 0) {
    set_last_error("b200dsa_topk_select: page_table given with page_size <= 0");
    return B200DSA_EINVAL;
  }
  TopkParams p{scores, row_stride, n_rows, n_cols, col_begin, col_end, k, keep_pos_inf, pos_map, pos_map_stride,
               page_table, page_table_stride, page_size, row_pos_offset, out_idx, out_val, out_stride};
  const size_t smem = kHistBins * sizeof(uint32_t) + (kCandCap + kEqCap) * sizeof(uint64_t);
  cudaError_t e = cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  const int threads = n_cols > 16384 ? 1024 : 512;
  int k_pow2 = 32;
  while (k_pow2 < k) k_pow2 <<= 1;
  topk_select_kernel<<<n_rows, threads, smem, static_cast<cudaStream_t>(stream)>>>(p, k_pow2);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
