// Log-sum-exp combine of key-sharded attention partials over NVLink peer memory, in one kernel.
//
// Every rank owns an exchange buffer of identical layout that all ranks of the node have mapped
// (CUDA IPC).  After its attention kernel a rank's buffer holds its normalised partial context
// (bf16 [n_rows, 512]) and lse (fp32 [n_rows]).  The kernel then
//   1. tells every peer "my partial of step e is ready" and waits for the same word from each peer,
//   2. for the rows it owns (a contiguous 1/world slice) loads the partials of all ranks with plain
//      peer loads, merges them   m = max_r lse_r,  w_r = exp(lse_r - m),
//      out = sum_r w_r ctx_r / sum_r w_r,  lse_out = m + log sum_r w_r
//      in fp32 and stores the bf16 result row into the result area of EVERY rank,
//   3. tells every peer "my slice is written" and leaves only when all peers said so.
// Step 3 makes the result complete on this rank when the kernel ends, and keeps a fast rank from
// overwriting its partial (next step) while a slow rank still reads it.
//
// Flags are step numbers that only grow, so nothing is ever reset.  The step number lives in local
// device memory and is advanced by the kernel itself, so a captured launch can be replayed.  Every
// wait is bounded: on expiry the status word gets kDevWaitTimeout and the kernel carries on and ends.
// Ranks are different GPUs; two such kernels must never be made to wait for each other on one GPU.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <string.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kPeerMaxRanks = 8;
constexpr int kPeerDv = 512;
constexpr long long kPeerWaitCyclesDefault = 1ll << 31;   // about a second
// Limit of every wait for a peer, in SM clock cycles; process-wide, set by b200dsa_peer_set_wait_limit
// and copied into the parameters of each launch.
static long long g_peer_wait_cycles = kPeerWaitCyclesDefault;
long long peer_wait_cycles() { return g_peer_wait_cycles; }
constexpr int kPeerDoneSlot = 16;                  // flags: ready[0..7], done[16..23] (uint32 words)

struct PeerCombineParams {
  unsigned char* buf[kPeerMaxRanks];  // exchange buffer of every rank (buf[rank] is local memory)
  int rank, world;
  int64_t n_rows;
  int64_t off_ctx, off_lse, off_out, off_lse_out, off_flags;   // byte offsets, the same on every rank
  int32_t* state;                     // local: [0] launches completed, [1] blocks finished in this launch
  int32_t* status;
  int no_sync;                        // skip the flag exchange (sequential emulation of ranks on one GPU)
  int pre_signalled;                  // the "partial ready" flags were raised by the kernel that wrote the partial
  int local_only;                     // reduce-scatter form: keep the merged rows of this rank's slice, tell nobody
  long long wait_cycles;              // bound of every wait for a peer's flag
};

__device__ __forceinline__ void fma_bf16x8(float* acc, const uint4& v, float w) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h[j]);
    acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
    acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
  }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float* a) {
  uint4 v;
  __nv_bfloat162 h;
  h = __floats2bfloat162_rn(a[0], a[1]); v.x = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(a[2], a[3]); v.y = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(a[4], a[5]); v.z = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(a[6], a[7]); v.w = *reinterpret_cast<uint32_t*>(&h);
  return v;
}

__global__ void __launch_bounds__(256, 2) peer_lse_combine_kernel(const PeerCombineParams p) {
  // nothing may be signalled to the peers before the kernels that produced this rank's partial are done
  pdl_launch_dependents();
  pdl_wait_prior();
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t step = static_cast<uint32_t>(*reinterpret_cast<volatile int32_t*>(p.state)) + 1u;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(p.buf[p.rank] + p.off_flags);

  // ---- 1. partials of this step are ready everywhere
  if (!p.no_sync) {
    if (blockIdx.x == 0 && tid < p.world && !p.pre_signalled)
      st_release_sys(reinterpret_cast<uint32_t*>(p.buf[tid] + p.off_flags) + p.rank, step);
    if (tid < p.world && !wait_step(my_flags + tid, step, p.wait_cycles)) atomicMax(p.status, kDevWaitTimeout);
    __syncthreads();
  }

  // ---- 2. merge the rows this rank owns, one warp per row; lane owns dims [8*lane, 8*lane+8) and
  //         [256 + 8*lane, 256 + 8*lane + 8): two fully coalesced 512-byte requests per partial
  const int64_t per = (p.n_rows + p.world - 1) / p.world;
  const int64_t r_begin = p.rank * per;
  const int64_t r_end = r_begin + per < p.n_rows ? r_begin + per : p.n_rows;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t row = r_begin + static_cast<int64_t>(blockIdx.x) * 8 + warp; row < r_end; row += warps_total) {
    // every load of the row is issued before the first use: one NVLink round trip per row, not two
    uint4 va[kPeerMaxRanks], vb[kPeerMaxRanks];
#pragma unroll
    for (int r = 0; r < kPeerMaxRanks; ++r) {
      if (r < p.world) {
        const unsigned char* src = p.buf[r] + p.off_ctx + row * (kPeerDv * 2) + lane * 16;
        va[r] = ld_sys_v4(src);
        vb[r] = ld_sys_v4(src + 512);
      }
    }
    float l = -INFINITY;
    if (lane < p.world) l = ld_sys_f32(reinterpret_cast<const float*>(p.buf[lane] + p.off_lse) + row);
    float m = l;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float w = (l == -INFINITY) ? 0.f : expf(l - m);
    float den = w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float inv = den > 0.f ? 1.0f / den : 0.f;
#pragma unroll
    for (int r = 0; r < kPeerMaxRanks; ++r) {
      if (r < p.world) {
        const float wr = __shfl_sync(0xffffffffu, w, r) * inv;
        if (wr != 0.f) {                      // an empty partial may hold anything
          fma_bf16x8(a, va[r], wr);
          fma_bf16x8(b, vb[r], wr);
        }
      }
    }
    const uint4 oa = pack_bf16x8(a), ob = pack_bf16x8(b);
    const float lse_out = den > 0.f ? m + logf(den) : -INFINITY;
    if (p.local_only) {
      unsigned char* dst = p.buf[p.rank] + p.off_out + row * (kPeerDv * 2) + lane * 16;
      *reinterpret_cast<uint4*>(dst) = oa;
      *reinterpret_cast<uint4*>(dst + 512) = ob;
      if (lane == 0) reinterpret_cast<float*>(p.buf[p.rank] + p.off_lse_out)[row] = lse_out;
      continue;
    }
#pragma unroll
    for (int r = 0; r < kPeerMaxRanks; ++r) {
      if (r < p.world) {
        unsigned char* dst = p.buf[r] + p.off_out + row * (kPeerDv * 2) + lane * 16;
        *reinterpret_cast<uint4*>(dst) = oa;
        *reinterpret_cast<uint4*>(dst + 512) = ob;
      }
    }
    if (lane < p.world) reinterpret_cast<float*>(p.buf[lane] + p.off_lse_out)[row] = lse_out;
  }

  // ---- 3. all slices written everywhere.  One system-scope fence per block, after the block barrier
  //         (the barrier orders the other threads' peer stores before it).  Draining the peer stores is
  //         the longest phase of the kernel (about 19 of 43 us at two ranks, cycle counters).
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    s_last = (atomicAdd(p.state + 1, 1) == static_cast<int>(gridDim.x) - 1);
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    if (!p.no_sync && !p.local_only && tid < p.world) {
      st_release_sys(reinterpret_cast<uint32_t*>(p.buf[tid] + p.off_flags) + kPeerDoneSlot + p.rank, step);
      if (!wait_step(my_flags + kPeerDoneSlot + tid, step, p.wait_cycles)) atomicMax(p.status, kDevWaitTimeout);
    }
    __syncthreads();
    if (tid == 0) {
      p.state[1] = 0;
      p.state[0] = static_cast<int32_t>(step);
    }
  }
}

// Node-wide barrier as a kernel of its own: flag word slot*8 + r of a buffer is written by rank r.
__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerCombineParams p, int slot) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int tid = threadIdx.x;
  const uint32_t step = static_cast<uint32_t>(*reinterpret_cast<volatile int32_t*>(p.state)) + 1u;
  __syncwarp();
  if (tid < p.world) {
    st_release_sys(reinterpret_cast<uint32_t*>(p.buf[tid] + p.off_flags) + slot * 8 + p.rank, step);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.buf[p.rank] + p.off_flags) + slot * 8 + tid;
    if (!wait_step(mine, step, p.wait_cycles)) atomicMax(p.status, kDevWaitTimeout);
  }
  __syncwarp();
  if (tid == 0) p.state[0] = static_cast<int32_t>(step);
}

// Barrier + all-gather in one kernel: after the flag exchange every block copies its share of every
// rank's `nbytes` at `off_src` into the local buffer dst[r * nbytes ...] with 16-byte loads, eight in
// flight per thread (element-wise peer loads of a consumer kernel would pay NVLink latency per element).
// state: [0] launches completed, [1] blocks finished in this launch.
__global__ void __launch_bounds__(256, 2) peer_gather_kernel(const PeerCombineParams p, int slot, int64_t off_src,
                                                          int64_t nbytes, unsigned char* __restrict__ dst) {
  pdl_launch_dependents();
  pdl_wait_prior();
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const uint32_t step = static_cast<uint32_t>(*reinterpret_cast<volatile int32_t*>(p.state)) + 1u;
  if (blockIdx.x == 0 && tid < p.world)
    st_release_sys(reinterpret_cast<uint32_t*>(p.buf[tid] + p.off_flags) + slot * 8 + p.rank, step);
  if (tid < p.world) {
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.buf[p.rank] + p.off_flags) + slot * 8 + tid;
    if (!wait_step(mine, step, p.wait_cycles)) atomicMax(p.status, kDevWaitTimeout);
  }
  __syncthreads();
  const int64_t n16 = nbytes >> 4;                       // 16-byte words per rank
  const int64_t total = n16 * p.world;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + tid; i < total; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int64_t j = i + u * stride;
      if (j < total) {
        const int r = static_cast<int>(j / n16);
        v[u] = ld_sys_v4(p.buf[r] + off_src + ((j - r * n16) << 4));
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int64_t j = i + u * stride;
      if (j < total) reinterpret_cast<uint4*>(dst)[j] = v[u];
    }
  }
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(p.state + 1, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (s_last && tid == 0) {
    p.state[1] = 0;
    p.state[0] = static_cast<int32_t>(step);
  }
}

__device__ __forceinline__ uint4 ld_plain_v4(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// Block-wide "everything this grid stored so far is visible system-wide, and I am the last block":
// one system fence per block after the block barrier (the barrier orders the other threads' stores
// before it), then a ticket.  Returns true in every thread of the last block.
__device__ __forceinline__ bool grid_ticket(int32_t* counter, int* s_last) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    *s_last = (atomicAdd(counter, 1) == static_cast<int>(gridDim.x) - 1);
  }
  __syncthreads();
  const bool last = *s_last != 0;
  if (last) {
    if (threadIdx.x == 0) *counter = 0;
    __threadfence();
  }
  return last;
}

// All-gather by posted stores: every rank copies `nbytes` at off_src of its own buffer into slot
// `rank` of the area at off_dst of EVERY rank's buffer, fences, and tells the peers; the last block
// leaves only when every peer's data has landed here, so the kernel after it reads local memory.
// One NVLink crossing per byte and per flag, no round trip.  state: [0] launches completed, [1] ticket.
__global__ void __launch_bounds__(256, 2) peer_push_kernel(const PeerCombineParams p, int slot, int64_t off_src,
                                                           int64_t nbytes, int64_t off_dst) {
  pdl_launch_dependents();
  pdl_wait_prior();
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const uint32_t step = static_cast<uint32_t>(*reinterpret_cast<volatile int32_t*>(p.state)) + 1u;
  const int64_t n16 = nbytes >> 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
  const unsigned char* src = p.buf[p.rank] + off_src;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + tid; i < n16; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * stride < n16) v[u] = ld_plain_v4(src + ((i + u * stride) << 4));
#pragma unroll
    for (int r = 0; r < kPeerMaxRanks; ++r) {
      if (r < p.world) {
        unsigned char* dst = p.buf[r] + off_dst + p.rank * nbytes;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i + u * stride < n16) *reinterpret_cast<uint4*>(dst + ((i + u * stride) << 4)) = v[u];
      }
    }
  }
  const bool last = grid_ticket(p.state + 1, &s_last);
  if (last) {
    if (tid < p.world) {
      st_release_sys(reinterpret_cast<uint32_t*>(p.buf[tid] + p.off_flags) + slot * 8 + p.rank, step);
      const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.buf[p.rank] + p.off_flags) + slot * 8 + tid;
      if (!wait_step(mine, step, p.wait_cycles)) atomicMax(p.status, kDevWaitTimeout);
    }
    __syncthreads();
    if (tid == 0) p.state[0] = static_cast<int32_t>(step);
  }
}

void set_last_error(const char* msg);

}  // namespace b200dsa

using namespace b200dsa;

extern "C" int b200dsa_peer_lse_combine(void* const* bufs, int32_t rank, int32_t world, int64_t n_rows,
                                        int64_t off_ctx, int64_t off_lse, int64_t off_out, int64_t off_lse_out,
                                        int64_t off_flags, int32_t* state, int32_t no_sync, int32_t pre_signalled,
                                        int32_t local_only, int32_t* status, void* stream) {
  if (!bufs || !state || !status || world < 1 || world > kPeerMaxRanks || rank < 0 || rank >= world || n_rows < 0 ||
      ((off_ctx | off_lse | off_out | off_lse_out | off_flags) & 15) || off_ctx < 0 || off_lse < 0 || off_out < 0 ||
      off_lse_out < 0 || off_flags < 0) {
    set_last_error("b200dsa_peer_lse_combine: bad argument (1 <= world <= 8, offsets 16-byte aligned)");
    return B200DSA_EINVAL;
  }
  PeerCombineParams p{};
  for (int r = 0; r < world; ++r) {
    if (!bufs[r] || (reinterpret_cast<uintptr_t>(bufs[r]) & 15)) {
      set_last_error("b200dsa_peer_lse_combine: every rank's buffer must be mapped and 16-byte aligned");
      return B200DSA_EALIGN;
    }
    p.buf[r] = static_cast<unsigned char*>(bufs[r]);
  }
  p.rank = rank;
  p.world = world;
  p.n_rows = n_rows;
  p.off_ctx = off_ctx;
  p.off_lse = off_lse;
  p.off_out = off_out;
  p.off_lse_out = off_lse_out;
  p.off_flags = off_flags;
  p.state = state;
  p.status = status;
  p.wait_cycles = g_peer_wait_cycles;
  p.no_sync = no_sync;
  p.pre_signalled = pre_signalled;
  p.local_only = local_only;
  const int64_t per = (n_rows + world - 1) / world;
  int64_t grid = (per + 7) / 8;
  if (grid < 1) grid = 1;
  if (grid > 296) grid = 296;          // every block must be resident (2 per SM): all of them wait for peers
  cudaError_t e = launch_chained(peer_lse_combine_kernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0,
                                 static_cast<cudaStream_t>(stream), p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_peer_barrier(void* const* bufs, int32_t rank, int32_t world, int64_t off_flags, int32_t slot,
                                    int32_t* state, int32_t* status, void* stream) {
  if (!bufs || !state || !status || world < 1 || world > kPeerMaxRanks || rank < 0 || rank >= world ||
      off_flags < 0 || (off_flags & 15) || slot < 0 || slot > 7 || slot == 0 || slot == 2) {
    set_last_error("b200dsa_peer_barrier: bad argument (1 <= world <= 8, slot 1 or 3..7)");
    return B200DSA_EINVAL;
  }
  PeerCombineParams p{};
  for (int r = 0; r < world; ++r) {
    if (!bufs[r]) {
      set_last_error("b200dsa_peer_barrier: every rank's buffer must be mapped");
      return B200DSA_EINVAL;
    }
    p.buf[r] = static_cast<unsigned char*>(bufs[r]);
  }
  p.rank = rank;
  p.world = world;
  p.off_flags = off_flags;
  p.state = state;
  p.status = status;
  p.wait_cycles = g_peer_wait_cycles;
  cudaError_t e = launch_chained(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), p,
                                 static_cast<int>(slot));
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_peer_gather(void* const* bufs, int32_t rank, int32_t world, int64_t off_src, int64_t nbytes,
                                   void* dst, int64_t off_flags, int32_t slot, int32_t* state, int32_t* status,
                                   void* stream) {
  if (!bufs || !dst || !state || !status || world < 1 || world > kPeerMaxRanks || rank < 0 || rank >= world ||
      off_src < 0 || nbytes <= 0 || ((off_src | nbytes | off_flags) & 15) || off_flags < 0 ||
      (reinterpret_cast<uintptr_t>(dst) & 15) || slot < 0 || slot > 7 || slot == 0 || slot == 2) {
    set_last_error("b200dsa_peer_gather: bad argument (1 <= world <= 8, slot 1 or 3..7, 16-byte aligned sizes)");
    return B200DSA_EINVAL;
  }
  PeerCombineParams p{};
  for (int r = 0; r < world; ++r) {
    if (!bufs[r] || (reinterpret_cast<uintptr_t>(bufs[r]) & 15)) {
      set_last_error("b200dsa_peer_gather: every rank's buffer must be mapped and 16-byte aligned");
      return B200DSA_EALIGN;
    }
    p.buf[r] = static_cast<unsigned char*>(bufs[r]);
  }
  p.rank = rank;
  p.world = world;
  p.off_flags = off_flags;
  p.state = state;
  p.status = status;
  p.wait_cycles = g_peer_wait_cycles;
  int64_t grid = (nbytes / 16 * world + 2047) / 2048;
  if (grid < 1) grid = 1;
  if (grid > 296) grid = 296;          // two blocks per SM: the whole 8-rank payload is in flight at once
  cudaError_t e = launch_chained(peer_gather_kernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0,
                                 static_cast<cudaStream_t>(stream), p, static_cast<int>(slot), off_src, nbytes,
                                 static_cast<unsigned char*>(dst));
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_peer_push(void* const* bufs, int32_t rank, int32_t world, int64_t off_src, int64_t nbytes,
                                 int64_t off_dst, int64_t off_flags, int32_t slot, int32_t* state, int32_t* status,
                                 void* stream) {
  if (!bufs || !state || !status || world < 1 || world > kPeerMaxRanks || rank < 0 || rank >= world ||
      off_src < 0 || off_dst < 0 || nbytes <= 0 || ((off_src | off_dst | nbytes | off_flags) & 15) || off_flags < 0 ||
      slot < 0 || slot > 7 || slot == 0 || slot == 2) {
    set_last_error("b200dsa_peer_push: bad argument (1 <= world <= 8, slot 1 or 3..7, 16-byte aligned sizes)");
    return B200DSA_EINVAL;
  }
  PeerCombineParams p{};
  for (int r = 0; r < world; ++r) {
    if (!bufs[r] || (reinterpret_cast<uintptr_t>(bufs[r]) & 15)) {
      set_last_error("b200dsa_peer_push: every rank's buffer must be mapped and 16-byte aligned");
      return B200DSA_EALIGN;
    }
    p.buf[r] = static_cast<unsigned char*>(bufs[r]);
  }
  p.rank = rank;
  p.world = world;
  p.off_flags = off_flags;
  p.state = state;
  p.status = status;
  p.wait_cycles = g_peer_wait_cycles;
  int64_t grid = (nbytes / 16 + 1023) / 1024;
  if (grid < 1) grid = 1;
  if (grid > 296) grid = 296;
  cudaError_t e = launch_chained(peer_push_kernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0,
                                 static_cast<cudaStream_t>(stream), p, static_cast<int>(slot), off_src, nbytes, off_dst);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_peer_set_wait_limit(int64_t cycles) {
  if (cycles < 0) {
    set_last_error("b200dsa_peer_set_wait_limit: the limit must be positive, or 0 for the default");
    return B200DSA_EINVAL;
  }
  g_peer_wait_cycles = cycles == 0 ? kPeerWaitCyclesDefault : static_cast<long long>(cycles);
  return B200DSA_OK;
}

// ---------------------------------------------------------------------------------------------
// Exchange buffers: plain device allocations that other processes of the node map through CUDA IPC.
// ---------------------------------------------------------------------------------------------
extern "C" int b200dsa_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle64) {
  if (bytes <= 0 || !ptr || !handle64) {
    set_last_error("b200dsa_peer_alloc: bad argument");
    return B200DSA_EINVAL;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* d = nullptr;
  cudaError_t e = cudaMalloc(&d, static_cast<size_t>(bytes));
  if (e == cudaSuccess) e = cudaMemset(d, 0, static_cast<size_t>(bytes));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    if (d) cudaFree(d);
    return B200DSA_ECUDA;
  }
  memcpy(handle64, &h, 64);
  *ptr = d;
  return B200DSA_OK;
}

extern "C" int b200dsa_peer_open(const unsigned char* handle64, void** ptr) {
  if (!handle64 || !ptr) {
    set_last_error("b200dsa_peer_open: bad argument");
    return B200DSA_EINVAL;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* d = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  *ptr = d;
  return B200DSA_OK;
}

extern "C" int b200dsa_peer_close(void* ptr) {
  if (!ptr) return B200DSA_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}

extern "C" int b200dsa_peer_free(void* ptr) {
  if (!ptr) return B200DSA_OK;
  const cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return B200DSA_ECUDA;
  }
  return B200DSA_OK;
}
