// Pieces shared by the sparse MLA attention kernels: parameters, tensor-memory stores, the MMA form that
// reads its A operand from tensor memory, shared-memory descriptors for the P and V operands.
#pragma once

#include <cuda_bf16.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

constexpr int kMlaHeadsTile = 64;    // heads per CTA (UMMA M)
constexpr int kMlaMaxHeads = 128;
constexpr int kMlaD = 576;          // latent width (512 value dims + 64 rope dims)
constexpr int kMlaDv = 512;
constexpr int kMlaChunks = 9;       // 576 / 64 elements (128-byte chunks)
constexpr int kMlaThreads = 288;
// keys per tile and gather pipeline depth: smaller tiles allow more row gathers in flight
constexpr int kMlaTile = 64;
constexpr int kMlaStages = 3;
constexpr int kMlaStageBytes = kMlaTile * kMlaD * 2;
constexpr int kMlaChunkBytesK = kMlaTile * 128;
constexpr int kMlaPBytes = kMlaHeadsTile * kMlaTile * 2;
constexpr int kMlaSmemBytes = kMlaStages * kMlaStageBytes + kMlaPBytes + 1024 + 256;
static_assert(kMlaTile == 32 || kMlaTile == 64, "tile must be 32 or 64 keys");
// Q staging: the last 72 KB of the key ring, rows padded to 1168 bytes (the tail reaches into the P tile)
constexpr int kMlaQRowBytes = kMlaD * 2 + 16;
constexpr int kMlaQStageOff = kMlaStages * kMlaStageBytes - kMlaHeadsTile * kMlaD * 2;
static_assert(kMlaQStageOff >= 0 && kMlaQStageOff % 16 == 0, "Q staging must lie inside the ring");
static_assert(kMlaQStageOff + kMlaHeadsTile * kMlaQRowBytes <= kMlaStages * kMlaStageBytes + kMlaPBytes, "Q staging overruns the P tile");
constexpr uint32_t kMlaTmemCols = 512;
constexpr uint32_t kMlaTmemO = 0;                 // lanes 0-15 of every sub-partition, columns 0..511
constexpr uint32_t kMlaTmemS = (16u << 16);       // lanes 16-31 of every sub-partition, columns 0..127
constexpr uint32_t kMlaTmemQ = (16u << 16) + 128; // Q as the A operand: upper half-lanes, columns 128..415
                                                  // (64 rows x 576 bf16, two per 32-bit cell)

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct MlaParams {
  const __nv_bfloat16* q;      // [n_items, n_heads, 576]
  const __nv_bfloat16* kv;     // [kv_rows, 576]
  int64_t kv_rows;
  const int64_t* kv_row_base;  // nullable [n_items]: row of position 0 of the item's sequence
  const int32_t* indices;      // [n_items, idx_stride] key positions, -1 = none
  int64_t idx_stride;
  int32_t n_idx;
  const int32_t* n_idx_item;   // nullable [n_items]: only the first n_idx_item[i] indices of item i are looked at
  const int32_t* q_pos;        // nullable [n_items]: keys beyond q_pos[item] + q_pos_bias are masked
  int q_pos_bias;
  int32_t pos_lo, pos_hi;      // only positions in [pos_lo, pos_hi) are attended (shard ownership)
  int32_t n_items, n_heads;
  float scale_log2;            // sm_scale * log2(e)
  void* ctx;                   // [n_items, n_heads, 512] fp32, or bf16 when ctx_bf16 != 0
  int ctx_bf16;
  float* lse;                  // [n_items, n_heads] fp32 (natural log)
  int32_t* status;
  // key-sharded decode: when every CTA has written (and fenced) its part of ctx / lse, the last one
  // raises this rank's flag word on every rank: "my partial of step state[0] + 1 is ready".  The
  // kernel that merges the partials (b200dsa_peer_lse_combine with pre_signalled) owns and advances
  // the step counter; this kernel only reads it.
  int signal_on;
  PeerLinkDev link;
  int32_t* ticket;             // local int32, zero between launches
};


// Key-sharded decode: after its last store every CTA takes a ticket; the last one raises this rank's flag
// word on every rank (see MlaParams::signal_on).  Called by all threads of the CTA.
__device__ __forceinline__ void mla_signal_peers(const MlaParams& p) {
  if (!p.signal_on) return;
  __shared__ int s_last_cta;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last_cta = (atomicAdd(p.ticket, 1) == static_cast<int>(gridDim.x) - 1);
  }
  __syncthreads();
  if (s_last_cta) {
    __threadfence();
    const uint32_t step = static_cast<uint32_t>(*reinterpret_cast<volatile int32_t*>(p.link.state)) + 1u;
    if (threadIdx.x < p.link.world) st_release_sys(link_flag(p.link, threadIdx.x, p.link.rank), step);
    if (threadIdx.x == 0) *p.ticket = 0;
  }
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (same lanes as D).
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {   // 2^x, ex2.approx: 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// K-major operand without swizzle: core matrices of 8 rows x 16 bytes stored contiguously
// (128 bytes); lbo = byte step between core matrices along K, sbo = along M/N.
__device__ __forceinline__ uint64_t make_desc_k_noswz(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// MN-major operand, 128-byte swizzle: atoms of 8 K-rows x 64 MN-elements (1024 bytes);
// lbo = byte step between atoms along MN, sbo = byte step between atoms along K.
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}


// Cluster-of-two form (sparse_mla_pair.cu): all heads of an item as UMMA M = 128, the latent dims split
// between the two CTAs.  Returns a cudaError_t as int.
int mla_pair_launch(const MlaParams& p, cudaStream_t stream);

}  // namespace b200dsa
