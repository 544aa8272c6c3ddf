/* b200dsa — C ABI of the B200 (sm_100a) sparse-attention selection kernels.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream (as void*),
 * launches asynchronously on that stream, allocates nothing and never synchronises.
 * Return value: 0 on success, a negative B200DSA_E* code when the arguments are rejected
 * (nothing is launched in that case).  Kernels that contain bounded waits or index checks
 * report through a caller-owned int32 `status` word in device memory (0 = ok,
 * 1 = a wait gave up, 2 = an out-of-range index was skipped, 3 = a fused selection without logits
 * could not prove a candidate list complete); the caller zeroes it once
 * and may read it whenever convenient.
 *
 * "Reference" citations name files of the TransArch repository whose behaviour the entry
 * point reproduces (path relative to its root).
 */
#ifndef B200DSA_H_
#define B200DSA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200DSA_OK 0
#define B200DSA_EINVAL (-1)      /* bad size / null pointer / unsupported combination */
#define B200DSA_EALIGN (-2)      /* pointer or stride not aligned as documented */
#define B200DSA_ECUDA (-3)       /* a CUDA runtime / driver call failed (see b200dsa_last_error) */
#define B200DSA_EUNSUPPORTED (-4)

/* Library / device introspection. */
int b200dsa_abi_version(void);
const char* b200dsa_last_error(void);

/* The GPUs of one node as the kernels of the key-sharded step see them: the exchange buffer of every
 * rank (b200dsa_peer_alloc / b200dsa_peer_open), a flag slot inside it, and this rank's step counter.
 *   bufs      HOST array of `world` device pointers as seen from the calling process
 *   off_flags byte offset of the 256 bytes of flags in every buffer (zero before the first call)
 *   slot      1 or 3..7 (0 and 2 belong to b200dsa_peer_lse_combine); one slot per kind of exchange
 *   state     two int32 of LOCAL device memory, zero before the first call: the step counter of this
 *             slot's user (kernels advance it themselves, so captured launches can be replayed)
 * Flags are step numbers that only grow; every wait is bounded (b200dsa_peer_set_wait_limit). */
typedef struct b200dsa_peer_link {
  void* const* bufs;
  int32_t rank, world;
  int64_t off_flags;
  int32_t slot;
  int32_t* state;
} b200dsa_peer_link;

/* Tensor-pipe peak probe (measurement aid, not on the serving path): `ctas` CTAs each issue
 * iters * 8 tcgen05 MMAs of shape M=128, N=256, K=32 bytes on shared-memory operands, FP8 e4m3
 * (fp8 != 0) or bf16, with no global-memory traffic.  Flops per launch = ctas * iters * 8 *
 * 2*128*256*K with K = 32 (FP8) or 16 (bf16); time it with events to obtain the tensor-pipe
 * roofline denominator of this GPU under its own clocks and power cap.  No counterpart in the
 * reference. */
int b200dsa_mma_peak_probe(int32_t fp8, int32_t ctas, int32_t iters, int32_t* status, void* stream);
/* The same loop for one bf16 instruction shape: m = 64 or 128, n = 32, 64, 128 or 256, the A operand from
 * shared memory (a_from_tmem = 0) or from tensor memory.  One launch issues ctas * iters * 4 MMAs of
 * 2*m*n*16 flops; clocks_out (optional, int64 [ctas]) receives each CTA's SM clock count from its first
 * issue to the retirement of its last MMA, so clocks per instruction do not depend on the clock rate.
 * Used to decide tile shapes (which shapes run at the full rate of the pipe). */
int b200dsa_mma_shape_probe(int32_t m, int32_t n, int32_t a_from_tmem, int32_t ctas, int32_t iters,
                            int64_t* clocks_out, int32_t* status, void* stream);
/* HBM read probe: `ctas` CTAs (two per SM is what the decode indexer runs) pull the chunks
 * base + offsets[i] (chunk_bytes each, a multiple of 16; chunks_per_stage of them, 1 to 4, share a ring slot
 * of at most 16896 bytes) into a five-stage shared-memory ring with bulk copies and drop them.  Timed by the
 * caller: the rate at which that list of chunks can be read at all, e.g. the pages of a paged cache in
 * block-table order. */
int b200dsa_hbm_read_probe(const void* base, const int64_t* offsets, int32_t n_chunks, int32_t chunk_bytes,
                           int32_t chunks_per_stage, int32_t ctas, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Row-wise top-k selection over fp32 scores.
 *
 * Replaces the torch.topk + "-1 where not finite" step of
 *   OpenDSA/opendsa/ops/topk_select.py:66-71
 * and the torch.topk + gather + mask sequences of
 *   MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/indexers.py:499-518, :566-568.
 *
 * Row r looks at columns [col_begin[r], col_end[r]) (defaults 0 and n_cols; clamped to
 * [0, n_cols]).  -inf and NaN are never selected; +inf only when keep_pos_inf != 0.  The k
 * largest remaining scores are chosen; equal scores are resolved towards the lowest
 * output position, so the selected SET is deterministic.  With sorted != 0 a row is written
 * in descending score order (ties: ascending position), as torch.topk(sorted=True) would;
 * with sorted == 0 the winners come in no particular order (torch.topk(sorted=False), which
 * the reference uses at misa_ops.py:402,710).  Rows are padded with -1 (values: -inf).
 *
 * Output position of column c in row r:
 *   pos_map   != NULL : pos_map[r*pos_map_stride + c]
 *   page_table!= NULL : page_table[r*page_table_stride + c/page_size]*page_size + c%page_size
 *   otherwise         : c
 * plus row_pos_offset[r] when that pointer is given.
 *
 * Segmented rows (seg_cols > 0): column c of a row is stored at offset
 * (c / seg_cols) * seg_stride + c % seg_cols from the row start, in scores and in pos_map
 * alike.  This reads the [n_ranks, n_rows, seg] layout an all-gather of per-shard candidates
 * produces without a transpose (row_stride = distance between rows inside one segment).
 * seg_offsets (optional HOST array, one entry per segment, at most 8): segment r starts
 * seg_offsets[r] elements from `scores` (and from `pos_map`) instead of r * seg_stride.  The
 * segments may then be separate buffers, for example the candidate buffers of peer GPUs mapped
 * into this process, read in place over NVLink (after b200dsa_peer_barrier).
 *
 * Limits: 1 <= k <= 8192.  scores rows need 4-byte alignment only.
 * ------------------------------------------------------------------------------------- */
int b200dsa_topk_select(const float* scores, int64_t row_stride, int32_t n_rows, int32_t n_cols,
                        const int32_t* col_begin, const int32_t* col_end, int32_t k,
                        int32_t keep_pos_inf, int32_t sorted,
                        const int32_t* pos_map, int64_t pos_map_stride,
                        const int32_t* page_table, int64_t page_table_stride, int32_t page_size,
                        const int32_t* row_pos_offset,
                        int32_t seg_cols, int64_t seg_stride, const int64_t* seg_offsets,
                        int32_t* out_idx, float* out_val, int64_t out_stride,
                        void* stream);

/* Same selection for few, long rows (decode: tens of rows of 10^5 scores), spread over the
 * whole GPU: `splits` CTAs per row collect the candidates of their slice into global scratch,
 * then one CTA per row finishes the exact selection.  Identity positions (+ row_pos_offset)
 * only.  Scratch: scratch_cand = n_rows*8192 uint64 (8-byte aligned), scratch_count = 2*n_rows
 * int32 whose first n_rows entries must be ZERO before the first call; the library leaves them
 * zero again after every call.  Calls that share scratch must not overlap on the GPU.  Results equal
 * b200dsa_topk_select's (same set; same order when sorted != 0). */
int b200dsa_topk_select_split(const float* scores, int64_t row_stride, int32_t n_rows, int32_t n_cols,
                              const int32_t* col_begin, const int32_t* col_end, int32_t k,
                              int32_t keep_pos_inf, int32_t sorted, const int32_t* row_pos_offset,
                              int32_t splits, void* scratch_cand, int32_t* scratch_count,
                              int32_t* out_idx, float* out_val, int64_t out_stride, void* stream);

/* b200dsa_topk_select_split for hosts that cannot provide scratch memory.  It has no counterpart
 * in the reference.  Some callers have no way to allocate on the device when they call us: an
 * inference server that gave almost the whole GPU to its own pool at start-up leaves no room
 * for a plug-in's cudaMalloc, and a bare C host may own neither workspace nor allocator.  Here
 * the candidate lists and counters sit in a 4 MiB array built into the library (present on every
 * GPU that loads it, until the process ends), so the call allocates nothing.
 *   - at most 64 rows; more is rejected with B200DSA_EINVAL and a message naming the limit;
 *   - the first call on a device looks up the array's device address; make that first call
 *     outside of any stream capture;
 *   - the array is shared by all calls on a device and keeps the previous call's contents (the
 *     counters are cleared at the start of each call, on `stream`); two calls that overlap on
 *     the GPU, from whatever streams or threads, corrupt each other;
 *   - same arguments and results as b200dsa_topk_select_split otherwise. */
int b200dsa_topk_select_split_static(const float* scores, int64_t row_stride, int32_t n_rows, int32_t n_cols,
                                     const int32_t* col_begin, const int32_t* col_end, int32_t k,
                                     int32_t keep_pos_inf, int32_t sorted, const int32_t* row_pos_offset,
                                     int32_t splits, int32_t* out_idx, float* out_val, int64_t out_stride,
                                     void* stream);

/* ---------------------------------------------------------------------------------------
 * Decode indexer logits over the paged FP8 key cache (tcgen05 FP8 contraction).
 *
 *   logits[r, c] = out_scale * k_scale[c] * sum_h weights[r,h] * relu(<q[r,h,:], k_fp8[c,:]>)
 *   for c < context_lens[r]; -inf for context_lens[r] <= c < roundup(context_lens[r], 128)
 *   (clipped to max_cols); columns beyond that are left untouched.
 *
 * Replaces MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:56-199
 * (paged_mqa_sparse_head_return_logits + interface) and the whole-cache dequantisation at
 * :360-378; same role as the DeepGEMM fp8_paged_mqa_logits call at
 * MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/indexers.py:182-191.
 *
 *   q_fp8        [n_rows, 64, 128] e4m3 (row r = request r/next_n, draft token r%next_n)
 *   weights      [n_rows, 64] fp32, with q scale, softmax scale and head scale folded in
 *                (MISA_preprint/.../misa_deepseek_v2.py:289-292)
 *   cache        [num_pages, page_size*(128+4)] bytes: page_size*128 e4m3 then page_size fp32
 *                scales (layout read at misa_ops.py:360-372); page_size in {32, 64, 128}
 *   context_lens [n_rows] int32, keys visible to row r
 *   block_table  [n_rows/next_n, block_table_stride] int32 page ids
 *   row_table    optional int32 [n_rows]: block-table row of each logits row (prefill chunks,
 *                where a request contributes a varying number of query rows); when given it
 *                replaces the row/next_n rule
 * Page ids outside [0, num_pages) are skipped and reported through status (2).
 * q, weights and cache must be 16-byte aligned.
 * head_mask / logits_gated (both or neither): when given, logits_gated[r, c] (same stride as
 * logits) receives the same sum restricted to the heads whose bit is set in head_mask[r]
 * (bit h = head h).  This is MISA's routed stage-1 score (zero weight on the dropped heads,
 * misa_ops.py:703-705) produced in the same pass over the cache as the all-head score that the
 * reference computes in a second pass (misa_ops.py:396-411).
 * ------------------------------------------------------------------------------------- */
int b200dsa_indexer_paged_fp8_logits(const void* q_fp8, const float* weights, const void* cache,
                                     int32_t num_pages, int32_t page_size, const int32_t* context_lens,
                                     const int32_t* block_table, int64_t block_table_stride,
                                     const int32_t* row_table, int32_t n_rows, int32_t next_n,
                                     int32_t max_cols, float out_scale,
                                     float* logits, int64_t logits_stride, const uint64_t* head_mask,
                                     float* logits_gated, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Token logits inside per-row lists of 128-key blocks of the PAGED FP8 cache (HISA stage 2 / block-sparse
 * re-scoring while serving): column c of row r is key position block_list[r, c/128]*128 + c%128 of the row's
 * request, found through the block table;
 *   logits[r, c] = out_scale * k_scale * sum_h weights[r,h]*relu(<q[r,h,:], k_fp8[pos,:]>)
 * when c < row_cols[r], block id >= 0 and pos < context_lens[r]; -inf otherwise (for c < row_cols[r] rounded
 * up to 128; columns beyond are left untouched).
 * Replaces MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/block_ops.py:151-379
 * (paged_block_sparse_mqa_attn_return_logits + interface), reading the FP8 pages in place instead of a
 * bf16 copy of the cache.  q / weights / cache / context_lens / block_table / row_table / next_n as for
 * b200dsa_indexer_paged_fp8_logits; row_cols [n_rows] = 128 * (listed blocks of the row).
 * ------------------------------------------------------------------------------------- */
int b200dsa_indexer_paged_blocklist_fp8_logits(const void* q_fp8, const float* weights, const void* cache,
                                               int32_t num_pages, int32_t page_size, const int32_t* context_lens,
                                               const int32_t* block_table, int64_t block_table_stride,
                                               const int32_t* row_table, int32_t n_rows, int32_t next_n,
                                               const int32_t* block_list, int64_t block_list_stride,
                                               const int32_t* row_cols, int32_t max_cols, float out_scale,
                                               float* logits, int64_t logits_stride, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fused decode selection: the same scores as b200dsa_indexer_paged_fp8_logits and, from them, the
 * top-k key positions of every row, in two launches and without a pass over the logits.  The
 * indexer's epilogue appends every score at or above a floor (taken from the first tiles each CTA
 * scores of a row) to the row's candidate list; the second kernel selects exactly from the list.
 * A list that cannot be proven complete (fewer than k entries at or above the largest floor used
 * for the row, or more than 16384 entries) is not trusted: the row is then selected from `logits`.
 * Replaces, in one call, MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:182
 * (+ :393-401, the logits matrix) and the torch.topk at indexers.py:566-568.
 *
 *   arguments up to out_scale: as b200dsa_indexer_paged_fp8_logits (no head mask)
 *   logits / logits_stride    [n_rows, >= max_cols] fp32, written as a by-product and read only by the
 *                             fallback.  May be NULL: nothing but the candidate lists is then written,
 *                             and a row whose list is not provably complete (about 1e-7 per row for
 *                             scores without long runs of ties) is selected from the list anyway with
 *                             *status raised to 3.
 *   k <= 2048, sorted, row_pos_offset, out_idx / out_val / out_stride: as b200dsa_topk_select_split;
 *                             results equal b200dsa_topk_select's on the same logits
 *   scratch_cand              n_rows * 16384 uint64 (8-byte aligned)
 *   scratch_count             2 * n_rows int32, ZERO before the first call; left zero by every call
 * Calls that share scratch must not overlap on the GPU.
 * ------------------------------------------------------------------------------------- */
int b200dsa_indexer_paged_fp8_topk(const void* q_fp8, const float* weights, const void* cache,
                                   int32_t num_pages, int32_t page_size, const int32_t* context_lens,
                                   const int32_t* block_table, int64_t block_table_stride,
                                   const int32_t* row_table, int32_t n_rows, int32_t next_n,
                                   int32_t max_cols, float out_scale, float* logits, int64_t logits_stride,
                                   int32_t k, int32_t sorted, const int32_t* row_pos_offset,
                                   void* scratch_cand, int32_t* scratch_count, int32_t* out_idx,
                                   float* out_val, int64_t out_stride, int32_t* status, void* stream);

/* b200dsa_indexer_paged_fp8_topk whose selection kernel also delivers the result to the peers (first
 * exchange of the key-sharded step, no kernel of its own): row r's k positions and k score bit patterns
 * are stored, as [2k] int32, at off_recv + (link->rank * n_rows + r) * 8k bytes of EVERY rank's buffer
 * (posted NVLink stores from the selection's write loop); the last CTA fences and raises this rank's
 * flag word (link->slot) on every rank and advances link->state[0].  It does not wait:
 * b200dsa_topk_merge_owned does.  No counterpart in the reference (single GPU). */
int b200dsa_indexer_paged_fp8_topk_push(const void* q_fp8, const float* weights, const void* cache,
                                        int32_t num_pages, int32_t page_size, const int32_t* context_lens,
                                        const int32_t* block_table, int64_t block_table_stride,
                                        const int32_t* row_table, int32_t n_rows, int32_t next_n,
                                        int32_t max_cols, float out_scale, float* logits, int64_t logits_stride,
                                        int32_t k, int32_t sorted, const int32_t* row_pos_offset,
                                        void* scratch_cand, int32_t* scratch_count, int32_t* out_idx,
                                        float* out_val, int64_t out_stride, const b200dsa_peer_link* link,
                                        int64_t off_recv, int32_t* status, void* stream);

/* Merge of the pushed per-rank selections: waits (bounded) until every rank's flag of link->slot reached
 * link->state[0] (the step this rank's own push recorded), then selects the global top-k of every row from
 * the world * k candidates in the LOCAL receive area recv = [world, n_rows, 2k] int32 (positions then
 * score bit patterns), exactly as b200dsa_topk_select would on the concatenated lists (ties to the lowest
 * position, so every rank gets the same result), and also writes the winners inside [own_lo, own_hi),
 * compacted and -1 padded, to owned [n_rows, owned_stride] with their number in owned_count[n_rows]:
 * the keys this rank attends.  Replaces all-gather + top-k + ownership compaction. */
int b200dsa_topk_merge_owned(const int32_t* recv, int32_t world, int32_t n_rows, int32_t k, int32_t sorted,
                             int32_t own_lo, int32_t own_hi, int32_t* out_idx, int64_t out_stride,
                             int32_t* owned, int64_t owned_stride, int32_t* owned_count,
                             const b200dsa_peer_link* link, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Token logits inside per-row lists of 128-key blocks, bf16 keys (tcgen05 bf16 contraction).
 * HISA stage 2 / block-sparse re-scoring.
 *
 *   column c of row r is key position block_list[r, c/128]*128 + c%128;
 *   logits[r, c] = out_scale * sum_h weights[r,h]*relu(<q[r,h,:], keys[pos,:]>) when
 *   c < row_cols[r] and pos_lo[r] <= pos < pos_hi[r] (bounds optional), else -inf.
 *
 * Replaces MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/block_ops.py:756-937
 * (block_sparse_mqa_attn_return_logits and its interface).
 *   q_bf16 [n_rows, 64, 128], keys_bf16 [n_keys, 128] (both 16-byte aligned),
 *   row_cols [n_rows] = 128 * (number of listed blocks), block ids in [0, ceil(n_keys/128)).
 * head_mask / logits_gated: as for b200dsa_indexer_paged_fp8_logits.
 * block_list may be NULL when pos_lo / pos_hi are given: row r then covers the consecutive
 * blocks pos_lo[r]/128, pos_lo[r]/128 + 1, ... (flat causal prefill needs no list).
 * ------------------------------------------------------------------------------------- */
int b200dsa_indexer_blocklist_bf16_logits(const void* q_bf16, const float* weights, const void* keys_bf16,
                                          int32_t n_keys, const int32_t* block_list,
                                          int64_t block_list_stride, const int32_t* row_cols,
                                          const int32_t* pos_lo, const int32_t* pos_hi, int32_t n_rows,
                                          int32_t max_cols, float out_scale, float* logits,
                                          int64_t logits_stride, const uint64_t* head_mask,
                                          float* logits_gated, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Token logits of every query on its OWN list of key positions (MISA stage 2 in prefill: all 64 heads on the
 * stage-1 candidates, MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:517-650, T2):
 *   logits[r, c] = out_scale * sum_h weights[r,h]*relu(<q[r,h,:], keys[cand[r,c],:]>) for c < row_cols[r];
 *   -inf where cand[r,c] is negative, not below n_keys or outside [pos_lo[r], pos_hi[r]) (intervals optional).
 * A tile's 128 key rows are gathered by 16-byte asynchronous copies into the tensor core's swizzled layout;
 * one N = 64 pass per (query, 128 candidates).  q_bf16 [n_rows, 64, 128], keys_bf16 [n_keys, 128],
 * cand int32 [n_rows, cand_stride], weights fp32 [n_rows, 64].
 * ------------------------------------------------------------------------------------- */
int b200dsa_indexer_gather_bf16_logits(const void* q_bf16, const float* weights, const void* keys_bf16,
                                       int32_t n_keys, const int32_t* cand, int64_t cand_stride,
                                       const int32_t* row_cols, const int32_t* pos_lo, const int32_t* pos_hi,
                                       int32_t n_rows, int32_t max_cols, float out_scale, float* logits,
                                       int64_t logits_stride, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Prefill token logits over flat bf16 keys with per-query intervals (tcgen05, four queries per key tile):
 *   column c of row r is key position col0[r] + c, col0[r] = 128 * (pos_lo[r] / 128);
 *   logits[r, c] = out_scale * sum_h weights[r,h]*relu(<q[r,h,:], keys[pos,:]>) for pos_lo[r] <= pos <
 *   pos_hi[r], -inf for the other columns c < row_cols[r]; columns beyond row_cols[r] are left untouched.
 * Replaces the score + mask steps of OpenDSA/opendsa/ops/topk_select.py:57-65 and
 * MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:415-515 (T1) without the fp32
 * [chunk, 64, Lk] intermediate.  Consecutive queries share each key tile (N = 256 per MMA), so keys are
 * fetched once per four queries.
 *   q_bf16 [n_rows, 64, 128], keys_bf16 [n_keys, 128] (16-byte aligned), weights [n_rows, 64] fp32,
 *   row_cols [n_rows] = 128 * ceil(pos_hi/128) - col0 (a multiple of 128).
 * ------------------------------------------------------------------------------------- */
/* The routed form (MISA stage 1 in prefill, misa_ops.py:415-515 with its block_Q = 128 / H query tiling):
 * q8_bf16 [n_rows, 8, 128] holds the 8 heads the router kept for each query, weights8 [n_rows, 8] their
 * weights; 32 queries share each key tile (N = 256 = 32 x 8), so the contraction costs an eighth of the
 * all-head form. */
int b200dsa_indexer_flat_bf16_logits_routed(const void* q8_bf16, const float* weights8, const void* keys_bf16,
                                            int32_t n_keys, const int32_t* pos_lo, const int32_t* pos_hi,
                                            const int32_t* row_cols, int32_t n_rows, int32_t max_cols,
                                            float out_scale, float* logits, int64_t logits_stride,
                                            int32_t* status, void* stream);
int b200dsa_indexer_flat_bf16_logits(const void* q_bf16, const float* weights, const void* keys_bf16,
                                     int32_t n_keys, const int32_t* pos_lo, const int32_t* pos_hi,
                                     const int32_t* row_cols, int32_t n_rows, int32_t max_cols,
                                     float out_scale, float* logits, int64_t logits_stride,
                                     int32_t* status, void* stream);

/* Causal intervals of packed queries, one launch: for row t at position p = q_pos[t] (t when q_pos is NULL),
 * lo[t] = start of the last document of cu_seqlens [n_cu] that begins at or before p, hi[t] = p + 1
 * (OpenDSA/opendsa/ops/flashkl_warmup.py:41-56 prepare_ks_ke, :235-248 prepare_ks_ke_cp), and the column frame the
 * flat logits kernels and the selection use: col0[t] = lo rounded down to a multiple of 128, row_cols[t] = the
 * multiple of 128 that covers [col0, hi).  All arrays int32 [n_rows]. */
int b200dsa_causal_row_intervals(const int32_t* cu_seqlens, int32_t n_cu, const int32_t* q_pos, int32_t n_rows,
                                 int32_t* lo, int32_t* hi, int32_t* col0, int32_t* row_cols, void* stream);

/* ---------------------------------------------------------------------------------------
 * Sparse MLA attention over selected keys in the absorbed latent space (tcgen05), one query
 * token per item; emits the latent-space context and the log-sum-exp so that partial results
 * over disjoint key sets can be merged.
 *
 *   valid(j) = idx_j >= 0 and idx_j <= q_pos[item] + q_pos_bias and pos_lo <= idx_j < pos_hi
 *              (q_pos_bias = -1 lets a caller pass context lengths as q_pos)
 *   s[h,j]   = sm_scale * <q[item,h,:], kv[kv_row_base[item] + idx_j - pos_lo, :]>
 *   ctx[item,h,:] = sum_j softmax_j(s)[h,j] * kv[row_j, 0:512]     (0 when no key is valid)
 *   lse[item,h]   = log sum_j exp(s[h,j])                           (-inf when no key is valid)
 *
 * Reproduces OpenDSA/opendsa/ops/sparse_mla.py:39-43 with the validity rule of :90, i.e.
 * _attend_absorbed_chunk before its W_UV up-projection (:44).
 *   q_bf16 [n_items, n_heads, 576], kv_bf16 [kv_rows, 576] (512 value dims then 64 rope dims),
 *   indices [n_items, idx_stride] int32, kv_row_base / q_pos optional (0 / no bound),
 *   ctx [n_items, n_heads, 512] fp32, or bf16 (the dtype the reference returns, sparse_mla.py:44-47)
 *   when ctx_bf16 != 0; lse [n_items, n_heads] fp32.  1 <= n_heads <= 128.
 * n_idx_item (optional int32 [n_items]) limits item i to its first n_idx_item[i] indices
 * (compacted shard lists).  Rows outside [0, kv_rows) are skipped and reported through status (2).
 * ------------------------------------------------------------------------------------- */
int b200dsa_sparse_mla_decode(const void* q_bf16, const void* kv_bf16, int64_t kv_rows,
                              const int64_t* kv_row_base, const int32_t* indices, int64_t idx_stride,
                              int32_t n_idx, const int32_t* n_idx_item, const int32_t* q_pos,
                              int32_t q_pos_bias, int32_t pos_lo, int32_t pos_hi,
                              int32_t n_items, int32_t n_heads, float sm_scale, void* ctx, int32_t ctx_bf16,
                              float* lse, int32_t* status, void* stream);

/* Same arguments and results as b200dsa_sparse_mla_decode, computed by the cluster-of-two kernel: the two
 * CTAs of an item split the latent dimensions instead of the heads, so that all 128 heads form one UMMA
 * M = 128 tile (full tensor rate) and every selected row is fetched once; partial scores and probabilities
 * cross the cluster through shared memory (bulk copies to one CTA, no multicast).  Measured slower than the
 * default kernel on B200 (86 against 63 us at 64 items x 128 heads x 2048 keys: the exchange is bound by
 * the bandwidth between the two CTAs' shared memories), so nothing in the library selects it by itself. */
int b200dsa_sparse_mla_decode_pair(const void* q_bf16, const void* kv_bf16, int64_t kv_rows,
                                   const int64_t* kv_row_base, const int32_t* indices, int64_t idx_stride,
                                   int32_t n_idx, const int32_t* n_idx_item, const int32_t* q_pos,
                                   int32_t q_pos_bias, int32_t pos_lo, int32_t pos_hi,
                                   int32_t n_items, int32_t n_heads, float sm_scale, void* ctx, int32_t ctx_bf16,
                                   float* lse, int32_t* status, void* stream);

/* b200dsa_sparse_mla_decode for a rank of the key-sharded step: after the last CTA has written (and
 * fenced) its part of ctx / lse, which the caller placed in this rank's exchange buffer, the kernel raises
 * this rank's "partial ready" flag on every rank, so that b200dsa_peer_lse_combine(pre_signalled = 1)
 * starts with the wait alone.  link: the combine's buffers and ITS state word (slot 0; read, not advanced);
 * ticket: one int32 of local device memory, zero before the first call. */
int b200dsa_sparse_mla_decode_signal(const void* q_bf16, const void* kv_bf16, int64_t kv_rows,
                                     const int64_t* kv_row_base, const int32_t* indices, int64_t idx_stride,
                                     int32_t n_idx, const int32_t* n_idx_item, const int32_t* q_pos,
                                     int32_t q_pos_bias, int32_t pos_lo, int32_t pos_hi, int32_t n_items,
                                     int32_t n_heads, float sm_scale, void* ctx, int32_t ctx_bf16, float* lse,
                                     const b200dsa_peer_link* link, int32_t* ticket, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Value up-projection of the latent-space context, the step right after the attention kernel:
 *   out[t, h, v] = sum_l ctx[t, h, l] * W_UV[h, v, l]        (a tcgen05 GEMM per head, K = 512)
 * Replaces the einsum at OpenDSA/opendsa/ops/sparse_mla.py:44 ("thl,hvl->thv").
 *   ctx_bf16 [n_tokens, n_heads, 512] bf16 (what b200dsa_sparse_mla_decode writes with ctx_bf16 = 1),
 *   w_uv_bf16 [n_heads, dv, 512] bf16, 1 <= dv <= 256, out [n_tokens, n_heads, dv] bf16 or fp32.
 * ------------------------------------------------------------------------------------- */
int b200dsa_wuv_up_project(const void* ctx_bf16, const void* w_uv_bf16, int32_t n_tokens, int32_t n_heads,
                           int32_t dv, void* out, int32_t out_f32, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Merge attention partials computed over disjoint key sets (key shards of several GPUs, or
 * splits on one GPU):  out = sum_r exp(lse_r - m) ctx_r / sum_r exp(lse_r - m),
 * lse_out = m + log(sum_r exp(lse_r - m)),  m = max_r lse_r.  No counterpart call in the
 * reference (its inference path is single-GPU); the nearest analogue is the context-parallel
 * key gather at OpenDSA/opendsa/modeling/dsa_attention.py:650-669.
 *   ctx_parts [n_parts, n_rows, 512] fp32, lse_parts [n_parts, n_rows] fp32,
 *   ctx_out [n_rows, 512] fp32, lse_out [n_rows] fp32 (optional).  n_parts <= 64.
 * ------------------------------------------------------------------------------------- */
int b200dsa_lse_combine(const float* ctx_parts, const float* lse_parts, int32_t n_parts, int64_t n_rows,
                        float* ctx_out, float* lse_out, void* stream);

/* ---------------------------------------------------------------------------------------
 * The same merge across the GPUs of one node in ONE kernel over NVLink peer memory (replaces
 * the all-gather of lse + all-reduce of the scaled partials).  No counterpart in the reference
 * (its context-parallel path gathers keys instead, OpenDSA/opendsa/modeling/dsa_attention.py:650-669).
 *
 * Every rank owns an exchange buffer of identical layout, mapped into every rank's address space
 * (b200dsa_peer_alloc / b200dsa_peer_open); bufs is a HOST array of the `world` device pointers
 * as seen from the calling process (bufs[rank] = its own buffer).  Byte offsets inside a buffer:
 *   off_ctx      bf16 [n_rows, 512]  this rank's normalised partial (written before the call)
 *   off_lse      fp32 [n_rows]       its log-sum-exp (-inf for an empty partial)
 *   off_out      bf16 [n_rows, 512]  merged result, complete on every rank when the kernel ends
 *   off_lse_out  fp32 [n_rows]
 *   off_flags    256 bytes of flags, zero before the first call and never touched by the host
 * state: two int32 of LOCAL device memory, zero before the first call (the step counter lives
 * there, so a captured launch can be replayed).  All ranks must make the same sequence of calls.
 * Waits for peers are bounded (about a second): on expiry *status gets 1 and the call
 * completes with an unusable result instead of hanging.  no_sync != 0 skips the flag exchange:
 * ranks emulated one after another on a single GPU (tests); ranks that wait for each other
 * must run on different GPUs.  pre_signalled != 0: the kernel that wrote the partial
 * (b200dsa_sparse_mla_decode_signal) has already raised this rank's "ready" flags, so the call
 * only waits for the peers'.  local_only != 0 is the reduce-scatter form: the rank merges its
 * slice of the rows (rows [rank*ceil(n_rows/world), ...)) into its OWN result area and neither stores
 * to the peers nor waits for them a second time; the other rows of its result area are not written
 * (a tensor-parallel output projection consumes exactly such a slice).  1 <= world <= 8.
 * ------------------------------------------------------------------------------------- */
int b200dsa_peer_lse_combine(void* const* bufs, int32_t rank, int32_t world, int64_t n_rows,
                             int64_t off_ctx, int64_t off_lse, int64_t off_out, int64_t off_lse_out,
                             int64_t off_flags, int32_t* state, int32_t no_sync, int32_t pre_signalled,
                             int32_t local_only, int32_t* status, void* stream);

/* Node-wide barrier on the stream: one small kernel writes this rank's step number into every
 * peer's flag word `slot*8 + rank` (uint32 words at off_flags; slots 0 and 2 belong to
 * b200dsa_peer_lse_combine, use 1 or 3..7) and waits, bounded, until all peers' words reached the same
 * step.  state: one int32 of local device memory per slot user, zero before the first call.  What
 * the peers wrote to their own buffers before their barrier call is readable afterwards. */
int b200dsa_peer_barrier(void* const* bufs, int32_t rank, int32_t world, int64_t off_flags, int32_t slot,
                         int32_t* state, int32_t* status, void* stream);

/* The same barrier followed, in the same kernel, by an all-gather: nbytes at off_src of every
 * rank's buffer are copied into dst[r * nbytes ...] of LOCAL memory (16-byte peer loads, coalesced).
 * state: two int32 of local device memory, zero before the first call.  Sizes and offsets are
 * multiples of 16.  Replaces the NCCL all-gather of the per-shard top-k candidates. */
int b200dsa_peer_gather(void* const* bufs, int32_t rank, int32_t world, int64_t off_src, int64_t nbytes,
                        void* dst, int64_t off_flags, int32_t slot, int32_t* state, int32_t* status,
                        void* stream);

/* All-gather by posted stores: nbytes at off_src of THIS rank's buffer are stored into slot `rank`
 * (off_dst + rank * nbytes) of EVERY rank's buffer; the call's kernel ends when all peers' slots
 * have landed in this rank's buffer.  One NVLink crossing per byte, no load round trip.  state: two
 * int32 of local device memory, zero before the first call. */
int b200dsa_peer_push(void* const* bufs, int32_t rank, int32_t world, int64_t off_src, int64_t nbytes,
                      int64_t off_dst, int64_t off_flags, int32_t slot, int32_t* state, int32_t* status,
                      void* stream);

/* Bound of every wait for a peer's flag in the four peer kernels above, in SM clock cycles (default
 * 2^31, about a second; 0 restores the default).  Process-wide; takes effect for launches made after
 * the call.  A serving loop that prefers a quick error over a second-long stall when a peer is gone
 * lowers it; when a wait runs out the kernel sets *status to 1, still advances its step counter and
 * ends, so the stream and the context stay usable and the host can decide what to do. */
int b200dsa_peer_set_wait_limit(int64_t cycles);

/* Exchange buffers.  peer_alloc: zeroed device allocation on the current device plus the 64-byte
 * CUDA IPC handle another process passes to peer_open (with ITS device current) to map it;
 * peer_close unmaps, peer_free releases the allocation in the owning process. */
int b200dsa_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle64);
int b200dsa_peer_open(const unsigned char* handle64, void** ptr);
int b200dsa_peer_close(void* ptr);
int b200dsa_peer_free(void* ptr);

/* Shard ownership compaction: per row, the positions inside [pos_lo, pos_hi) are moved to the
 * front of out (relative order kept), the rest of the row is -1, count[row] = how many.  Lets a
 * rank attend only the selected keys it owns.  out must not alias indices. */
int b200dsa_compact_owned(const int32_t* indices, int64_t idx_stride, int32_t n_rows, int32_t n_idx,
                          int32_t pos_lo, int32_t pos_hi, int32_t* out, int64_t out_stride,
                          int32_t* count, void* stream);

/* All-reduce form of the merge above, for partials that live on different GPUs.  After a MAX
 * all-reduce of lse gives lse_max, prescale writes 516-float wire rows
 * (ctx*exp(lse-lse_max) [512], exp(lse-lse_max), 3 zero pads); the caller SUM-all-reduces
 * (or reduce-scatters) the wire buffer; finalize divides by the summed weight and writes
 * lse_out = lse_max + log(weight sum).  wire is [n_rows, 516] fp32, 16-byte aligned. */
int b200dsa_lse_prescale(const float* ctx, const float* lse, const float* lse_max, int64_t n_rows,
                         float* wire, void* stream);
int b200dsa_lse_finalize(const float* wire, const float* lse_max, int64_t n_rows, float* ctx_out,
                         float* lse_out, void* stream);

/* Compact form for bf16 results: lse_all [n_parts, n_rows] holds every rank's lse (all-gathered,
 * 4 bytes per row and rank); the rank writes out = bf16(ctx * exp(lse_me - m) / sum_r exp(lse_r - m))
 * and lse_out = m + log(sum); one SUM all-reduce of the bf16 [n_rows, 512] rows then gives the
 * merged context on every rank (half the bytes of the fp32 wire, no finalize pass). */
int b200dsa_lse_prescale_norm(const float* ctx, const float* lse_all, int32_t n_parts, int32_t my_part,
                              int64_t n_rows, void* out_bf16, float* lse_out, void* stream);

/* ---------------------------------------------------------------------------------------
 * FP8 quantisation of the index queries with the scale folded into the head weights:
 *   scale = max(amax|q[t,h,:]|, 1e-10)/448, q_fp8 = e4m3(q/scale), weights = w * scale * fold.
 * use_ue8m0 != 0 rounds the scale UP to a power of two first, scale = 2^ceil(log2(scale)): the
 * "ue8m0" scale format the reference always asks for (scale_fmt is "ue8m0" at
 * misa_deepseek_v2.py:177, passed as use_ue8m0=self.scale_fmt is not None at :280-285).
 * Replaces MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_deepseek_v2.py:279-292
 * (per_token_group_quant_fp8 over the 128-wide head + weight folding; fold carries
 * softmax_scale * n_head**-0.5 there).
 *   q_bf16 [n_rows, 128] (n_rows = tokens*heads), w [n_rows] fp32,
 *   q_fp8 [n_rows, 128] e4m3 out, weights [n_rows] fp32 out.
 * ------------------------------------------------------------------------------------- */
int b200dsa_quant_q_fold_weights(const void* q_bf16, const float* w, int64_t n_rows, float fold,
                                 int32_t use_ue8m0, void* q_fp8, float* weights, void* stream);

/* ---------------------------------------------------------------------------------------
 * Elementwise tails of the indexer's projections, fused (the three dense projections themselves are
 * plain GEMMs and stay with the BLAS library):
 *
 * keys:    k = RoPE(LayerNorm(wk(h))): LayerNorm over the 128 dims (weight, bias, eps), rotate-half
 *          RoPE on 64 rope dims with per-token cos / sin [n_tokens, 64] fp32.  rope_first = 0: the rope
 *          dims are the last 64 (OpenDSA/opendsa/modeling/indexer.py:70-79); 1: the first 64
 *          (MISA_preprint/.../misa_deepseek_v2.py:232-250).  k_out (optional) receives the rows in the
 *          input's dtype; with a cache the rows are also quantised (as b200dsa_indexer_k_quant_and_cache
 *          would quantise their bf16 rounding) and stored at slot_mapping[t]: the cache insert fused with
 *          norm + RoPE, no bf16 row round trip (the step before the selection path,
 *          indexers.py:454-460).  ln_w / cos may be NULL to skip that stage.
 * queries: RoPE on every (token, head) row of wq(q_in) [n_tokens, n_heads, 128]; q_out (optional) receives
 *          the rows; with q_fp8 the rows are also quantised per (token, head) and weights[t,h] =
 *          w[t,h] * scale * fold (misa_deepseek_v2.py:279-292 fused with the RoPE before it).
 * in_f32: inputs (and row outputs) are fp32 instead of bf16.
 * ------------------------------------------------------------------------------------- */
int b200dsa_indexer_k_norm_rope(const void* k_proj, int32_t in_f32, int64_t n_tokens, const float* ln_w,
                                const float* ln_b, float ln_eps, const float* cos, const float* sin,
                                int32_t rope_first, void* k_out, const int64_t* slot_mapping, void* cache,
                                int64_t num_pages, int32_t page_size, int32_t use_ue8m0, int32_t* status,
                                void* stream);
int b200dsa_indexer_q_rope(const void* q_proj, int32_t in_f32, int64_t n_tokens, int32_t n_heads,
                           const float* cos, const float* sin, int32_t rope_first, void* q_out,
                           const float* w, float fold, int32_t use_ue8m0, void* q_fp8, float* weights,
                           void* stream);

/* ---------------------------------------------------------------------------------------
 * Backward of the sparse MLA attention (the training form of sparse_attend_absorbed_chunked,
 * OpenDSA/opendsa/ops/sparse_mla.py:26-48 under autograd): the two memory-bound steps around the dense
 * products, per chunk of queries.
 *   pointwise: p = exp(scale*s - lse) on valid entries (index >= 0 and <= q_pos), else 0;
 *              ds = p * (dp - delta) * scale.   s, dp, p, ds: [n_queries, n_heads, n_idx] bf16 or fp32
 *              (is_bf16), lse / delta fp32 [n_queries, n_heads], indices int32 [n_queries, n_idx] (a multiple
 *              of 8 columns), q_pos int32 [n_queries].
 *   scatter:   d_latent[indices[t,j], :] += rows_qk[t,j,0:576] + rows_v[t,j,0:512] (rows_v may be NULL) for
 *              valid entries; d_latent fp32 [n_latent_rows, 576], accumulated with 16-byte vector reductions.
 * ------------------------------------------------------------------------------------- */
int b200dsa_sparse_attn_bwd_pointwise(const void* s, const void* dp, int32_t is_bf16, const float* lse,
                                      const float* delta, const int32_t* indices, const int32_t* q_pos,
                                      int32_t n_queries, int32_t n_heads, int32_t n_idx, float scale,
                                      void* p_out, void* ds_out, void* stream);
int b200dsa_scatter_add_latent_rows(float* d_latent, int64_t n_latent_rows, const void* rows_qk,
                                    const void* rows_v, int32_t is_bf16, const int32_t* indices,
                                    const int32_t* q_pos, int32_t n_queries, int32_t n_idx, int32_t* status,
                                    void* stream);

/* ---------------------------------------------------------------------------------------
 * Block mean pooling of index keys: pooled[j] = mean(keys[j*block : min((j+1)*block, n)]),
 * fp32 accumulation, the tail block divided by its true length.
 * Replaces MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/block_ops.py:685-754
 * (block_mean_pooling + interface; output cast back to bf16 as at :752) and, for the paged
 * FP8 cache, :381-486 (paged_mean_pooling: fp32 [n_requests, max_pool_blocks, 128], blocks
 * beyond a request's context are zero).  Either output pointer of the bf16 variant may be NULL.
 * ------------------------------------------------------------------------------------- */
int b200dsa_block_mean_pool_bf16(const void* keys_bf16, int32_t n_keys, int32_t block, void* out_bf16,
                                 float* out_f32, void* stream);
int b200dsa_paged_mean_pool_fp8(const void* cache, int32_t num_pages, int32_t page_size,
                                const int32_t* context_lens, const int32_t* block_table,
                                int64_t block_table_stride, int32_t n_requests, int32_t block,
                                int32_t max_pool_blocks, float* out, int32_t* status, void* stream);
/* Pooled-key maintenance for decode: the same means, kept up to date instead of pooled again every step
 * (the reference pools the whole cache on every call, misa_ops.py:381).  sums and out are persistent
 * fp32 [n_requests, max_pool_blocks, 128]; request b went from prev_lens[b] to context_lens[b] keys since
 * the last call and only those keys are read.  prev_lens[b] = 0 rebuilds request b from the cache and
 * clears the blocks beyond its context (a slot taken over by a new request).  The running sums add in
 * position order, as the full kernel does: out is bit-identical to b200dsa_paged_mean_pool_fp8 on the
 * same cache.  ctas_per_request CTAs share the blocks of one request (1-2 for decode steps, more when
 * requests are rebuilt). */
int b200dsa_paged_mean_pool_fp8_update(const void* cache, int32_t num_pages, int32_t page_size,
                                       const int32_t* prev_lens, const int32_t* context_lens,
                                       const int32_t* block_table, int64_t block_table_stride,
                                       int32_t n_requests, int32_t block, int32_t max_pool_blocks,
                                       int32_t ctas_per_request, float* sums, float* out, int32_t* status,
                                       void* stream);

/* ---------------------------------------------------------------------------------------
 * MISA head routers.  Each writes head_idx [n_tokens, n_keep] int32 (descending router score,
 * ties to the lowest head) and weights_out [n_tokens, 64] fp32 that is zero on dropped heads,
 * so the 64-head indexer entry points apply the gating through their weight operand.
 *
 *  qnorm      : largest ||q[t,h,:]||_2; kept heads keep w[t,h].  Reference:
 *               MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_deepseek_v2.py:254-266
 *               with the weight gather of misa_ops.py:703-705.
 *  block_score: largest sum over pooled key blocks j in [blk_lo[t], blk_hi[t]) of
 *               |w[t,h]*relu(<q[t,h,:], pooled[set(t), j, :]>)|; kept heads keep w[t,h].
 *               Reference: block_ops.py:488-573 (prefill) and :11-98 (decode), consumed at
 *               misa_ops.py:694-705 and :380-388.  pooled_keys is fp32 [n_sets, pooled_set_stride/128, 128];
 *               pooled_set (optional) maps a token to its set (decode: the request).
 *  linear     : logits = x[t,:] @ W_r (bf16 inputs, fp32 accumulate), top-n heads, weights =
 *               softmax over the kept logits.  No counterpart in the reference: a learned
 *               router reading the token's hidden state (hidden = 7168, n = 8 of 64 heads in the
 *               DeepSeek-V3.2 shape) instead of the query norms; logits_out optional; out_scale
 *               (optional fp32 [n_tokens, 64]) multiplies the weights written, e.g. the folded
 *               per-head scales of the FP8 queries.
 * ------------------------------------------------------------------------------------- */
int b200dsa_router_qnorm_topk(const void* q_bf16, const float* w, int32_t n_tokens, int32_t n_keep,
                              float* weights_out, int32_t* head_idx, void* stream);
int b200dsa_router_block_score_topk(const void* q_bf16, const float* w, const float* pooled_keys,
                                    int64_t pooled_set_stride, const int32_t* pooled_set,
                                    const int32_t* blk_lo, const int32_t* blk_hi, int32_t n_tokens,
                                    int32_t n_keep, float* weights_out, int32_t* head_idx,
                                    float* scores_out, void* stream);
int b200dsa_router_linear_topk_softmax(const void* x_bf16, const void* w_r_bf16, int32_t n_tokens,
                                       int32_t hidden, int32_t n_keep, const float* out_scale,
                                       float* weights_out, int32_t* head_idx, float* logits_out,
                                       void* stream);

/* ---------------------------------------------------------------------------------------
 * Insert new index keys into the paged FP8 cache: per-token e4m3 quantisation
 * (scale = max(amax,1e-4)/448, rounded up to a power of two when use_ue8m0 != 0, which is what
 * the reference's scale_fmt = "ue8m0" selects) written to slot_mapping[t] = page*page_size +
 * offset (negative = skip).  Stands in for the third-party vLLM op the reference calls at
 * MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/indexers.py:454-460
 * (ops.indexer_k_quant_and_cache), producing the page layout read at misa_ops.py:360-372.
 *   k_bf16 [n_tokens, 128], slot_mapping int64 [n_tokens], cache [num_pages, page_size*132].
 * ------------------------------------------------------------------------------------- */
int b200dsa_indexer_k_quant_and_cache(const void* k_bf16, const int64_t* slot_mapping, int64_t n_tokens,
                                      void* cache, int64_t num_pages, int32_t page_size, int32_t use_ue8m0,
                                      int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200DSA_H_ */
