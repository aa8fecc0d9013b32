/*
 * liblocks_b200 -- C ABI of the B200 (sm_100a) LOCKS decode hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, and
 * returns 0 on success or a negative LOCKS_ERR_* code (message available from
 * locks_last_error()).  Unless stated otherwise an entry point only enqueues
 * work on `stream`: it never allocates, never synchronises and never throws,
 * so every call is legal inside CUDA-graph capture.  The caller owns every
 * buffer.  Strides are in ELEMENTS of the pointed-to type.
 *
 * Each declaration names the reference interface it replaces (paths relative to
 * the reference's src/locks/).  The reference binds its kernels with pybind11
 * modules that take torch::Tensor (e.g. selection/rki4_score_cuda.py:2518-2619);
 * the raw-pointer argument lists below carry the same information.
 *
 * Geometry supported by this build: head_dim 128, page 16, summary rank 8,
 * int4 basis, 1 <= G <= 16 query heads per KV head.
 */
#ifndef LOCKS_B200_H_
#define LOCKS_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LOCKS_ABI_VERSION 1

/* One summary record per (physical block, kv-head):
 *   [0,512)   V basis, 8 columns x 64 B, int4 (low nibble = even d row)
 *   [512,640) page centroid mu, int8 x 128
 *   [640,768) coefficients C, int8, 16 tokens x 8
 *   [768,800) per-token C scales, bf16 x 16
 *   [800,816) per-column V scales, bf16 x 8
 *   [816,818) mu scale, bf16          [818,832) zero padding
 * Same fields as the reference's six slabs (selection/rki4_state.py:7-22), laid
 * out as its 832-byte "AoS" record (selection/rki4_state.py:93-102,198-220). */
#define LOCKS_REC_BYTES 832
#define LOCKS_TAG_WIDTH 8

#define LOCKS_OK             0
#define LOCKS_ERR_ARG       (-1)  /* null pointer, negative size, bad stride  */
#define LOCKS_ERR_GEOMETRY  (-2)  /* head_dim/page/G outside the supported set */
#define LOCKS_ERR_LAUNCH    (-3)  /* CUDA reported an error at launch          */
#define LOCKS_ERR_SIZE      (-4)  /* size beyond a stated maximum              */

/* values a kernel may leave in a caller-provided device `status` word */
#define LOCKS_ST_OK            0
#define LOCKS_ST_WAIT_TIMEOUT  1  /* a bounded on-chip wait ran out            */
#define LOCKS_ST_CP_OVERFLOW   2  /* context parallel: more kept pages than     */
                                  /* candidate slots (cap sized too small)      */

#define LOCKS_COMBINE_NONE 0      /* `score` already holds the combined score  */
#define LOCKS_COMBINE_NRM  1      /* sum_g exp(S[g,p] - max_p S[g,p])          */
#define LOCKS_COMBINE_MAX  2      /* max_g S[g,p]                              */

typedef void* locks_stream_t;     /* a cudaStream_t */

/* Programmatic dependent launch between score -> select -> fused decode -> next
 * layer's score (on by default; returns the previous setting).  With it the
 * scorer prefetches summary records while the previous layer's select / decode
 * still run.  The reference chains its kernels the same way with
 * griddepcontrol (selection/select_cuda.py:202-206, attention/decode_cuda.py:
 * 304-315).  Contract: block tables must not be written by the kernel launched
 * immediately before a scorer launch on the same stream. */
int locks_set_pdl(int enable);

int locks_version(void);
const char* locks_last_error(void);
/* Bytes of one summary record (without the tag).  Replaces
 * selection/rki4_state.py:124-141 record_bytes() for the supported geometry;
 * returns LOCKS_ERR_GEOMETRY otherwise. */
int locks_record_bytes(int head_dim, int page);

/* ---- Stage A.0: rki4 summary build ---------------------------------------
 * For every layer in [layer0, layer0+n_layers) and every block id in
 * blocks[0..n_blocks): read the 16 x head_dim bf16 keys of each kv-head, form the
 * centroid, the centred 16x16 Gram, its eigen-decomposition (Jacobi, fp32), the
 * rank-8 factors, quantise and write the record + the content tag.  Block ids
 * outside [0, min(num_blocks_state, num_blocks_cache)) are skipped.
 * k_layers: DEVICE array of n_total_layers pointers to each layer's K plane.
 * records: (n_total_layers, num_blocks_state, n_kv, 832) bytes; tags: same
 * leading dims x 8 bf16.
 * Replaces selection/rki4_build.py:228-261 (_rki4_write: _write_pre, eigh,
 * _write_post) and the (layer, block) pair expansion of selection/build.py:388-396. */
int locks_rki4_build(const void* const* k_layers, int64_t k_stride_block,
                     int64_t k_stride_tok, int64_t k_stride_head,
                     void* records, void* tags, const int32_t* blocks,
                     int n_blocks, int layer0, int n_layers,
                     int num_blocks_state, int num_blocks_cache, int n_kv,
                     int head_dim, int page, locks_stream_t stream);

/* Content-tag staleness scan: stale[i] = 1 when valid[i] != 0 and the stored
 * tag of blocks[i] differs from the live keys in ANY layer (NaN never equals).
 * Replaces selection/build.py:475-488 (_delta_select) up to its final boolean
 * gather, which stays on the host. */
int locks_rki4_tag_scan(const void* const* k_layers, int64_t k_stride_block,
                        int64_t k_stride_tok, int64_t k_stride_head,
                        const void* tags, const int32_t* blocks,
                        const uint8_t* valid, uint8_t* stale, int n_blocks,
                        int n_layers, int num_blocks_state, int n_kv, int page,
                        locks_stream_t stream);

/* ---- Stage A.1: per-step page parameters ---------------------------------
 * n_pages = ceil(seq_len/page); n_sel_hi = n_pages - window;
 * s = n_sel_hi - sink; b = budget_pages > 0 ? max(min(budget_pages, max(s,1)),1)
 *                        : min(max((int)ceil(s*budget),1), max(s,1)) in fp64.
 * Replaces selection/select.py:28-58 (derive_page_params). */
int locks_derive_page_params(const int32_t* seq_lens, int n_req, int page,
                             int window_pages, int sink_pages, int budget_pages,
                             double budget, int32_t* n_pages, int32_t* n_sel_hi,
                             int32_t* b_fix, locks_stream_t stream);

/* The same with one page budget PER REQUEST: budget_pages_req[r] > 0 is request
 * r's budget in pages, <= 0 falls back to the fraction `budget`.  The reference
 * keeps b_fix per request (the selector reads b_fix[r], selection/select.py:
 * 92-105) but derives it from one engine-wide constant (BUDGET_ABS,
 * selection/select.py:29-58); a continuous batch whose requests carry their own
 * budgets passes them here. */
int locks_derive_page_params_req(const int32_t* seq_lens, int n_req, int page,
                                 int window_pages, int sink_pages,
                                 const int32_t* budget_pages_req, double budget,
                                 int32_t* n_pages, int32_t* n_sel_hi,
                                 int32_t* b_fix, locks_stream_t stream);

/* ---- Stage A.2: page score ------------------------------------------------
 * score_h[r,kh,g,p] = logsumexp_t scale*(cs[t]*sum_r C8[t,r]*qt[g,r] + mu.q)
 * for p < n_sel_hi[r], with q round-tripped through per-head int8 and the page
 * summary read at block_table[r,p] (clamped into [0,num_blocks)).
 * q: bf16 (n_req, n_kv*G, head_dim).  score_h: f32 (n_req, n_kv, G, max_pages).
 * hmax: optional (n_req, n_kv, G) uint32 keys, atomically raised to the
 * order-preserving key of each head's maximum score (pass NULL to skip).
 * zsplit <= 0 selects the page split automatically.  status: optional device int.
 * Replaces selection/rki4_score_cuda.py:2518-2619 (rki4_score_bt) /
 * :3263-3448 (rki4_score_only); CPU twin selection/rki4_score_torch.py:111-160. */
int locks_rki4_score_bt(const void* q, int64_t q_stride_req,
                        const void* records_layer, const int32_t* block_table,
                        int64_t bt_stride, const int32_t* n_sel_hi,
                        float* score_h, uint32_t* hmax, int n_req, int n_kv,
                        int G, int head_dim, int page, int max_pages,
                        int bt_width, int num_blocks, float scale, int zsplit,
                        int* status, locks_stream_t stream);

/* ---- Stage A.3: GQA combine + exact top-b ---------------------------------
 * combine: LOCKS_COMBINE_*.  For NRM/MAX the combined score of pages
 * [0, n_sel_hi) is also written to `score` (n_req, n_kv, max_pages).
 * tau = b-th largest score over [sink, n_sel_hi); keep {> tau}, then {== tau}
 * in ascending page order until exactly b are kept, plus [0,sink) and
 * [n_sel_hi, n_pages); keep everything if n_sel_hi - sink <= 1.  page_table
 * (n_req, n_kv, max_pages) gets ascending page ids, -1 padded; page_cnt the count.
 * hmax: optional keys published by locks_rki4_score_bt (read, then reset to 0).
 * Replaces selection/select_cuda.py:492-938 (nrmtopb_select_kernel),
 * :162-449 (topb_select_kernel) and the long-context chain :1786-3249;
 * goldens selection/select.py:65-117 and :123-180. */
int locks_topb_select(int combine, const float* score_h, float* score,
                      uint32_t* hmax, const int32_t* n_pages,
                      const int32_t* n_sel_hi, const int32_t* b_fix,
                      int32_t* page_table, int32_t* page_cnt, int n_req,
                      int n_kv, int G, int max_pages, int sink_pages,
                      locks_stream_t stream);

/* ---- Stage B: sparse paged decode -----------------------------------------
 * Split-K flash decode over the selected pages.  k_cache/v_cache: bf16 planes
 * addressed [block*stride_block + tok*stride_tok + head*stride_head + d].
 * pps = max(ceil(cnt/split), pps_min); split sp covers table entries
 * [sp*pps, min((sp+1)*pps, cnt)); inactive splits store nothing.
 * m_part, l_part: f32 (n_req, n_kv, split, G); acc_part: (.., G, head_dim).
 * Replaces attention/decode.py:209-322 (sparse_decode_split_kernel) and
 * attention/decode_cuda.py:269-547 (locks_decode_split). */
int locks_decode_split(const void* q, int64_t q_stride_req, const void* k_cache,
                       const void* v_cache, int64_t kv_stride_block,
                       int64_t kv_stride_tok, int64_t kv_stride_head,
                       const int32_t* block_table, int64_t bt_stride,
                       const int32_t* page_table, const int32_t* page_cnt,
                       const int32_t* seq_lens, float* m_part, float* l_part,
                       float* acc_part, int n_req, int n_kv, int G,
                       int head_dim, int page, int max_pages, int split,
                       int pps_min, float scale, int* status,
                       locks_stream_t stream);

/* Merge of the active split partials into out (bf16, row stride
 * out_stride_req, heads contiguous); rows without attended pages become 0.
 * Replaces attention/merge.py:105-152 (merge_splits_kernel). */
int locks_merge_splits(const float* m_part, const float* l_part,
                       const float* acc_part, const int32_t* page_cnt,
                       void* out, int64_t out_stride_req, int n_req, int n_kv,
                       int G, int head_dim, int split, int pps_min,
                       locks_stream_t stream);

/* One-launch decode: a CTA per (kv-head, request) walks all selected pages and
 * writes the final bf16 output (no partials, no merge launch).
 * Replaces attention/decode_cuda.py:587-884 (locks_decode_fused). */
int locks_decode_fused(const void* q, int64_t q_stride_req, const void* k_cache,
                       const void* v_cache, int64_t kv_stride_block,
                       int64_t kv_stride_tok, int64_t kv_stride_head,
                       const int32_t* block_table, int64_t bt_stride,
                       const int32_t* page_table, const int32_t* page_cnt,
                       const int32_t* seq_lens, void* out,
                       int64_t out_stride_req, int n_req, int n_kv, int G,
                       int head_dim, int page, int max_pages, float scale,
                       int* status, locks_stream_t stream);

/* Launch order for large ragged batches.  No counterpart in the reference.
 * CTAs start roughly in grid order; with several hundred (request, kv-head)
 * rows of very different lengths over ~150-300 resident CTAs, a long row that
 * happens to start last is the whole tail of the launch.  locks_row_order ranks
 * the requests of the step on the device (one small launch, after the page
 * parameters were derived; n_req <= 4096): order_select[z] = the request with
 * the z-th most pages to select from, order_decode[z] = the request whose
 * decode attends the z-th most pages (ties by index; both permutations of
 * [0, n_req)).  locks_topb_select_rows / locks_decode_fused_rows are
 * locks_topb_select / locks_decode_fused whose grid row z handles request
 * row_order[z]; locks_rki4_score_bt_rows is locks_rki4_score_bt dealing the
 * CTAs of a kv-head to the requests in that order when it shares them by
 * length (several requests); results are identical. */
int locks_row_order(const int32_t* n_pages, const int32_t* n_sel_hi,
                    const int32_t* b_fix, int n_req, int sink_pages,
                    int32_t* order_select, int32_t* order_decode,
                    locks_stream_t stream);
int locks_rki4_score_bt_rows(const void* q, int64_t q_stride_req,
                             const void* records_layer, const int32_t* block_table,
                             int64_t bt_stride, const int32_t* n_sel_hi,
                             float* score_h, uint32_t* hmax, int n_req, int n_kv,
                             int G, int head_dim, int page, int max_pages,
                             int bt_width, int num_blocks, float scale, int zsplit,
                             const int32_t* row_order, int* status,
                             locks_stream_t stream);
int locks_topb_select_rows(int combine, const float* score_h, float* score,
                           uint32_t* hmax, const int32_t* n_pages,
                           const int32_t* n_sel_hi, const int32_t* b_fix,
                           int32_t* page_table, int32_t* page_cnt, int n_req,
                           int n_kv, int G, int max_pages, int sink_pages,
                           const int32_t* row_order, locks_stream_t stream);
int locks_decode_fused_rows(const void* q, int64_t q_stride_req, const void* k_cache,
                            const void* v_cache, int64_t kv_stride_block,
                            int64_t kv_stride_tok, int64_t kv_stride_head,
                            const int32_t* block_table, int64_t bt_stride,
                            const int32_t* page_table, const int32_t* page_cnt,
                            const int32_t* seq_lens, void* out,
                            int64_t out_stride_req, int n_req, int n_kv, int G,
                            int head_dim, int page, int max_pages,
                            const int32_t* row_order, float scale, int* status,
                            locks_stream_t stream);

/* locks_decode_fused with the K/V pages staged by tiled tensor-map copies
 * (cp.async.bulk.tensor.2d into 128-byte-swizzled shared memory, two 16 x 64
 * boxes per plane and page) instead of 16-byte cp.async.  Same arguments plus
 * num_blocks (the planes' block count: the maps' row extent); same results.
 * The planes must be device memory laid out (num_blocks, 16, n_kv, 128) with
 * kv_stride_block a multiple of kv_stride_tok (16 x for separate planes, 32 x
 * for K and V interleaved per block) and kv_stride_head a multiple of 64
 * (LOCKS_ERR_GEOMETRY otherwise: use locks_decode_fused).  The maps cover the
 * launching GPU's memory only; no load is multicast.  No counterpart in the
 * reference (its decode stages pages with cp.async, attention/decode_cuda.py:
 * 269-584). */
int locks_decode_fused_tma(const void* q, int64_t q_stride_req, const void* k_cache,
                           const void* v_cache, int64_t kv_stride_block,
                           int64_t kv_stride_tok, int64_t kv_stride_head,
                           const int32_t* block_table, int64_t bt_stride,
                           const int32_t* page_table, const int32_t* page_cnt,
                           const int32_t* seq_lens, void* out,
                           int64_t out_stride_req, int n_req, int n_kv, int G,
                           int head_dim, int page, int max_pages, int num_blocks,
                           float scale, int* status, locks_stream_t stream);

/* locks_decode_fused with V behind a two-level tier (the decode seam of the
 * reference's DRAM V tier: attention/decode.py:52-100, tier/decode_mem.py:
 * 168-180, pool tier/pool.py:104-184).  K stays in the engine cache.  The V of
 * EVERY physical block lives in v_host, a pinned host pool mapped into the
 * device address space, laid out with the K plane's strides; v_hot is a bounded
 * staging buffer in device memory (slots hot_stride_block elements apart, token
 * and head strides as K's) and v_map[block] the block's slot in it, or -1.  A
 * page whose block has a slot is read from v_hot, any other page in place from
 * v_host over the host link: the same bytes either way, so the output equals
 * locks_decode_fused on a resident V plane bit for bit.
 * Residency notes for the host, written by the same launch: slot_ref[slot] = 1
 * for every slot read; the block of every COMPLETE page that missed is appended
 * to miss_list once per note round (*note_round, a positive device word the
 * host advances whenever it has consumed the list; pending[block], one int32
 * per block, initially 0, remembers the round a block was last listed in;
 * *miss_cnt counts every append, entries beyond miss_cap are dropped and may be
 * listed again).  The host may clear miss_cnt and slot_ref while kernels run: a
 * note lost that way comes back in the next round.  Who fills v_hot and v_map, and when, is the caller's business
 * (locks.attention.vtier: one copy-engine cudaMemcpyAsync per run of contiguous
 * blocks on a side stream between steps); the kernel only requires that a slot
 * named by v_map holds its block's V while the kernel runs. */
int locks_decode_fused_vtier(const void* q, int64_t q_stride_req, const void* k_cache,
                             const void* v_host, int64_t kv_stride_block,
                             int64_t kv_stride_tok, int64_t kv_stride_head,
                             const void* v_hot, int64_t hot_stride_block,
                             const int32_t* v_map, uint8_t* slot_ref,
                             int32_t* pending, int32_t* miss_list, int32_t* miss_cnt,
                             int miss_cap, const int32_t* note_round,
                             const int32_t* block_table,
                             int64_t bt_stride, const int32_t* page_table,
                             const int32_t* page_cnt, const int32_t* seq_lens,
                             void* out, int64_t out_stride_req, int n_req, int n_kv,
                             int G, int head_dim, int page, int max_pages,
                             float scale, int* status, locks_stream_t stream);

/* V tier promotion: n_blocks consecutive blocks of the pinned host pool into
 * n_blocks consecutive slots of the staging buffer as ONE copy-engine transfer
 * (cudaMemcpyAsync, or cudaMemcpy2DAsync with one row per block when a side is
 * pitched) on `stream` -- the reference's CopyEngine.memcpy_async /
 * memcpy_2d_async (tier/dma.py:103-125).  No SM takes part.  src must be pinned
 * for the copy to overlap the kernels of other streams. */
int locks_vtier_copy_run(void* dst, int64_t dst_pitch_bytes, const void* src,
                         int64_t src_pitch_bytes, int64_t block_bytes, int n_blocks,
                         locks_stream_t stream);

/* Merge of split partials gathered from several ranks (context parallel: every
 * rank decodes the selected pages it holds, the partial sets are all-gathered,
 * every rank merges them).  No counterpart in the reference, which is single
 * GPU; the merge formula is attention/merge.py:105-152.
 * packs: n_groups sets, pack_stride floats apart (a multiple of 4); one set is
 * m (n_req, n_kv, split, G) | l (same) | acc (n_req, n_kv, split, G, head_dim),
 * contiguous, i.e. what locks_decode_split wrote through three pointers into
 * one buffer.  EVERY split of every set is read; a split that attended nothing
 * must carry l = 0 (clear l before the decode).  packs 16-byte aligned,
 * n_req*n_kv*split*G even. */
int locks_merge_gathered(const float* packs, int64_t pack_stride, int n_groups,
                         void* out, int64_t out_stride_req, int n_req, int n_kv,
                         int G, int head_dim, int split, locks_stream_t stream);

/* Summary build driven by the step's cache slots: job (layer, token, kv head)
 * builds block slot / page when slot_mapping[token] is the LAST token of its
 * block (the write completed the page) and does nothing otherwise.  Which blocks
 * to refresh is thus decided on the device from the same slot_mapping the KV
 * write used: the launch has a fixed shape and can sit in a CUDA graph (on a
 * forked branch: the page is not scored before it leaves the recent window).
 * Replaces the host-driven tail refresh of selection/rki4_build.py:318-364
 * (rki4_build_tail) / selection/rki4_tailgraph.py. */
int locks_rki4_build_slots(const void* const* k_layers, int64_t k_stride_block,
                           int64_t k_stride_tok, int64_t k_stride_head,
                           void* records, void* tags, const int64_t* slot_mapping,
                           int n_tok, int layer0, int n_layers,
                           int num_blocks_state, int num_blocks_cache, int n_kv,
                           int head_dim, int page, locks_stream_t stream);

/* ---- KV-write neighbour: rotate K, store K/V into the paged cache, build the
 * summary of a page the token completes ------------------------------------------
 * key, val: bf16 (n_tok, n_kv, head_dim), row / head strides in elements.  Row r
 * goes to slot = slot_mapping[r] (block slot / page, token slot % page); slot < 0
 * skips the row.  cos_sin: optional bf16 (P, rot_dim) table, cos half then sin
 * half per position; K channels below rot_dim are rotated at positions[r] in
 * half-split (neox != 0) or interleaved pairing with separately rounded fp32
 * products (no fused multiply-add), the rest of K and all of V are copied.
 * Replaces tier/k5_cuda.py:55-77, 660-687 (rope_and_cache_fixc_kernel).
 * records_layer / tags_layer: optional, this layer's (NB, n_kv, 832) summary
 * records and (NB, n_kv, 8) tags; when the row lands on token page-1 of its block
 * the block's summaries are rebuilt from the cache in the same launch -- the
 * arithmetic of locks_rki4_build (selection/rki4_build.py:45-225), which replaces
 * the separate tail refresh of selection/rki4_tailgraph.py.  A launch of several
 * rows may hold more than one row of the same page (a prefill chunk, speculative
 * tokens): with n_tok > 1 all rows are stored by a first launch and the pages
 * they completed are summarised by a second one behind it, so a summary never
 * reads a row a sibling has yet to store. */
int locks_kv_write(const void* key, int64_t k_row_stride, int64_t k_head_stride,
                   const void* val, int64_t v_row_stride, int64_t v_head_stride,
                   void* k_cache, void* v_cache, int64_t kv_stride_block,
                   int64_t kv_stride_tok, int64_t kv_stride_head,
                   const int64_t* slot_mapping, const int64_t* positions,
                   const void* cos_sin, int64_t cos_sin_row_stride, int rot_dim,
                   int neox, void* records_layer, void* tags_layer, int n_tok,
                   int n_kv, int head_dim, int page, int num_blocks,
                   locks_stream_t stream);

/* ---- Decode-step bookkeeping on the device ------------------------------------
 * For every request row: positions[r] = seq_lens[r] (index of the token this
 * step appends), slot_prev[r] = slot_mapping[r], slot_mapping[r] = block_table[r,
 * tok / page] * page + tok % page (-1 when the table has no such column),
 * seq_lens[r] += 1, then the page parameters of locks_derive_page_params for the
 * new length.  One launch, so a captured decode loop carries no host decision.
 * (The reference gets slot_mapping / positions from the engine's host-side
 * scheduler and derives the page parameters in selection/select.py:51-58.) */
int locks_append_advance(int32_t* seq_lens, const int32_t* block_table,
                         int64_t bt_stride, int bt_width, int n_req, int page,
                         int window_pages, int sink_pages, int budget_pages,
                         double budget, int64_t* slot_mapping, int64_t* slot_prev,
                         int64_t* positions, int32_t* n_pages, int32_t* n_sel_hi,
                         int32_t* b_fix, locks_stream_t stream);

/* locks_append_advance with per-request page budgets (see
 * locks_derive_page_params_req). */
int locks_append_advance_req(int32_t* seq_lens, const int32_t* block_table,
                             int64_t bt_stride, int bt_width, int n_req, int page,
                             int window_pages, int sink_pages,
                             const int32_t* budget_pages_req, double budget,
                             int64_t* slot_mapping, int64_t* slot_prev,
                             int64_t* positions, int32_t* n_pages,
                             int32_t* n_sel_hi, int32_t* b_fix,
                             locks_stream_t stream);

/* ---- Selection that also carries the layer's KV write -------------------------
 * The store of locks_kv_write (same arguments, same arithmetic, no summary
 * build), one token per request row: row r of key / val goes to slot_mapping[r].
 * It rides in the selector's grid -- in a helper CTA of the row's cluster that
 * has nothing left to do while CTA 0 selects -- so the step has no separate
 * KV-write launch; the sparse decode that follows on the stream reads the new
 * token from the cache as usual.  The reference hides the same write behind its
 * select launch (backend/_runtime.py fixc_flush, tier/k5_cuda.py:660-687). */
typedef struct locks_kv_append {
    const void* key;                 /* bf16 (n_req, n_kv, head_dim) */
    int64_t k_row_stride, k_head_stride;
    const void* val;
    int64_t v_row_stride, v_head_stride;
    void* k_cache;
    void* v_cache;
    int64_t kv_stride_block, kv_stride_tok, kv_stride_head;
    const int64_t* slot_mapping;     /* (n_req,), < 0 skips the row */
    const int64_t* positions;        /* (n_req,), needed with cos_sin */
    const void* cos_sin;             /* optional bf16 (P, rot_dim) */
    int64_t cos_sin_row_stride;
    int32_t rot_dim, neox, head_dim, page, num_blocks;
} locks_kv_append_t;

int locks_topb_select_append(int combine, const float* score_h, float* score,
                             uint32_t* hmax, const int32_t* n_pages,
                             const int32_t* n_sel_hi, const int32_t* b_fix,
                             int32_t* page_table, int32_t* page_cnt, int n_req,
                             int n_kv, int G, int max_pages, int sink_pages,
                             const locks_kv_append_t* append,
                             locks_stream_t stream);

/* ---- Context parallel (one sequence over several GPUs) -------------------------
 * No counterpart in the reference (single GPU).  Every rank scores and selects
 * on its own page range with the GLOBAL budget b (locks_rki4_score_bt after an
 * all-reduce(max) of hmax, locks_topb_select); the two calls below sit on either
 * side of the all-gather of the candidates.  Local page j is global page p0 + j;
 * sink_loc / nsh_loc are the sequence's sink count and n_sel_hi in local page
 * numbers, clamped to the range.
 * locks_cp_pack: cand_rows = this rank's (2, n_kv, cap) floats: the combined
 *   score and the global page of the first cap page-table entries that are
 *   selectable pages; forced pages and empty slots travel as -inf.
 * locks_cp_select: cand = the gathered rows, cand_stride floats apart.  Keeps, in
 *   this rank's page table, its forced pages and those of its candidates that are
 *   among the b best of ALL candidates by (score descending, page ascending) --
 *   the exact-b tie rule of selection/select.py:183-222 -- in ascending page
 *   order, -1 padded up to cap; page_cnt = entries kept. */
int locks_cp_pack(const int32_t* page_table, const float* score, float* cand_rows,
                  int n_kv, int max_pages, int cap, int sink_loc, int nsh_loc,
                  int p0, locks_stream_t stream);
int locks_cp_select(const float* cand, int64_t cand_stride, int32_t* page_table,
                    int32_t* page_cnt, int world, int rank, int n_kv, int cap,
                    int max_pages, int b, int sink_loc, int nsh_loc,
                    locks_stream_t stream);

/* Peer exchange for the context-parallel path: all-gather (mode 0) or
 * element-wise unsigned max of uint32 words (mode 1) of a small payload, one
 * kernel per rank over NVLink peer memory.  Every rank allocates one region
 * (locks_cp_region_bytes gives the size; locks_cp_alloc: cudaMalloc, zeroed),
 * exports it (locks_cp_ipc_export: 64-byte CUDA IPC handle) and opens the
 * peers' regions (locks_cp_ipc_open); peers[r] is rank r's region as seen from
 * this process (peers[rank] = the local pointer).  All ranks must issue the same
 * sequence of exchanges on a region, at most 8 ranks.  nbytes, slot_bytes:
 * multiples of 16, nbytes <= slot_bytes.  mode 0: out = (world, nbytes);
 * mode 1: out = nbytes.  Modes 2 and 3 are the same two operations through
 * 8-byte {word, epoch} packets that the receiver polls directly (no fence, no
 * flag: lower latency for payloads of a few KB; 2 * nbytes <= slot_bytes; a
 * region must be used with one of the two transports only).  A rank that does not see all peers within about two
 * seconds sets *status to LOCKS_ST_WAIT_TIMEOUT and returns (out undefined). */
int locks_cp_region_bytes(int slot_bytes, int64_t* out);
int locks_cp_alloc(int64_t bytes, void** out);
int locks_cp_free(void* region);
int locks_cp_ipc_export(void* region, unsigned char* handle64);
int locks_cp_ipc_open(const unsigned char* handle64, void** out);
int locks_cp_ipc_close(void* peer_region);
int locks_cp_exchange(void* const* peers, int world, int rank, const void* payload,
                      int nbytes, int slot_bytes, void* out, int mode, int* status,
                      locks_stream_t stream);

/* ---- Context parallel with the exchanges INSIDE the kernels ----------------------
 * The three per-layer exchanges (per-head score maxima, best-b candidates,
 * attention partials) are done by the selector and the decode kernel
 * themselves: they store their words into every peer's link region and poll
 * their own region for the peers' words, so a layer is three launches (score,
 * select, decode) at any number of GPUs, chained by programmatic dependent
 * launch exactly as on one GPU.  No counterpart in the reference.
 *
 * A link region (one per rank; locks_cp_link_bytes gives its size for a
 * geometry; allocate with locks_cp_alloc, share with locks_cp_ipc_export /
 * _open) starts with the rank's decode-step counter.  Every rank calls
 * locks_cp_begin_step once per decode step, before the first layer: exchange
 * epochs are step * n_layers + layer + 1, equal on all ranks with no
 * communication.  locks_cp_link_reset zeroes a region and sets its step
 * counter: after a wait ran out (LOCKS_ST_WAIT_TIMEOUT) all ranks reset to a
 * common step value, behind a host-side barrier, before the next step.
 *
 * locks_cp_link_t: regions[r] = rank r's region as seen from this process
 * (regions[rank] the local one; with world == 1 the kernels talk to themselves
 * through the local region).  Pages: local page j is global page p0 + j;
 * sink_loc / nsh_loc = the sequence's sink count and n_sel_hi in local page
 * numbers, clamped to the range; b_global = the sequence's page budget; cap =
 * candidate slots per (rank, kv head) >= the entries a rank's local selection
 * can keep (b_global + its forced pages).
 *
 * locks_topb_select_cp: locks_topb_select(LOCKS_COMBINE_NRM) for ONE sequence
 *   (n_req = 1) with hmax = the keys the local scorer published; the maxima are
 *   max-reduced over the ranks before the combine, and after the local selection
 *   (with b_fix = b_global) the candidates of all ranks meet: the page table
 *   keeps this rank's forced pages and those of its candidates that are among
 *   the b_global best of ALL ranks by (score descending, page ascending) -- the
 *   exact-b tie rule of selection/select.py:183-222 -- ascending, -1 padded.
 * locks_decode_fused_cp: locks_decode_fused for ONE sequence; the (m, l, O) of
 *   the pages this rank attended are exchanged and merged with the formula of
 *   attention/merge.py:106-152, every rank writes the full output row.
 * Waits are bounded (about two seconds, then *status = LOCKS_ST_WAIT_TIMEOUT
 * and the kernel returns with an undefined result). */
#define LOCKS_CP_MAX_RANKS 8
typedef struct locks_cp_link_t {
    void* regions[LOCKS_CP_MAX_RANKS];
    int32_t world, rank;
    int32_t layer, n_layers;
    int32_t p0, cap, b_global, sink_loc, nsh_loc;
} locks_cp_link_t;

int locks_cp_link_bytes(int n_kv, int G, int cap, int64_t* out);
int locks_cp_begin_step(void* region, locks_stream_t stream);
int locks_cp_link_reset(void* region, int64_t bytes, uint32_t step,
                        locks_stream_t stream);
int locks_topb_select_cp(const float* score_h, float* score, uint32_t* hmax,
                         const int32_t* n_pages, const int32_t* n_sel_hi,
                         const int32_t* b_fix, int32_t* page_table,
                         int32_t* page_cnt, int n_kv, int G, int max_pages,
                         int sink_pages, const locks_cp_link_t* link, int* status,
                         locks_stream_t stream);
int locks_decode_fused_cp(const void* q, int64_t q_stride_req, const void* k_cache,
                          const void* v_cache, int64_t kv_stride_block,
                          int64_t kv_stride_tok, int64_t kv_stride_head,
                          const int32_t* block_table, int64_t bt_stride,
                          const int32_t* page_table, const int32_t* page_cnt,
                          const int32_t* seq_lens, void* out, int64_t out_stride_req,
                          int n_kv, int G, int head_dim, int page, int max_pages,
                          float scale, const locks_cp_link_t* link, int* status,
                          locks_stream_t stream);

/* Split decode + merge WITHOUT caller-provided partial buffers.  No counterpart
 * in the reference (its kernels always take caller-allocated partials).
 * For callers that cannot allocate device memory -- e.g. a host-language
 * binding that may only forward pointers it was handed, or code running where
 * cudaMalloc would stall the device -- the (m, l, acc) partials live in a fixed
 * array inside the library: LOCKS_NOALLOC_MAX_ROWS x 130 floats (about 8.5 MB
 * that every GPU loading the library keeps until the process exits).
 * Same arguments and results as locks_decode_split followed by
 * locks_merge_splits.  Limits and rules:
 *   - n_req*n_kv*split*G must not exceed LOCKS_NOALLOC_MAX_ROWS, otherwise
 *     LOCKS_ERR_SIZE is returned and nothing is launched;
 *   - the first call on a device resolves the array's device address (a CUDA
 *     runtime query, not a stream operation): make that first call before any
 *     stream capture begins on that device, with the device current; the
 *     address is kept for the life of the device's primary context (after a
 *     cudaDeviceReset the library must be reloaded), and the look-up is
 *     serialised between host threads;
 *   - all calls share the one array and it keeps the previous call's contents;
 *     nothing in it has to start at zero (only partials written by the current
 *     call are read back), but two calls whose kernels overlap on the GPU --
 *     different streams, or graph branches -- race on it: serialise them;
 *   - it performs no cudaMalloc/cudaFree and calls no allocating library. */
#define LOCKS_NOALLOC_MAX_ROWS 16384
int locks_decode_split_noalloc(
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    void* out, int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, int split, int pps_min, float scale, int* status,
    locks_stream_t stream);

/* Dense full-KV paged decode (every page of every request) with the same
 * split kernel and merge: the baseline of the sparse/dense crossover curve.
 * The reference takes its dense baseline from FlashAttention
 * (backend/attn.py:253-267 delegates there); it has no kernel of its own. */
int locks_dense_decode(const void* q, int64_t q_stride_req, const void* k_cache,
                       const void* v_cache, int64_t kv_stride_block,
                       int64_t kv_stride_tok, int64_t kv_stride_head,
                       const int32_t* block_table, int64_t bt_stride,
                       const int32_t* seq_lens, float* m_part, float* l_part,
                       float* acc_part, void* out, int64_t out_stride_req,
                       int n_req, int n_kv, int G, int head_dim, int page,
                       int split, float scale, int* status,
                       locks_stream_t stream);

/* ---- MLA (latent KV) path ------------------------------------------------
 * Geometry: latent width kv_lora_rank 512 + rope 64 = 576, page 16, 16 query
 * heads sharing one latent head (16 is the fragment height; fewer heads are
 * padded by the caller with zero rows).
 *
 * One factor record per physical block (LOCKS_MLA_REC_BYTES):
 *   [0,8192)    Rf  fp16 8 x 512   right factors, row r = mode r (descending)
 *   [8192,8448) Lf  fp16 16 x 8    left factors (token x mode), Lf Rf ~ page
 * The rope part of the keys is read from the latent cache itself. */
#define LOCKS_MLA_REC_BYTES 8448
#define LOCKS_MLA_LKV 512
#define LOCKS_MLA_ROPE 64
#define LOCKS_MLA_HEADS 16

/* Rank-8 factors of each listed block's 16 x 512 latent page: Gram (16x16),
 * Jacobi eigh, top-8 modes in descending order, modes at or below
 * sigma_1*sqrt(eps) zeroed; Lf = W sigma, Rf = W^T page / sigma.
 * cache: bf16 (num_blocks, 16, 576) with the given element strides.
 * Replaces selection/mla_select.py:26-108 (_page_basis, build_page_factors). */
int locks_mla_build_factors(const void* cache, int64_t stride_block,
                            int64_t stride_tok, void* records,
                            const int32_t* blocks, int n_blocks, int num_blocks,
                            locks_stream_t stream);

/* Factor bookkeeping of a decode batch ON THE DEVICE (two launches, no host
 * synchronisation, fixed shape): a gate kernel decides per row whether its
 * factors are missing or stale -- entries are remembered under the row's first
 * block id as (content fingerprint of the first and the last covered prompt page,
 * number of covered pages); a row with no entry, a row that shrank below its
 * entry, or a fingerprint mismatch (block ids reused by another request) is
 * flagged -- writes need[row] and n_cache[row] (pages with factors), and the
 * factor kernel then rebuilds all pages of the flagged rows.  fp_tab (f32) and
 * nc_tab (i32, initialised to -1) have num_blocks entries per layer.
 * Replaces the host-side factor cache of backend/mla_attn.py:212-239 and its
 * per-step .tolist() synchronisations (:118-133). */
int locks_mla_refresh_rows(const void* cache, int64_t stride_block,
                           int64_t stride_tok, void* records,
                           const int32_t* block_table, int64_t bt_stride,
                           const int32_t* seq_lens, float* fp_tab, int32_t* nc_tab,
                           int32_t* need, int32_t* n_cache, int n_rows,
                           int max_pages, int num_blocks, locks_stream_t stream);

/* Per-row page parameters of the MLA keep rule: n_pages = ceil(L/16);
 * n_sel_hi = n_pages - window; b = n_pages when n_pages <= budget_pages (keep
 * all), else budget_pages - |sink pages U last window pages| (>= 0).
 * Replaces the bookkeeping of selection/mla_score_torch.py:51-73 (topb_middle). */
int locks_mla_derive(const int32_t* seq_lens, int n_rows, int budget_pages,
                     int sink_pages, int window_pages, int32_t* n_pages,
                     int32_t* n_sel_hi, int32_t* b_fix, locks_stream_t stream);

/* score[row,p] = scale * max_h max_t ((q_c[h] Rf^T) Lf^T + q_rope[h] k_rope^T)[t]
 * for p < n_cache[row]; -inf for n_cache[row] <= p < n_pages[row].
 * q: bf16 (n_rows, 16, 576) = [q_c | q_rope].  score: f32 (n_rows, max_pages).
 * Replaces selection/mla_score_triton.py:98-151 (factored batched scorer);
 * CPU twin selection/mla_score_torch.py:27-48.  Selection itself is
 * locks_topb_select(LOCKS_COMBINE_NONE) with n_kv = 1. */
int locks_mla_score(const void* q, int64_t q_stride_row, const void* records,
                    const void* cache, int64_t stride_block, int64_t stride_tok,
                    const int32_t* block_table, int64_t bt_stride,
                    const int32_t* n_cache, const int32_t* n_pages, float* score,
                    int n_rows, int max_pages, int num_blocks, float scale,
                    int zsplit, int* status, locks_stream_t stream);

/* Attention of every row over its kept pages of the latent cache:
 * o[row,h,:512] = softmax(scale * q[h] . kv^T) kv[:, :512], lse = logsumexp.
 * Tokens at or beyond seq_lens[row] are masked.  o: bf16 (n_rows,16,512),
 * lse: f32 (n_rows,16).  One thread-block cluster per row.
 * Replaces backend/mla_attn.py:178-201. */
int locks_mla_decode(const void* q, int64_t q_stride_row, const void* cache,
                     int64_t stride_block, int64_t stride_tok,
                     const int32_t* block_table, int64_t bt_stride,
                     const int32_t* page_table, const int32_t* page_cnt,
                     const int32_t* seq_lens, void* out, float* lse, int n_rows,
                     int max_pages, float scale, int* status,
                     locks_stream_t stream);

/* locks_mla_decode on the tcgen05 tensor cores, tokens in the M dimension:
 * S^T[128 tokens x 16 heads] = K[128 x 576] Q^T and O^T[512 x 16] = V^T[512 x 128]
 * P^T, accumulators in tensor memory, pages gathered through the block table by
 * TMA tensor copies (2-D map over the cache seen as (num_blocks * 16, 576), box
 * 16 x 64, 128-byte swizzle) -- one copy of a page feeds both products.  Same
 * arguments and results as locks_mla_decode plus num_blocks (the tensor map's
 * extent) and cnt_hint (the page count a long row is expected to keep, normally
 * the budget: lets the kernel fetch its first page-table entries together with
 * the count; any value is correct, a wrong guess costs one round trip).  Needs stride_block == 16 * stride_tok (LOCKS_ERR_GEOMETRY
 * otherwise: use locks_mla_decode).  The reference computes this step with
 * eager fp32 bmm (backend/mla_attn.py:178-201). */
int locks_mla_decode_tc(const void* q, int64_t q_stride_row, const void* cache,
                        int64_t stride_block, int64_t stride_tok,
                        const int32_t* block_table, int64_t bt_stride,
                        const int32_t* page_table, const int32_t* page_cnt,
                        const int32_t* seq_lens, void* out, float* lse, int n_rows,
                        int max_pages, int num_blocks, int cnt_hint, float scale,
                        int* status, locks_stream_t stream);
/* The thread-block cluster size (CTAs per row) locks_mla_decode_tc will use for
 * n_rows rows whose page lists hold about pages_hint entries: host-side query,
 * no launch.  A caller choosing between locks_mla_decode_tc and locks_mla_decode
 * by the number of 8-page tiles a CTA would walk needs it. */
int locks_mla_decode_tc_cluster_size(int n_rows, int pages_hint);


#ifdef __cplusplus
}
#endif
#endif  /* LOCKS_B200_H_ */
