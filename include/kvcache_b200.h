/*
 * kvcache_b200.h — C ABI of the B200 (sm_100a) retrieval-sparse decode attention library.
 *
 * One shared library, plain pointers and sizes, no C++ or torch types. Every entry point
 *   - takes DEVICE pointers unless a parameter says "host",
 *   - takes the CUDA device ordinal and the stream (a cudaStream_t passed as void*),
 *   - validates shapes, strides and alignment on the host and returns a kvb_status
 *     BEFORE anything is launched when they are wrong,
 *   - never allocates, never frees, never synchronises the device, never throws
 *     (the exceptions, kvb_device_status and kvb_exchange_alloc / _free, say so).
 *
 * Tensor naming: B batch, Hq query heads, Hkv KV heads, G = Hq / Hkv, D head dim (128),
 * T cached ("history") tokens, C partial channels (even, <= 128), k top-k, S length of a
 * final index list. "bf16" is the 16-bit brain float; rows are contiguous along D.
 *
 * Reference interfaces these entry points stand in for (paths inside littlexi001/kv_cache):
 *   QCK  = ymluo/projects/qwen3_top2_head_limit3_ppl/src/qabs_cuda_kernels.py
 *   EVAL = ymluo/projects/qwen3_top2_head_limit3_ppl/src/evaluate_qwen3_top2_head_limit3_ppl.py
 */
#ifndef KVCACHE_B200_H
#define KVCACHE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum kvb_status {
  KVB_OK = 0,
  KVB_BAD_SHAPE = 1,          /* a dimension is zero/negative/unsupported                */
  KVB_BAD_ALIGN = 2,          /* a pointer or stride breaks the alignment rule stated     */
  KVB_BAD_DEVICE = 3,         /* device ordinal out of range or cudaSetDevice failed      */
  KVB_WORKSPACE_TOO_SMALL = 4,
  KVB_TIMEOUT = 5,            /* a bounded device-side wait gave up (see kvb_device_status)*/
  KVB_CUDA_ERROR = 6,         /* a CUDA runtime call or a launch returned an error        */
  KVB_BAD_ARG = 7,            /* null pointer where one is required, bad flag, ...        */
  KVB_SCRATCH_LIMIT = 8       /* the problem needs more than the library's built-in scratch */
} kvb_status;

/* Library version (major*10000 + minor*100 + patch) and a static string for a status. */
int kvb_version(void);
const char* kvb_status_string(int status);

/* Reads and clears the sticky per-device status word that kernels set when a bounded wait
 * (mbarrier / pipeline) runs out. SYNCHRONISES the device; meant for health checks and
 * tests, never for the hot path. *out_status receives a kvb_status. */
int kvb_device_status(int device, int* out_status);

/* ---------------------------------------------------------------------------------------
 * Stage 1 — quantize / pack K to int4 over C chosen channels, per-token symmetric scale.
 *
 * No counterpart in the reference (its K stays bf16); the closest structure is the
 * incrementally appended side copy of K, EVAL:2018-2042 (SparQMeanState.key_dim_major).
 *
 *   key          bf16 [B,Hkv,T,D] view: element strides key_sb/key_sh/key_st, D contiguous;
 *                the pointer and all strides must be multiples of 8 elements (16 bytes).
 *   channel_idx  int32 [Hkv,C], ascending per head, each in [0,D).
 *   packed       uint8 cache [B,Hkv,cap,C/2]; byte strides packed_sb/packed_sh; token
 *                stride is C/2. Byte j of a token: low nibble = code of channel_idx[2j],
 *                high nibble = code of channel_idx[2j+1], two's complement, in [-7,7].
 *   scale        fp32 cache [B,Hkv,cap]; element strides scale_sb/scale_sh.
 *   t_dst        first destination token in the caches (rows t_dst .. t_dst+T-1 are written).
 * scale = max(absmax, 2^-24) / 7 (IEEE division), code = clamp(rint(x / scale), -7, 7).
 * kvb_quantize_append is the T == 1 form used once per decode step.
 * ------------------------------------------------------------------------------------- */
int kvb_quantize_pack(const void* key, int64_t key_sb, int64_t key_sh, int64_t key_st,
                      const int32_t* channel_idx,
                      uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                      float* scale, int64_t scale_sb, int64_t scale_sh,
                      int B, int Hkv, int T, int D, int C, int64_t t_dst,
                      int device, void* stream);

int kvb_quantize_append(const void* key_row, int64_t key_sb, int64_t key_sh,
                        const int32_t* channel_idx,
                        uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                        float* scale, int64_t scale_sb, int64_t scale_sh,
                        int B, int Hkv, int D, int C, int64_t t_dst,
                        int device, void* stream);

/* ---------------------------------------------------------------------------------------
 * Stage 2 — decode scoring: one query token per sequence against all T packed keys.
 *
 * Stands in for partial_scores / partial_scores_dim_major (QCK:654-665; kernels QCK:63-158;
 * torch form EVAL:4443-4446) with the channel list as an input like dim_indices there, but
 * computed exactly in integers on the int4 cache:
 *   qcode[b,h,c] = clamp(rint(q[b,h,ch[h/G][c]] / qscale[b,h]), -127, 127),
 *   qscale = max(absmax_c, 2^-24) / 127,
 *   acc[b,h,t]  = sum_c qcode * code                       (int32, exact)
 *   deq[b,h,t]  = (float(acc) * scale[b,h/G,t]) * qscale[b,h]   (two rounded fp32 products)
 *   gmax[b,g,t] = max over the G heads of group g of deq, with -0 stored as +0.
 *
 *   query     bf16 [B,Hq,D], element strides q_sb/q_sh, D contiguous.
 *   packed/scale/channel_idx as in stage 1. For the streaming fast path (C in {32,64,128},
 *   G in {1,2,4,8}) packed must be 16-byte aligned with 16-byte-multiple strides and scale
 *   16-byte aligned with strides that are multiples of 4 elements; other even C <= 128 and
 *   other G <= 16 take a slower generic kernel.
 *   gmax_out  fp32 [B,Hkv,T] or NULL; acc_out int32 [B,Hq,T] or NULL; deq_out fp32 [B,Hq,T]
 *   or NULL — all dense. At least one must be given.
 *   hist_out  uint32 [B*Hkv, 4096] or NULL: when given (and gmax_out is given) the kernel
 *   ADDS the histogram of the top 12 bits of the order-preserving key of gmax into it
 *   (the caller zeroes it); kvb_select_topk can then skip its own histogram pass.
 * ------------------------------------------------------------------------------------- */
int kvb_score_decode(const void* query, int64_t q_sb, int64_t q_sh,
                     const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                     const float* scale, int64_t scale_sb, int64_t scale_sh,
                     const int32_t* channel_idx,
                     int B, int Hq, int Hkv, int T, int D, int C,
                     float* gmax_out, int32_t* acc_out, float* deq_out,
                     uint32_t* hist_out,
                     int device, void* stream);

/* Stage 2, candidate form (what the fused step uses): instead of writing a score per token, the
 * scorer appends every token whose group maximum reaches a per-row threshold to that row's
 * candidate list, so no score row ever goes to memory. No counterpart in the reference.
 *
 * kvb_candidate_capacity(top_k): entries per row the lists must hold (0 if top_k is too large).
 * kvb_sample_thresholds: tau[b*Hkv+g] from a 1/32 sample of the row (32 evenly spaced runs, at most
 *   4096 tokens): the sample value whose rank predicts max(1.75 top_k, 96 / sampled fraction)
 *   tokens above it; -inf when T <= capacity. The prediction is statistical: callers must check
 *   top_k <= count <= capacity afterwards (kvb_decode_step does, and re-scores the rare failing
 *   row exactly).
 * kvb_score_candidates: cand[row, i] = (order-preserving key of gmax) << 32 | (0xFFFFFFFF - token),
 *   cand_count[row * 32] = number appended (it keeps counting past cand_cap; entries beyond the
 *   capacity are dropped). cand_count must be zeroed by the caller. Streaming configurations only
 *   (C in {32,64,128}, G in {1,2,4,8}, aligned side cache), else KVB_BAD_SHAPE. */
int kvb_candidate_capacity(int top_k);

int kvb_sample_thresholds(const void* query, int64_t q_sb, int64_t q_sh,
                          const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                          const float* scale, int64_t scale_sb, int64_t scale_sh,
                          const int32_t* channel_idx,
                          int B, int Hq, int Hkv, int T, int D, int C, int top_k,
                          float* tau, int device, void* stream);

int kvb_score_candidates(const void* query, int64_t q_sb, int64_t q_sh,
                         const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                         const float* scale, int64_t scale_sb, int64_t scale_sh,
                         const int32_t* channel_idx,
                         int B, int Hq, int Hkv, int T, int D, int C,
                         const float* tau, uint64_t* cand, uint32_t* cand_count, int cand_cap,
                         int device, void* stream);

/* ---------------------------------------------------------------------------------------
 * Stage 3 — exact top-k select per row; among equal scores the lower index wins.
 *
 * Stands in for the torch.topk candidate selection of the reference (EVAL:4448, count rule
 * EVAL:4423) with the tie-break pinned, so the selected SET is unique. -0 and +0 compare
 * equal. The kk winners are written in one of two pinned orders:
 *   order 0: (score descending, index ascending) — the order torch.topk(sorted=True) aims at;
 *   order 1: index ascending — cheaper to produce and friendlier to the K/V gather that follows.
 *
 *   scores    fp32 [R,T] rows (row_stride elements apart), no NaN.
 *   payload   int32 [R,T] (same row stride) or NULL. With NULL the index of column t is
 *             t + idx_offset; otherwise it is payload[r,t] (used to merge per-rank candidate
 *             lists that carry global token ids). Indices must be unique within a row and
 *             fit in int32.
 *   k         requested count; kk = min(k, T) entries are produced per row. k <= 16384.
 *   out_idx32 int32 [R,kk] or NULL; out_idx64 int64 [R,kk] or NULL; out_scores fp32 [R,kk]
 *             or NULL (dense, row stride kk).
 *   hist_in   uint32 [R,4096] histogram already produced by kvb_score_decode, or NULL.
 *   workspace >= kvb_select_topk_workspace_bytes(R, T, k) bytes, 256-byte aligned.
 * ------------------------------------------------------------------------------------- */
size_t kvb_select_topk_workspace_bytes(int R, int T, int k);

int kvb_select_topk(const float* scores, int64_t row_stride, const int32_t* payload,
                    int R, int T, int k, int64_t idx_offset, int order,
                    int32_t* out_idx32, int64_t* out_idx64, float* out_scores,
                    const uint32_t* hist_in,
                    void* workspace, size_t workspace_bytes,
                    int device, void* stream);

/* Top-k select for callers that cannot allocate device memory. It has no counterpart in the
 * reference. Some hosts of this library own no allocator they may call at this point: code that
 * runs inside a stream-ordered region where cudaMalloc would synchronise the device, a plugin
 * whose embedding runtime forbids it from allocating, a tight memory budget already handed out in
 * full. kvb_select_topk needs a workspace from its caller; this variant keeps the same workspace
 * in a fixed array inside the library image instead (kvb_select_topk_static_limit_bytes() bytes,
 * 4 MiB; every GPU that loads the library carries it until the process ends). Inputs and outputs
 * are still the caller's. Same semantics and arguments as kvb_select_topk without payload,
 * hist_in and workspace.
 *   - Problems whose workspace (kvb_select_topk_workspace_bytes(R, T, k)) exceeds the limit are
 *     refused with KVB_SCRATCH_LIMIT before anything is launched (about 50 rows at k <= 4096).
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call outside any stream capture. A first call whose stream is being
 *     captured is refused with KVB_BAD_ARG before any runtime call, so the capture survives.
 *   - Nothing is allocated or freed; counters and histogram are cleared by the call itself.
 *   - All calls share the one array: two calls that may overlap on the GPU (different streams)
 *     race with each other. Serialise them on one stream or with events. */
size_t kvb_select_topk_static_limit_bytes(void);

int kvb_select_topk_static(const float* scores, int64_t row_stride, int R, int T, int k,
                           int64_t idx_offset, int order,
                           int32_t* out_idx32, int64_t* out_idx64, float* out_scores,
                           int device, void* stream);

/* ---------------------------------------------------------------------------------------
 * Final index list — selected || sink || recent || self with protected ranges invalidated.
 * Restates _qabs_final_indices_from_selected (EVAL:2938-2982); with append_protected != 0,
 * _qabs_final_indices_append_protected (EVAL:2985-3022), which keeps the selected entries
 * valid even inside the protected ranges.
 *
 *   sel_idx     int32 [R,kk] selected history indices; sel_valid uint8 [R,kk] or NULL (all valid)
 *   out_idx     int32 [R,S], out_valid uint8 [R,S] with
 *               S = kvb_final_index_count(kk, history_count, sink, recent, keep_self).
 * ------------------------------------------------------------------------------------- */
int kvb_final_index_count(int kk, int history_count, int protect_sink, int protect_recent,
                          int keep_self);

int kvb_build_final_indices(const int32_t* sel_idx, const uint8_t* sel_valid, int R, int kk,
                            int history_count, int key_count,
                            int protect_sink, int protect_recent, int keep_self,
                            int append_protected,
                            int32_t* out_idx, uint8_t* out_valid,
                            int device, void* stream);

/* ---------------------------------------------------------------------------------------
 * Stage 4 — exact attention over gathered rows (split over the list, log-sum-exp merge).
 *
 * Stands in for final_attention (QCK:694-705, kernel QCK:335-419) and the torch form
 * _qabs_attention_from_final_indices (EVAL:4612-4647); like the Triton kernels of the
 * reference it reads UN-repeated K/V (kv_head = head / G,
 * run_longrange_book_index_sparse_eval.py:879).
 *
 *   query    bf16 [B,Hq,D] (strides q_sb/q_sh); key/value bf16 [B,Hkv,Tk,D] views with
 *            element strides *_sb/*_sh/*_st, D = 128 contiguous, all multiples of 8.
 *   indices  [B,Hi,S] with Hi == Hkv (one list per KV head, shared by its G query heads) or
 *            Hi == Hq (one list per query head, the reference layout); int32, or int64 when
 *            idx_is_i64 != 0; dense.
 *   valid    uint8 [B,Hi,S] or NULL (all valid). Entries that are invalid or outside
 *            [0,Tk) get weight zero (QCK:366-367).
 *   mask     fp32 additive mask rows [B,Tk] (element stride mask_sb) or NULL
 *            (the torch form adds mask[b, 0, 0, idx], EVAL:4637-4641).
 *   out      bf16 [B,1,Hq,D] dense, or NULL.
 *   out_partial fp32 [B,Hq,D+2] or NULL: un-normalised accumulator scaled to the row
 *            maximum m, then m, then l = sum exp(s - m) — what a sequence shard contributes
 *            (kvb_lse_merge combines shards). A row with no valid entry gives zeros in out
 *            (QCK:388,404) and (0, -inf, 0) in out_partial.
 *   workspace >= kvb_sparse_attend_workspace_bytes(B, Hq, Hi, S), 256-byte aligned.
 * ------------------------------------------------------------------------------------- */
size_t kvb_sparse_attend_workspace_bytes(int B, int Hq, int Hi, int S);

int kvb_sparse_attend(const void* query, int64_t q_sb, int64_t q_sh,
                      const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
                      const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st,
                      const void* indices, int idx_is_i64, const uint8_t* valid,
                      const float* mask, int64_t mask_sb,
                      int B, int Hq, int Hkv, int Hi, int Tk, int D, int S,
                      float scaling,
                      void* out, float* out_partial,
                      void* workspace, size_t workspace_bytes,
                      int device, void* stream);

/* Attention over the IMPLICIT list  selected || sink || recent || self  (nothing materialised):
 * the composition of kvb_build_final_indices and kvb_sparse_attend, i.e. the tail of
 * _qabs_candidate_attention_forward (EVAL:4460-4501), with one list per KV head.
 *
 *   selected   int32 [B*Hkv, kk] token ids; an id contributes iff 0 <= id - id_base < history_count
 *              (and it is not in a protected range unless append_protected). With id_base != 0
 *              the ids are global and this rank owns [id_base, id_base + history_count): what a
 *              sequence shard needs after the global top-k merge.
 *   sel_count  optional int32 [B*Hkv]: row r uses only its first sel_count[r] (<= kk) entries of
 *              `selected`, and the work is divided over that shorter list (the compacted "owned"
 *              lists of kvb_merge_candidates); NULL = all kk.
 *   key/value  views whose rows 0 .. history_count-1 are the history and, when keep_self != 0,
 *              row history_count is the token being decoded (Tk >= history_count + keep_self).
 *   out / out_partial / mask / workspace as in kvb_sparse_attend; workspace size from
 *   kvb_sparse_attend_workspace_bytes(B, Hq, Hkv, kvb_final_index_count(kk, history_count, ...)). */
int kvb_attend_selected(const void* query, int64_t q_sb, int64_t q_sh,
                        const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
                        const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st,
                        const int32_t* selected, int kk, const int32_t* sel_count,
                        int64_t id_base, int history_count,
                        int protect_sink, int protect_recent, int keep_self, int append_protected,
                        const float* mask, int64_t mask_sb,
                        int B, int Hq, int Hkv, int Tk, int D, float scaling,
                        void* out, float* out_partial,
                        void* workspace, size_t workspace_bytes,
                        int device, void* stream);

/* Sequence-shard front end and merge (no counterpart in the reference, which has no sharding).
 *
 * kvb_shard_candidates: the exact local top-k of a shard in one call (sampled threshold, candidate
 *   scorer, bounds check with exact rescue, exact finish): out_comp uint64 [B*Hkv, kk],
 *   kk = min(top_k, T), each entry (order-preserving key of the group max) << 32 |
 *   (0xFFFFFFFF - (token + id_offset)), in no particular order except that, with 0 < split_k < kk,
 *   the split_k best entries come first (a reader may take that prefix as the local top-split_k).
 *   Needs the streaming configuration
 *   and top_k small enough for the candidate capacity (else KVB_BAD_SHAPE: use kvb_score_decode +
 *   kvb_select_topk). workspace >= kvb_shard_candidates_workspace_bytes(B, Hkv, T, top_k).
 * kvb_merge_candidates: the global top-k of N such lists after an all-gather: gathered uint64
 *   [N, R, kk] -> out_idx int32 [R, min(top_k, N*kk)] global token ids, ascending when
 *   id_range (the total token count) is at most 262144 (a cheap on-chip bitmap), otherwise in
 *   arbitrary order (the set is exact either way). With N > 1 every list must hold top_k entries (kk == top_k).
 *   The composites are unique, so every rank that runs this on the same gathered data gets the
 *   same set.
 *   prefix_k > 0 says that every list has its prefix_k best entries first (split_k above). When the
 *   N prefixes fit on chip (N * prefix_k <= 8192, N <= 64) the kernel selects from them alone and
 *   accepts the result iff, for every list, the smallest entry of its prefix is itself no larger than
 *   the k-th winner (nothing behind the prefix can then be a winner); otherwise it repeats the select
 *   over the whole lists. The result is the same exact set either way.
 *   out_owned (optional, with out_owned_count int32 [R]): the winners whose id lies in
 *   [own_base, own_limit), compacted per row (row pitch as out_idx), for kvb_attend_selected's
 *   sel_count; the output order is then arbitrary. */
size_t kvb_shard_candidates_workspace_bytes(int B, int Hkv, int T, int top_k);

int kvb_shard_candidates(const void* query, int64_t q_sb, int64_t q_sh,
                         const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                         const float* scale, int64_t scale_sb, int64_t scale_sh,
                         const int32_t* channel_idx,
                         int B, int Hq, int Hkv, int T, int D, int C, int top_k, int split_k,
                         int64_t id_offset,
                         uint64_t* out_comp, void* workspace, size_t workspace_bytes,
                         int device, void* stream);

int kvb_merge_candidates(const uint64_t* gathered, int N, int R, int kk, int top_k, int64_t id_range,
                         int prefix_k, int32_t* out_idx,
                         int64_t own_base, int64_t own_limit, int32_t* out_owned, int32_t* out_owned_count,
                         int device, void* stream);

/* Stages 2 and 3 in one call: the exact top-k token ids per (batch, KV head) straight from the int4 cache
 * (sampled threshold -> candidate-emitting scorer -> exact finish; the chain of kvb_shard_candidates with ids
 * instead of composites). It stands where the reference runs its partial scoring followed by torch.topk
 * (EVAL:4435-4448) when only the candidate ids are wanted (the rerank modes). out_idx int32
 * [B*Hkv, min(top_k,T)], ascending when `ascending` != 0 and the row's bitmap fits on chip (T up to ~600K),
 * otherwise in no particular order; same shape limits and workspace as kvb_shard_candidates. */
int kvb_score_select(const void* query, int64_t q_sb, int64_t q_sh,
                     const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                     const float* scale, int64_t scale_sb, int64_t scale_sh,
                     const int32_t* channel_idx,
                     int B, int Hq, int Hkv, int T, int D, int C, int top_k, int ascending,
                     int32_t* out_idx, void* workspace, size_t workspace_bytes,
                     int device, void* stream);

/* Exact rerank of a candidate union given as id LISTS: replaces candidate_full_scores (QCK:668-691, kernel
 * QCK:160-216: three dense bool masks [B,H,T] in, a dense fp32 [B,H,T] row out) followed by torch.topk
 * (EVAL:4297-4302), i.e. the core of the reference's rerank / reuse modes (EVAL:4147-4311) and of its
 * "top2" modes (EVAL:4704-4720).
 *   list0 / list1 / list2   int32 [R, n_i] token ids (current candidates; previous candidates; previous final
 *                           set; list1, list2 may be NULL), R = B * Hi list rows with Hi = Hkv (one list per KV
 *                           head, shared by its G query heads) or Hq (one per query head, the reference's form).
 *                           count_i int32 [R] or NULL: row r uses its first count_i[r] entries. Ids outside
 *                           [0, history_count) (-1 padding, ids of a longer past) are ignored; duplicates within
 *                           and across the lists are merged.
 *   force_sink / force_recent  additionally put [0, force_sink) and [history_count - force_recent, history_count)
 *                           into the union (the reference's lagged modes, EVAL:4209-4214); 0 = off.
 *   score                   max over the query heads that share the list of (q . k) in fp32 over all D channels,
 *                           times `scaling`, plus mask[b, token] (fp32 [B, >= history_count] or NULL).
 *   out_idx                 int32 [R, keep]: the min(keep, |union|) best ids by (score desc, id asc), written in
 *                           ASCENDING id order, the rest of the row -1; out_count int32 [R] how many.
 * Limits: n0 + n1 + n2 + forced <= 16384, history_count small enough for two on-chip bitmaps (about 600K
 * tokens), D = 128; otherwise KVB_BAD_SHAPE. workspace >= kvb_rerank_union_workspace_bytes(R, n0+n1+n2+forced). */
size_t kvb_rerank_union_workspace_bytes(int R, int max_union);

int kvb_rerank_union(const void* query, int64_t q_sb, int64_t q_sh,
                     const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
                     const int32_t* list0, int n0, const int32_t* count0,
                     const int32_t* list1, int n1, const int32_t* count1,
                     const int32_t* list2, int n2, const int32_t* count2,
                     int force_sink, int force_recent,
                     const float* mask, int64_t mask_sb,
                     int B, int Hq, int Hkv, int Hi, int history_count, int D, float scaling, int keep,
                     int32_t* out_idx, int32_t* out_count,
                     void* workspace, size_t workspace_bytes, int device, void* stream);

/* Final keep set of the rerank modes as a list: the given ids, plus the protected ranges [0, force_sink) and
 * [history_count - force_recent, history_count) (EVAL:4306-4311), each token then widened to its aligned block
 * of block_size tokens (_expand_history_keep_to_aligned_blocks, EVAL:2914-2922; block_size 1 = no widening),
 * de-duplicated, in ascending order. list int32 [R, n] with optional per-row count; ids outside
 * [0, history_count) are ignored. out_idx int32 [R, out_cap] (entries beyond out_cap are dropped, the unused
 * tail is -1), out_count int32 [R]. history_count / block_size up to about 1.8 M bits (on-chip bitmap). */
int kvb_expand_final(const int32_t* list, int n, const int32_t* count, int R, int history_count,
                     int force_sink, int force_recent, int block_size,
                     int32_t* out_idx, int out_cap, int32_t* out_count, int device, void* stream);

/* SparQ-style mean-value correction (the reference's "sparqfast" mode,
 * _sparq_fast_attention_output_for_query, EVAL:2646-2722, with its running mean of V, EVAL:2006-2016):
 * the exact attention over the selected tokens is blended with the mean of V by the softmax mass alpha that
 * the selected tokens carry under the APPROXIMATE logits. Here those logits are the dequantised int4 partial
 * scores of the side cache, s[b,h,t] = deq[b,h,t] / sqrt(D * |q_sel|_1 / |q|_1) (+ mask[b,t]), q_sel = the
 * query on the layer's channel list (EVAL:2683-2686 for the scale), softmax over all T cached tokens.
 *   kvb_sparq_alpha         alpha fp32 [B*Hq] = sum over the ids in `selected` (int32 [B*Hkv, kk], optional
 *                           per-row sel_count, ids outside [0,T) ignored) of softmax_h(s)[id]. One streaming
 *                           pass over the int4 cache plus a re-score of the selected rows; C a multiple of 8,
 *                           G <= 8. workspace >= kvb_sparq_alpha_workspace_bytes(B, Hq, T).
 *   kvb_attend_selected_blend  kvb_attend_selected (no protected ranges, local ids) whose output is
 *                           value_mean + alpha * (attention - value_mean); value_mean fp32 [B,Hkv,D] dense is
 *                           the caller's running mean of V over all Tk rows. */
size_t kvb_sparq_alpha_workspace_bytes(int B, int Hq, int T);

int kvb_sparq_alpha(const void* query, int64_t q_sb, int64_t q_sh,
                    const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                    const float* scale, int64_t scale_sb, int64_t scale_sh,
                    const int32_t* channel_idx, const float* mask, int64_t mask_sb,
                    const int32_t* selected, int kk, const int32_t* sel_count,
                    int B, int Hq, int Hkv, int T, int D, int C,
                    float* alpha, void* workspace, size_t workspace_bytes, int device, void* stream);

int kvb_attend_selected_blend(const void* query, int64_t q_sb, int64_t q_sh,
                              const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
                              const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st,
                              const int32_t* selected, int kk, const int32_t* sel_count,
                              int history_count, int keep_self,
                              const float* mask, int64_t mask_sb,
                              const float* alpha, const float* value_mean,
                              int B, int Hq, int Hkv, int Tk, int D, float scaling,
                              void* out, void* workspace, size_t workspace_bytes,
                              int device, void* stream);

/* ---------------------------------------------------------------------------------------
 * Sequence-sharded decode step without a collective call (no counterpart in the reference, which
 * has no sharding). Rank r of `world` owns the history tokens [id_offset, id_offset + t_local) of
 * every sequence (bf16 K/V rows and the int4 side cache); query, channel list and the decoded
 * token's K/V row are replicated. One call enqueues the whole step on `stream`:
 *   phase 1  sample -> candidate scorer -> exact local top-k; the last kernel stores its
 *            min(top_k, 8192/world) best (score, global id) composites per (batch, KV head) into
 *            EVERY rank's exchange buffer over NVLink as tagged pairs — each 32-bit half of a composite
 *            beside the step number in one aligned 8-byte store, so a reader that finds the step number
 *            has the half, without a fence or a flag — and then raises a per-(source rank, row) flag
 *            there (st.release.sys), which says that the row's WHOLE local list may be read;
 *   phase 2  global merge: polls the pairs of the `world` prefixes of its row in its LOCAL buffer (bounded),
 *            selects the global top-k from them with the acceptance test of kvb_merge_candidates (a
 *            row that fails it waits for the `world` flags and reads the ranks' whole lists with plain
 *            loads from their memory), compacts the winners this rank owns; attention over those rows;
 *            the chunk merge stores the un-normalised (o, m, l) of every (batch, head) into every rank's
 *            buffer, again as tagged pairs;
 *   phase 3  polls the `world` partials' pairs and combines them by log-sum-exp into `out` (the same
 *            bits on every rank).
 * Pairs and flags carry a step number kept in the exchange buffer, so the same call sequence can be
 * captured once in a CUDA graph and replayed. Every wait gives up after wait_polls polls (0 = a few
 * seconds' worth), sets KVB_TIMEOUT in the device status word and lets the kernel return. Only plain and
 * volatile loads and stores and the flags' release/acquire operations touch peer memory.
 *
 * All ranks must call with the same B, Hq, Hkv, top_k, world and take the same number of steps.
 * Needs the streaming scorer configuration (C in {32,64,128}, G in {1,2,4,8}, aligned side cache),
 * 3 * top_k <= 16384 and top_k <= t_local on every rank; otherwise KVB_BAD_SHAPE and the caller
 * composes the step from the operators above around its own all-gathers.
 *
 * Exchange buffers. kvb_exchange_alloc / kvb_exchange_free are the only entry points of this
 * library that allocate device memory (cudaMalloc / cudaFree, zero-filled, synchronising): call
 * them at set-up. Each rank allocates kvb_sharded_exchange_bytes(...) bytes, publishes the 64-byte
 * handle to its peers (any host transport), and maps theirs with kvb_exchange_open (CUDA IPC with
 * lazy peer access; the owning device may differ from `device`). exchange[r] in the parameters is
 * rank r's buffer as mapped in the calling process; exchange[rank] is the local allocation.
 *
 * `phases` (bit 0, 1, 2 = phase 1, 2, 3; 7 = the whole step) exists so that several ranks can be
 * stepped from ONE process on one GPU, phase by phase (all ranks' phase 1, then all ranks' phase
 * 2, ...): kernels that wait for each other must never be queued behind one another on one GPU.
 * ------------------------------------------------------------------------------------- */
typedef struct kvb_sharded_step_params {
  const void* query;  int64_t q_sb, q_sh;                 /* bf16 [B,Hq,D]                         */
  const void* key;    int64_t k_sb, k_sh, k_st;           /* bf16 [B,Hkv,t_local+1,D]: the shard's   */
  const void* value;  int64_t v_sb, v_sh, v_st;           /* rows, then the decoded token's row     */
  const uint8_t* packed; int64_t packed_sb, packed_sh;    /* int4 cache of the shard's rows         */
  const float* scale;    int64_t scale_sb, scale_sh;
  const int32_t* channel_idx;                             /* int32 [Hkv,C]                          */
  int B, Hq, Hkv, D, C;
  int t_local;                                            /* history tokens this rank owns          */
  int64_t id_offset;                                      /* global id of local row 0               */
  int64_t total_tokens;                                   /* global history length                  */
  int top_k;
  int rank, world;
  float scaling;
  void* out;                                              /* bf16 [B,1,Hq,D] (phase 3)              */
  int32_t* sel_idx_out;                                   /* int32 [B*Hkv,top_k] global ids, any order, or NULL */
  void* workspace; size_t workspace_bytes;                /* kvb_sharded_step_workspace_bytes       */
  void* exchange[8]; size_t exchange_bytes;               /* see above                              */
  int phases;
  unsigned wait_polls;
} kvb_sharded_step_params;

size_t kvb_sharded_exchange_bytes(int B, int Hq, int Hkv, int top_k, int world);
size_t kvb_sharded_step_workspace_bytes(int B, int Hq, int Hkv, int t_local, int top_k);
int kvb_exchange_alloc(size_t bytes, int device, void** out_ptr, void* out_handle /* 64 bytes */);
int kvb_exchange_open(const void* handle /* 64 bytes */, int device, void** out_ptr);
int kvb_exchange_close(void* ptr, int device);
int kvb_exchange_free(void* ptr, int device);
int kvb_sharded_decode_step(const kvb_sharded_step_params* p, int device, void* stream);

/* Combine N shard partials [N,B,Hq,D+2] (layout of out_partial above) into bf16 [B,1,Hq,D]:
 * o = sum_r e^{m_r-m} o_r / sum_r e^{m_r-m} l_r, shards with l == 0 ignored. No reference
 * counterpart (the reference has no sequence sharding). */
int kvb_lse_merge(const float* partials, int N, int B, int Hq, int D, void* out,
                  int device, void* stream);

/* ---------------------------------------------------------------------------------------
 * Chunked-prefill block scoring (Tq query tokens at once) and block-level selection.
 *
 * No counterpart in the reference: every QABS path there refuses query_count != 1
 * (EVAL:4006-4007, 4413-4414). The nearest analogs are the decode-only block maximum
 * (EVAL:5036-5046: pad, view(B,H,nblk,blk).amax(-1), topk over blocks) and the block-mean scoring
 * for q_len > 1 in ymluo/projects/qwen3_kcache_avg_topk/src/qwen3_kcache_avg_topk.py:82-103.
 *
 * kvb_quantize_query_tokens: per (b, head, token) int8 codes of the query over the channels of
 *   its KV head: qscale = max(absmax, 2^-24) / 127, code = clamp(rint(q / qscale), -127, 127).
 *   query bf16 [B,Hq,Tq,D] with element strides q_sb/q_sh/q_st; qcode int8 [B,Hq,Tq,C] dense,
 *   qscale fp32 [B,Hq,Tq] dense.
 * kvb_score_prefill_blocks: block_scores[b,g,i,j] = max over the G heads of KV head g and the
 *   tokens t of block j (block_size = 64; the last block may be short) of
 *   (float(sum_c qcode*code) * kscale[b,g,t]) * qscale[b,h,i]; all Tk keys are visible to every
 *   query of the chunk. C in {32,64,128}, G in {1,2,4,8}; packed/scale aligned as for the
 *   streaming decode scorer. block_scores fp32 [B,Hkv,Tq,ceil(Tk/64)] dense; -0 stored as +0.
 *   kvb_score_prefill_blocks_engine is the same with the implementation chosen by the caller
 *   (all give identical bits): 0 = automatic (the tensor-memory path with the fp16 encoding where the
 *   shape allows it), 1 = warp-level int8 MMA, 2 = tcgen05
 *   kind::i8 with int32 accumulators in tensor memory, 3 = tcgen05 kind::f16 with the integer
 *   codes carried exactly as fp16 values and fp32 accumulators.
 * Pre-widened key operands. A chunked prefill scores every chunk of queries against the same keys, so the
 *   int4 -> tensor-core operand conversion can be paid once per cache instead of once per CTA:
 *   kvb_prefill_operand_bytes(B, Hkv, key_capacity, C, engine) is the size of a buffer holding the operands of
 *   key_capacity tokens per (batch, KV head): [B*Hkv][ceil(key_capacity/128)][128*C*es] bytes, es = 2 for
 *   engine 0/3 (fp16 values of the codes), 1 for engine 2 (int8 bytes 16*code); each tile of 128 tokens is
 *   stored in the 8-row x 16-byte core-matrix order the tensor core reads from shared memory, so a CTA
 *   fetches a tile with ONE bulk copy. kvb_widen_keys writes the tiles that hold tokens first_token .. Tk-1
 *   (tokens at or beyond Tk inside the last tile become zero rows); after an append call it again with
 *   first_token = the old Tk. kvb_score_prefill_blocks_widened is kvb_score_prefill_blocks_engine reading
 *   those operands (same engine number as they were widened for); identical bits. operands must be
 *   128-byte aligned. No reference counterpart.
 * kvb_block_topk: per row of block scores ([R,nblk], nblk <= 4096) the min(k,nblk) best blocks
 *   ordered by (score desc, block asc); out_idx int32 [R,kk], out_scores fp32 [R,kk] or NULL.
 * ------------------------------------------------------------------------------------- */
int kvb_quantize_query_tokens(const void* query, int64_t q_sb, int64_t q_sh, int64_t q_st,
                              const int32_t* channel_idx, int8_t* qcode, float* qscale,
                              int B, int Hq, int Hkv, int Tq, int D, int C,
                              int device, void* stream);

int kvb_score_prefill_blocks(const int8_t* qcode, const float* qscale,
                             const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                             const float* scale, int64_t scale_sb, int64_t scale_sh,
                             int B, int Hq, int Hkv, int Tq, int Tk, int C, int block_size,
                             float* block_scores, int device, void* stream);

int kvb_score_prefill_blocks_engine(const int8_t* qcode, const float* qscale,
                                    const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                                    const float* scale, int64_t scale_sb, int64_t scale_sh,
                                    int B, int Hq, int Hkv, int Tq, int Tk, int C, int block_size,
                                    float* block_scores, int engine, int device, void* stream);

size_t kvb_prefill_operand_bytes(int B, int Hkv, int key_capacity, int C, int engine);

int kvb_widen_keys(const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                   int B, int Hkv, int Tk, int key_capacity, int C, int engine, int first_token,
                   void* operands, size_t operand_bytes, int device, void* stream);

int kvb_score_prefill_blocks_widened(const int8_t* qcode, const float* qscale,
                                     const void* operands, size_t operand_bytes, int key_capacity,
                                     const float* scale, int64_t scale_sb, int64_t scale_sh,
                                     int B, int Hq, int Hkv, int Tq, int Tk, int C, int block_size,
                                     float* block_scores, int engine, int device, void* stream);

int kvb_block_topk(const float* block_scores, int64_t row_stride, int64_t R, int nblk, int k,
                   int32_t* out_idx, float* out_scores, int device, void* stream);

/* ---------------------------------------------------------------------------------------
 * The reference's fp32 front-end operators on un-quantised bf16 K, kept for call sites that use them.
 *
 * kvb_qabs_partial_scores replaces partial_scores (QCK:654-656, kernel QCK:98-158) when dim_indices
 *   is NULL — per (batch, head) the dim_count channels with the largest |q| are chosen greedily,
 *   ties to the lower channel (QCK:123-145) — and partial_scores_dim_major (QCK:659-665, kernel
 *   QCK:63-96) when dim_indices int64 [B,H,S] is given. out[b,h,t] = sum_s q[idx_s] * K[t, idx_s]
 *   in fp32 (torch form: EVAL:4443-4446). key is a [B,Hk,T,D] VIEW with element strides
 *   k_sb/k_sh/k_st/k_sd (token-major: k_sd = 1; dim-major storage: k_st = 1); Hk may be the number
 *   of KV heads (head h reads KV head h / (H/Hk)) or H (keys repeated, as the reference passes them).
 *   query [B,H,D] dense, out fp32 [B,H,T] dense. elem_type is the type of query and key elements:
 *   0 = bf16, 1 = fp16, 2 = fp32 (the three types the reference dispatches over, QCK:430-458).
 * kvb_qabs_candidate_full_scores replaces candidate_full_scores (QCK:668-691, kernel QCK:160-216):
 *   out[b,h,t] = scaling * q.k over all D channels where current | previous_candidate |
 *   previous_final (uint8 [B,H,T]; the previous_* may be NULL) or t < protect_sink or
 *   t >= T - protect_recent; -inf elsewhere. key token-major with D contiguous.
 * ------------------------------------------------------------------------------------- */
int kvb_qabs_partial_scores(const void* query, const void* key,
                            int64_t k_sb, int64_t k_sh, int64_t k_st, int64_t k_sd,
                            const int64_t* dim_indices, int dim_count, float* out,
                            int B, int H, int Hk, int T, int D, int elem_type, int device, void* stream);

int kvb_qabs_candidate_full_scores(const void* query, const void* key,
                                   int64_t k_sb, int64_t k_sh, int64_t k_st,
                                   const uint8_t* current, const uint8_t* previous_candidate,
                                   const uint8_t* previous_final, int protect_sink, int protect_recent,
                                   float scaling, float* out,
                                   int B, int H, int Hk, int T, int D, int elem_type, int device, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fused decode step for one layer: quantize-append of the new K row, score, select,
 * final index list, attend — all enqueued on `stream`, nothing else touched.
 * Equivalent to the sequence _qabs_candidate_attention_forward runs (EVAL:4400-4502) with the
 * int4 scorer in place of its fp32 partial score and the group-max select in place of its
 * per-head torch.topk. `key`/`value` hold key_count = history+1 rows (the last row is the
 * token being decoded, EVAL:4421-4425); the packed cache holds rows [0, history) on entry
 * and, when append_self != 0, row `history` on return.
 * ------------------------------------------------------------------------------------- */
typedef struct kvb_decode_step_params {
  const void* query;  int64_t q_sb, q_sh;                 /* bf16 [B,Hq,D]            */
  const void* key;    int64_t k_sb, k_sh, k_st;           /* bf16 [B,Hkv,key_count,D] */
  const void* value;  int64_t v_sb, v_sh, v_st;
  uint8_t* packed;    int64_t packed_sb, packed_sh;       /* int4 cache               */
  float* scale;       int64_t scale_sb, scale_sh;
  const int32_t* channel_idx;                             /* int32 [Hkv,C]            */
  const float* mask;  int64_t mask_sb;                    /* fp32 [B,key_count] or NULL */
  int B, Hq, Hkv, D, C;
  int history_count;                                      /* T; key_count = T + 1 (the upper bound of T when history_count_dev is set) */
  int top_k;
  int protect_sink, protect_recent, keep_self, append_protected;
  int append_self;
  float scaling;
  void* out;                                              /* bf16 [B,1,Hq,D]          */
  int32_t* sel_idx_out;                                   /* int32 [B,Hkv,kk] or NULL */
  void* workspace; size_t workspace_bytes;
  /* Optional device-side history length, for CUDA-graph replays over a growing cache: when not
   * NULL the kernels read T from *history_count_dev (int32, 1 <= T <= history_count; sizes and the
   * workspace are derived from history_count) and, with advance_history != 0, add one to it at the
   * end of the step. Only the streaming configurations support it (C in {32,64,128}, G in
   * {1,2,4,8}, aligned side cache, top_k <= history_count <= 131072); others return KVB_BAD_SHAPE. */
  const int32_t* history_count_dev;
  int advance_history;
  /* Optional: the decoded token's K and V rows, bf16 [B,Hkv,D] dense. When not NULL the step first
   * stores them as row T of `key` / `value` (T from history_count_dev when that is set), which spares
   * a caller inside a graph its own scatter at a device-side position. Both or neither. */
  const void* new_key_row;
  const void* new_value_row;
  /* 0: the selected ids (sel_idx_out, and the order in which the attention walks them) ascend, and the
   * step is reproducible bit for bit. Non-zero: any order — the same exact set, about 3 us less per
   * step at config 2, but the order (and with it the last bits of the fp32 accumulation) varies from
   * run to run. */
  int selected_any_order;
  /* Optional paged K/V. When kv_page_table is not NULL, `key` and `value` are page POOLS, bf16
   * [num_pages, Hkv, kv_page_tokens, D] dense (D = 128), and token t of batch row b lives in page
   * kv_page_table[b * kv_page_table_stride + t / kv_page_tokens] at row t % kv_page_tokens; the strides
   * k_sb .. v_st are ignored. kv_page_tokens is a power of two; the table must cover row history_count (the
   * decoded token's row, which the step reads and, with new_key_row, writes). A pool holds fewer than 2^31
   * rows. The int4 side cache stays contiguous (36 bytes per token at C = 64 against 512 for K and V).
   * No reference counterpart (the reference keeps HF's contiguous cache, EVAL:7278). */
  const int32_t* kv_page_table;
  int64_t kv_page_table_stride;
  int kv_page_tokens;
} kvb_decode_step_params;

size_t kvb_decode_step_workspace_bytes(int B, int Hq, int Hkv, int history_count, int top_k,
                                       int protect_sink, int protect_recent, int keep_self);

int kvb_decode_step(const kvb_decode_step_params* p, int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KVCACHE_B200_H */
