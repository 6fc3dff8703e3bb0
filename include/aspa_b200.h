/*
 * aspa_b200.h — C ABI of libaspa_b200.so: the sm_100a kernels behind the ASPA
 * attention hot path (router, token/head selection, row packing, RoPE +
 * head-major relayout, INT8 per-head quantisation, shortlist planning,
 * gathered attention, prototype EMA, chunk selection and merge).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller unless it is marked
 *     "host"; nothing is allocated or freed inside the library except by the
 *     functions that say so; scratch memory is passed in by the caller;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and is
 *     valid in stream order; no call synchronises the device;
 *   - every function returns 0 on success or a negative ASPA_ERR_* code;
 *     aspa_last_error_string() describes the last failure of the calling thread;
 *   - dtype codes: ASPA_F32 = 0, ASPA_BF16 = 1, ASPA_I8 = 2;
 *   - "bh" means the flattened (batch, head) index b * H + h, "row" means one
 *     active (bh, token) pair; rows are grouped by bh and ascend in token order.
 *
 * Each entry point cites the reference code it replaces, as path:line inside
 * the reference project (aspa.py = src/proteus_attention/models/aspa.py,
 * sa.py = src/proteus_attention/kernels/sparse_attn.py,
 * cs.py = src/proteus_attention/tools/chunked_shortlist.py,
 * cpp = src/proteus_attention/kernels/aspa_cuda/aspa_cuda.cpp).
 */
#ifndef ASPA_B200_H
#define ASPA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ASPA_F32 0
#define ASPA_BF16 1
#define ASPA_I8 2

#define ASPA_OK 0
#define ASPA_ERR_ARG (-1)      /* bad size, dtype or null pointer */
#define ASPA_ERR_UNSUPPORTED (-2)
#define ASPA_ERR_CUDA (-3)     /* a CUDA runtime call failed */
#define ASPA_ERR_TIMEOUT (-4)  /* a bounded device-side wait ran out */

/* Output layouts of the attention kernels. */
#define ASPA_OUT_HEAD_MAJOR 0  /* out[(bh * T + t) * D + d]            (sa.py:1646) */
#define ASPA_OUT_TOKEN_MAJOR 1 /* out[((b * T + t) * H + h) * D + d]   (aspa.py:1806-1807, 1845) */

const char* aspa_last_error_string(void);
int aspa_version(void);

/* Router: gate probabilities, prototype similarity, blend scalar and token
 * importance for n = B*T tokens in one pass over x.
 * Replaces SwitchRouter.forward (aspa.py:149-157), _route_tokens
 * (aspa.py:628-690) and the importance blend (aspa.py:1521-1530).
 *   x            (n, C) of x_dtype (F32 or BF16); w_router (G, C) same dtype
 *   proto_hat    (G, C) fp32 rows of L2-normalised prototypes, or NULL (prototypes off)
 *   conf_eps     (G) fp32 = routing_confidence + 1e-6, or NULL
 *   usage_bias   (G) fp32 = softmax(-(usage+1e-6)), or NULL when usage_boost == 0
 *   gate_probs   (n, G) fp32 out; importance (n) fp32 out;
 *   proto_sim, blend (n) fp32 out, may be NULL when proto_hat is NULL
 *   proto_span   = (float)max(1e-6, 1 - proto_threshold), formed in double on the host like the reference
 *   stat_partials (3 * ceil(n/64)) fp32 scratch/out: per-tile sums of proto_sim, blend and
 *                count(blend > 0); may be NULL
 */
int aspa_router_fwd(const void* x, int x_dtype, int64_t n, int C, const void* w_router, int G,
                    const float* proto_hat, const float* conf_eps, const float* usage_bias,
                    float proto_temp, float proto_threshold, float proto_span, float proto_blend,
                    float usage_boost, float* gate_probs, float* importance, float* proto_sim, float* blend,
                    float* stat_partials, void* stream);

/* The same router on tcgen05 tensor cores for bf16 activations: persistent CTAs, 128-token tiles, TMA-staged
 * operands, double-buffered accumulator in tensor memory.  Results as aspa_router_fwd (fp32 accumulation order
 * differs).  stat_partials here holds 3 * ceil(n/32) entries (one partial per 32 tokens).
 *   aspa_router_tc_scratch_bytes: bytes of 16-byte aligned scratch the call needs, or 0 when the shape is
 *     not supported (needs C % 64 == 0, G % 4 == 0, 4*G <= 128 with prototypes, G <= 128 without);
 *   n >= 128; status (1) int32, zeroed by the caller: set non-zero if a bounded device-side wait ran out
 *     (the outputs are then invalid). */
int64_t aspa_router_tc_scratch_bytes(int C, int G, int has_proto);
int aspa_router_fwd_tc(const void* x, int64_t n, int C, const void* w_router, int G, const float* proto_hat,
                       const float* conf_eps, const float* usage_bias, float proto_temp, float proto_threshold,
                       float proto_span, float proto_blend, float usage_boost, float* gate_probs,
                       float* importance, float* proto_sim, float* blend, float* stat_partials, void* scratch,
                       int32_t* status, void* stream);

/* Read (and with reset != 0 clear) the status word a device-side bounded wait raises.  Synchronises `stream`.
 * Returns ASPA_OK when the word is zero, else ASPA_ERR_TIMEOUT with aspa_last_error_string() naming the wait that
 * ran out; the outputs of the call that raised it are invalid.  The reference has no device-side waits; its
 * counterpart is the RuntimeWarning + fallback around a failed native launch (sa.py:1524-1525), which this
 * implementation turns into an error because it has no fallback. */
int aspa_read_status(int32_t* status, int reset, void* stream);

/* aspa_router_fwd_tc with the two knobs a test needs to see a bounded wait run out without faulting the device:
 * `spin_limit` (>= 1024) replaces the built-in iteration limit of every wait, and the producer skips the copy of the
 * first k-block of tile `withhold_tile` (-1: none), so the consumers of that stage give up, the kernel frees its
 * tensor memory and returns with *status != 0.  Fixed prototype parameters (temp 0.3, threshold 0.2, blend 0.5),
 * no usage bias, no statistics.  No counterpart in the reference. */
int aspa_router_fwd_tc_probe(const void* x, int64_t n, int C, const void* w_router, int G, const float* proto_hat,
                             const float* conf_eps, float* gate_probs, float* importance, float* proto_sim,
                             float* blend, void* scratch, int32_t* status, uint32_t spin_limit, int64_t withhold_tile,
                             void* stream);

/* L2-normalise the G prototype rows (F.normalize(..., eps=1e-6), aspa.py:639-640). */
int aspa_normalize_rows(const float* src, int rows, int cols, float eps, float* dst, void* stream);

/* Token keep: per batch row, mark the `need` most important tokens (ties to the
 * lowest index), everything >= threshold when threshold > 0, and the first
 * `guard` tokens.  Replaces _select_active_tokens (aspa.py:790-842).
 *   importance (B, T) fp32; token_mask (B, T) uint8 out; kept (B) int32 out.  */
int aspa_token_select(const float* importance, int B, int T, int need, float threshold, int guard,
                      uint8_t* token_mask, int32_t* kept, void* stream);

/* Token keep plus the ordered list of kept tokens in one launch (no reference counterpart: the reference indexes
 * with the boolean mask, aspa.py:1715-1721).  Batch row b owns slots [b*slots_per_row, (b+1)*slots_per_row):
 *   kept_idx (B*slots_per_row) int64: flat index b*T + t of the kept tokens of row b, ascending, padded with -1;
 *   slot_of (B*T) int32: slot of every kept token (entries of dropped tokens are left unwritten).
 * Kept tokens beyond slots_per_row are dropped from kept_idx (kept[] still counts them).  T <= ASPA_TOKEN_COMPACT_MAX_T. */
#define ASPA_TOKEN_COMPACT_MAX_T 65536
int aspa_token_select_compact(const float* importance, int B, int T, int need, float threshold, int guard,
                              uint8_t* token_mask, int32_t* kept, int64_t* kept_idx, int32_t* slot_of,
                              int slots_per_row, void* stream);

/* Column sums of gate_probs mapped to heads, then the nucleus head count and the
 * blended per-token head budget, all on the device.
 * Replaces _nucleus_head_count (aspa.py:749-780) and the budget blend (aspa.py:1575-1586).
 *   gate_probs (n, G); gate_to_head (G) int32; scratch: (H * ceil(n/1024)) fp32
 *   k_out (2) int32 out: [0] = heads per token (topk), [1] = adaptive (nucleus) budget */
int aspa_head_budget(const float* gate_probs, int64_t n, int G, const int32_t* gate_to_head, int H,
                     double top_p, int dense_k, int h_active_min, int linear_head_k, double alpha,
                     float* scratch, int32_t* k_out, void* stream);

/* Per-token top-k heads (ties to the lowest head) and the (B,T) x H activity bit
 * mask ANDed with the token mask.  Replaces aspa.py:1540-1542, 1590-1598.
 *   k_dev: device int32 holding k, or NULL to use k_host; kmax = row width of the outputs
 *   head_bits (n) uint64 out; top_idx (n, kmax) int32 out; top_score (n, kmax) fp32 out
 *   stat_partials (2 * ceil(n/256)) fp32 out: per-block sum of selected scores and
 *   sum of gate entropy; may be NULL */
int aspa_head_select(const float* gate_probs, int64_t n, int G, const int32_t* gate_to_head, int H,
                     int k_host, const int32_t* k_dev, int kmax, const uint8_t* token_mask,
                     uint64_t* head_bits, int32_t* top_idx, float* top_score, float* stat_partials,
                     void* stream);

/* Row packing: (bh, token) rows grouped by bh, tokens ascending.
 * Replaces _pack_active_rows (sa.py:924-947; cpp:47-75).
 *   head_bits (B*T) uint64; row_offsets (B*H + 1) int32 out; token_idx (capacity) int32 out
 *   seg_scratch: (B*H * ceil(T/256) + 1) int32 scratch
 *   Returns the scratch size in int32 elements from aspa_pack_rows_scratch(). */
int64_t aspa_pack_rows_scratch(int B, int H, int T);
int aspa_pack_rows(const uint64_t* head_bits, int B, int T, int H, int32_t* seg_scratch,
                   int32_t* row_offsets, int32_t* token_idx, int64_t capacity, void* stream);

/* aspa_head_select followed by aspa_pack_rows in fewer launches: when T is a multiple of 256 the head choice
 * counts the rows of every (head, 256-token segment) itself, which is the first phase of the packing.
 * gate_probs (B*T, G); the other arguments as in the two separate calls. */
int aspa_head_select_pack(const float* gate_probs, int B, int T, int G, const int32_t* gate_to_head, int H, int k_host,
                          const int32_t* k_dev, int kmax, const uint8_t* token_mask, uint64_t* head_bits,
                          int32_t* top_idx, float* top_score, float* stat_partials, int32_t* seg_scratch,
                          int32_t* row_offsets, int32_t* token_idx, int64_t capacity, void* stream);

/* aspa_pack_rows for callers that cannot provide scratch memory.  It has no counterpart in the
 * reference: it exists for hosts that must not allocate at call time — a serving loop whose device
 * arena was sized once at start-up and which bans allocator calls on the request path (they may
 * synchronise the device or fragment the arena), or a foreign-language binding with no CUDA allocator
 * that only forwards the input and output buffers it was given.  The segment-count scratch lives in a
 * fixed array inside the library: aspa_pack_rows_static_capacity() int32 entries (1 MiB) on every GPU
 * that loads the library, until the process exits.  Same inputs, outputs and results as aspa_pack_rows.
 *   - B*H*ceil(T/256) + 1 must not exceed the capacity; larger problems are rejected with ASPA_ERR_ARG
 *     and a message (use aspa_pack_rows then);
 *   - no cudaMalloc, cudaFree or other allocating call is made; the first call on each device looks up
 *     the array's device address (cudaGetSymbolAddress with that device current) — make that first
 *     call before any stream capture;
 *   - all calls share the one array, which keeps whatever the previous call left in it (nothing in it
 *     needs to start at zero); two calls that overlap on the GPU (different streams, or different
 *     threads on one device) race on it, so serialise them. */
int64_t aspa_pack_rows_static_capacity(void);
int aspa_pack_rows_static(const uint64_t* head_bits, int B, int T, int H, int32_t* row_offsets,
                          int32_t* token_idx, int64_t capacity, void* stream);

/* Pack a (heads, T) uint8 activity mask (the functional API's active_mask). */
int aspa_pack_mask(const uint8_t* mask, int heads, int T, int32_t* seg_scratch, int32_t* row_offsets,
                   int32_t* token_idx, int64_t capacity, void* stream);

/* RoPE tables: cos/sin (T, D/2) fp32 holding values rounded to `dtype`
 * (aspa.py:576-604).  inv_freq (D/2) fp32 comes from the host so that it is
 * bit-identical to the reference's buffer (aspa.py:241-246). */
int aspa_rope_table(const float* inv_freq, int T, int D, int dtype, float* cos_t, float* sin_t, void* stream);

/* RoPE on q,k + split of the fused QKV projection into head-major q,k,v.
 * Replaces _apply_rope_embedding (aspa.py:606-618) and the permutes (aspa.py:1644-1656).
 *   qkv (B, T, 3*H*D) of dtype; q,k,v (B*H, T, D) same dtype out
 *   cos_t/sin_t NULL = no rotation; amax (3, B*H) fp32 in/out or NULL: running max |.| of q,k,v
 *   per bh (caller zeroes it), feeding the INT8 quantiser.
 *   q_keep (B, T) uint8 or NULL: when given, the query rows of tokens with q_keep == 0 are skipped (their q is
 *   left unwritten); only tokens that survive the token keep ever act as queries (aspa.py:1594-1598). */
int aspa_rope_relayout(const void* qkv, int dtype, int B, int T, int H, int D, const float* cos_t,
                       const float* sin_t, void* q, void* k, void* v, float* amax, const uint8_t* q_keep,
                       void* stream);

/* The same work for a projection that was split in two so that queries are only computed for kept tokens
 * (no reference counterpart: the reference projects q for every token, aspa.py:1641):
 *   aspa_rope_relayout_kv: kv (B, T, 2*H*D) -> k (rotated), v, both (B*H, T, D);
 *   aspa_rope_rows_q: q_rows (max_rows, H*D), row i belonging to token kept_idx[i] (flat b*T + t; rows with
 *   i >= *count_dev or an index outside [0, B*T) are skipped) -> rotated into q (B*H, T, D). */
int aspa_rope_relayout_kv(const void* kv, int dtype, int B, int T, int H, int D, const float* cos_t,
                          const float* sin_t, void* k, void* v, void* stream);
/* RoPE in place on rows that stay where the projection wrote them: x points at the first row, rows are H*D wide
 * and `row_stride` elements apart, row r belongs to position r % T. */
int aspa_rope_inplace(void* x, int dtype, int64_t n_rows, int T, int64_t row_stride, int H, int D, const float* cos_t,
                      const float* sin_t, void* stream);
/* The same rotation written head-major: heads_out is (n_rows / T * H, T, D), x is left as it was (NULL heads_out:
 * in place).  Keys of one head at consecutive positions end up contiguous, which is what a window of keys wants. */
int aspa_rope_rows_to_heads(void* x, int dtype, int64_t n_rows, int T, int64_t row_stride, int H, int D,
                            const float* cos_t, const float* sin_t, void* heads_out, void* stream);
int aspa_rope_rows_q(const void* q_rows, int dtype, const int64_t* kept_idx, const int32_t* count_dev,
                     int64_t max_rows, int B, int T, int H, int D, const float* cos_t, const float* sin_t, void* q,
                     void* stream);

/* RoPE + head-major split + symmetric per-head INT8 in two passes over the fused bf16 projection (the first pass
 * only takes the per-head amax of the rotated values): same results as aspa_rope_relayout followed by
 * aspa_quantize_int8 on q, k and v, without the bf16 head-major intermediates (aspa.py:1312-1363, 1644-1656).
 *   qkv (B, T, 3*H*D) bf16; q8, k8, v8 (B*H, T, D) int8 out; amax, scales (3, B*H) fp32 out. */
int aspa_rope_quantize(const void* qkv, int B, int T, int H, int D, const float* cos_t, const float* sin_t,
                       int8_t* q8, int8_t* k8, int8_t* v8, float* amax, float* scales, void* stream);

/* max |x| per head of a (heads, T*D) tensor (aspa.py:1328). amax is overwritten. */
int aspa_head_amax(const void* x, int dtype, int heads, int64_t per_head, float* amax, void* stream);

/* Per-head quantile of |x| for the percentile modes of the quantiser (aspa.py:1330-1338): base[h] =
 * torch.quantile(|x_h|, q) with linear interpolation between the two neighbouring order statistics (rank = q*(n-1)
 * evaluated in float32, as torch does), replaced by amax[h] where it is not positive.  Exact order statistics by a
 * four-pass radix select.  x (heads, per_head) F32 or BF16; 0 < q <= 1; amax from aspa_head_amax; scratch of
 * aspa_head_abs_quantile_scratch(heads) bytes; base (heads) fp32 out, usable as the `amax` of aspa_quantize_int8. */
int64_t aspa_head_abs_quantile_scratch(int heads);
int aspa_head_abs_quantile(const void* x, int dtype, int heads, int64_t per_head, double q, const float* amax,
                           void* scratch, float* base, void* stream);

/* Symmetric per-head INT8: scale = max(amax/127, 1e-6); q = clamp(rint(x/scale), +-127).
 * Replaces _quantize_per_head_int8 (aspa.py:1312-1363); `amax` is the per-head base of whichever mode: the maximum,
 * the percentile of aspa_head_abs_quantile, or its running average. */
int aspa_quantize_int8(const void* x, int dtype, int heads, int64_t per_head, const float* amax,
                       int8_t* out, float* scales, void* stream);

/* Structural description of every row's candidate set (sa.py:457-596 without
 * materialising the (N, L) table).  Row t attends to
 *   - local:   keys max(0, t-window+1) .. t      (window == 0: only t itself)
 *   - anchors: max(t - j*anchor_stride, 0), j = 1..anchor_slots
 *   - proto:   the min(t+1, proto_cap) best prototype scores among keys <= t
 * de-duplicated.  The caller guarantees window + anchor_slots + proto_cap <= L,
 * so the reference's "keep the L smallest" cut never triggers. */
typedef struct {
  int32_t window;
  int32_t anchor_slots;
  int32_t anchor_stride;
  int32_t proto_cap;          /* 0 = no prototype piece */
  int32_t proto_block;        /* tokens per plan block (128) */
  int32_t proto_list_stride;  /* int32 entries per block list = proto_cap + proto_block */
  const int32_t* proto_lists; /* (B, nblk, proto_list_stride): key ids, best first, -1 padded */
  const int32_t* proto_limit; /* (B, T): per token, number of leading list entries to scan */
} aspa_shortlist_plan;

/* Build proto_lists / proto_limit from per-token prototype scores (B, T).
 * Replaces _shortlist_prepare_proto_candidates[_grouped] (sa.py:260-373): block-wise prefix top-k.
 *   scratch bytes from aspa_proto_plan_scratch(). */
int64_t aspa_proto_plan_scratch(int B, int T, int proto_cap);
int aspa_proto_plan(const float* proto_scores, int B, int T, int proto_cap, void* scratch,
                    int32_t* proto_lists, int32_t* proto_limit, void* stream);

/* Explicit candidate table, exactly as build_packed_shortlist_candidates returns it
 * (sa.py:457-596): (N, L) int64 ascending unique ids padded with the row id, and lengths (N) int64.
 *   rows (N) int64; row_batch (N) int64 or NULL; proto_scores (Bp, seq_len) fp32 or NULL
 *   caps < 0 mean "not given" (the reference's None).  */
int aspa_build_candidates(const int64_t* rows, const int64_t* row_batch, int64_t N, int seq_len, int L,
                          int linear_window, int anchor_stride, int use_local, int use_anchors,
                          const float* proto_scores, int local_cap, int anchor_cap, int proto_cap,
                          int64_t* cand_out, int64_t* len_out, void* stream);

/* Attention over packed rows.  One call covers the three shapes of the
 * reference op (aspa_sparse_attention, sa.py:1373-1646; _fallback_sparse_attention
 * sa.py:950-1046; Triton kernel sa.py:597-919; cpp:118-343):
 *   - cand != NULL: explicit (N, L) candidate table + lengths;
 *   - plan != NULL: candidates generated on the fly from the structural plan;
 *   - neither: every key 0..t (or 0..max token of the head when add_mask is given).
 * q,k,v (heads, T, D) of qkv_dtype (F32, BF16 or I8 with per-head fp32 scales);
 * add_mask optional (T, T) fp32 additive mask (sa.py:997-1000, 1018-1021);
 * out of out_dtype in out_layout; rows of inactive (bh, token) pairs are NOT
 * written — the caller zero-fills `out` first.  H is only used by the
 * token-major layout.  max_rows = largest per-head row count (grid sizing).
 * workspace: aspa_attn_workspace_bytes(total_rows, D) bytes (partial softmax
 * state exchanged between the window pass and the extras pass). */
int64_t aspa_attn_workspace_bytes(int64_t total_rows, int D);
int aspa_gather_attn_fwd(const void* q, const void* k, const void* v, int qkv_dtype, const float* q_scale,
                         const float* k_scale, const float* v_scale, int heads, int T, int D, int H,
                         const int32_t* row_offsets, const int32_t* token_idx, int max_rows,
                         int64_t total_rows, const int64_t* cand, const int64_t* cand_len, int L,
                         const aspa_shortlist_plan* plan, const float* add_mask, void* out, int out_dtype,
                         int out_layout, void* workspace, void* stream);

/* Element strides of k and v: row of (batch b, head h, token t) starts at b*batch + h*head + t*token.
 * Head-major (heads, T, D) is {H*T*D, T*D, D}; the k half of a fused (B, T, 2, H, D) projection is
 * {T*2*H*D, D, 2*H*D}.  Every row start must stay 16-byte aligned. */
typedef struct aspa_kv_layout {
  int64_t k_batch, k_head, k_token;
  int64_t v_batch, v_head, v_token;
} aspa_kv_layout;

/* aspa_gather_attn_fwd with two extras (no reference counterpart for either):
 *   out_row_map (B*T) int32 or NULL: row b*T + t of the token-major `out` becomes row out_row_map[b*T + t]
 *   (the compact slot of a kept token, from aspa_compact_mask), so that the output projection runs over kept
 *   tokens only — the reference projects every row, dropped tokens included (aspa.py:1854);
 *   kv_layout or NULL: k and v read where the projection left them instead of from head-major copies (the
 *   reference permutes them, aspa.py:1644-1656).  Needs H > 0;
 *   regroup_ws or NULL: scratch of aspa_attn_regroup_bytes() bytes.  With it, and enough rows per (head,
 *   token % anchor_stride) group, the strided anchor keys t - j*stride of a plan run as a third tile pass over the
 *   rows regrouped by residue class (the anchors of one class are a window over K[rho + stride*i]); without it they
 *   are gathered row by row. */
int aspa_gather_attn_fwd_ex(const void* q, const void* k, const void* v, int qkv_dtype, const float* q_scale,
                            const float* k_scale, const float* v_scale, int heads, int T, int D, int H,
                            const int32_t* row_offsets, const int32_t* token_idx, int max_rows,
                            int64_t total_rows, const int64_t* cand, const int64_t* cand_len, int L,
                            const aspa_shortlist_plan* plan, const float* add_mask, void* out, int out_dtype,
                            int out_layout, const int32_t* out_row_map, const aspa_kv_layout* kv_layout,
                            void* workspace, void* regroup_ws, void* stream);
/* The same call with the regrouping of its anchor tile pass done ahead of time: aspa_attn_regroup_rows depends on the
 * packed rows and the plan only, not on q, k, v, so a caller whose projection is still running on another stream can
 * issue it before waiting for that stream.  It fills regroup_ws and sets *prepared (host int) to 1 when the call below,
 * given the same arguments, will take the anchor tile pass; regroup_prepared passes that flag on.  No reference
 * counterpart. */
int aspa_attn_regroup_rows(int qkv_dtype, int heads, int T, int D, const int32_t* row_offsets, const int32_t* token_idx,
                           int64_t total_rows, const aspa_shortlist_plan* plan, void* regroup_ws, int32_t* prepared,
                           void* stream);
int aspa_gather_attn_fwd_prepared(const void* q, const void* k, const void* v, int qkv_dtype, const float* q_scale,
                                  const float* k_scale, const float* v_scale, int heads, int T, int D, int H,
                                  const int32_t* row_offsets, const int32_t* token_idx, int max_rows, int64_t total_rows,
                                  const int64_t* cand, const int64_t* cand_len, int L, const aspa_shortlist_plan* plan,
                                  const float* add_mask, void* out, int out_dtype, int out_layout,
                                  const int32_t* out_row_map, const aspa_kv_layout* kv_layout, void* workspace,
                                  void* regroup_ws, int regroup_prepared, void* stream);
/* Tile kernel of the window passes (head_dim 64, bf16 or int8).  Two kernels replace the Triton kernel's tiled
 * products (sa.py:597-919): a tcgen05 / tensor-memory kernel on 128-row x 128-key tiles and a warp-MMA kernel on
 * 16-row groups for rows too sparse to fill 128-row tiles.  aspa_attn_tc_mode selects: 0 never the tcgen05 kernel,
 * 1 (default) when window >= 64 * mean token gap between the rows of a head, 2 whenever the shape allows; returns the
 * previous mode (any other argument only queries).  aspa_attn_tc_status reads (reset != 0: and clears) the word a
 * bounded device-side wait of the tcgen05 kernel raises: ASPA_OK, or ASPA_ERR_TIMEOUT when a wait ran out since
 * the last reset (outputs of that call are invalid).  Synchronises `stream`. */
int aspa_attn_tc_mode(int mode);
/* Passes that follow the window tiles of a structural plan (the candidate pieces of sa.py:260-596), on warp-MMA tiles
 * where rows share their keys (int8 or bf16 q/k/v, head_dim 64):
 *  - prototype picks: the rows of one (head, 128-token block) pair walk the same score-sorted list of
 *    aspa_proto_plan, so a warp takes the pair with up to 16 rows as the M dimension of mma.sync tiles (s8 x s8 for
 *    Q K^T of int8 inputs, f16 / bf16 for P V) and reads each key and value row once for all of them;
 *  - anchors of (head, token % stride) groups too small for the 64-row tile pass: the same kernel over the strided key
 *    sequence of the residue class, the slot that clamps to key 0 included;
 *  - when the 64-row tile passes took window and anchors and the plan has no picks, a one-warp-per-row finaliser for the
 *    clamping slot and the normalisation.
 * mode 0: always the per-row kernel; 1 (default): these kernels where they apply.  Returns the previous mode (any
 * other argument only queries).  The environment variable ASPA_ATTN_PICKS_MODE sets it when the Python binding loads
 * the library. */
int aspa_attn_picks_mode(int mode);
int aspa_attn_tc_status(int reset, void* stream);

/* Bytes of regroup_ws for the call above (0 when the plan has no anchors). */
int64_t aspa_attn_regroup_bytes(int64_t total_rows, int heads, int anchor_stride);

/* Prototype EMA (aspa.py:692-718): counts = sum_t probs; mean = probs^T x / counts;
 * prototypes, usage and confidence updated in place for gates with counts > 1e-6.
 *   scratch: aspa_proto_ema_scratch() bytes. Returns via updated (1) int32 the number of gates touched. */
int64_t aspa_proto_ema_scratch(int64_t n, int C, int G);
int aspa_proto_ema_update(const void* x, int x_dtype, int64_t n, int C, const float* gate_probs, int G,
                          double decay, float* prototypes, float* usage, float* confidence, void* scratch,
                          int32_t* updated, void* stream);

/* Chunk promotion (cs.py:140-208): softmax mass over masked importance, nucleus
 * count, top-`budget` tokens.  One chunk per call.
 *   importance (T) fp32, token_mask (T) uint8 or NULL, offset added to indices
 *   out_scores (budget) fp32, out_idx (budget) int64, out_count (1) int32 — count valid entries,
 *   in score-descending order (ties by index). */
int aspa_chunk_select(const float* importance, const uint8_t* token_mask, int T, int budget, float top_p,
                      int64_t offset, float* out_scores, int64_t* out_idx, int32_t* out_count, void* stream);

/* The same promotion with the record slot read from device memory: the results go to rec_scores / rec_idx
 * (n_slots, budget) and rec_count (n_slots) at slot *slot_dev, and slot_offsets[*slot_dev] is added to the
 * indices.  One captured launch (a CUDA-graph node) can thus serve every chunk of a pass; the caller only rewrites
 * *slot_dev between replays.  T <= 65536. */
int aspa_chunk_select_slot(const float* importance, const uint8_t* token_mask, int T, int budget, float top_p,
                           const int32_t* slot_dev, const int64_t* slot_offsets, float* rec_scores, int64_t* rec_idx,
                           int32_t* rec_count, void* stream);

/* Merge of all chunks' promotions (cs.py:211-254): one representative score per
 * unique index (the lowest, as the reference's sort key does), the max_tokens
 * best of them, ascending index order.
 *   scores/indices (n): entries with index < 0 are ignored; seq_len bounds the indices
 *   table: scratch of aspa_merge_finalise_scratch(seq_len) bytes, 16-byte aligned; keep_idx (max_tokens) int64,
 *   padded with seq_len beyond keep_count when n <= ASPA_MERGE_POS_MAX; keep_scores (max_tokens) fp32,
 *   keep_count (1) int32 out.  keep_pos (max_tokens) int64 or NULL: position in scores/indices of the
 *   entry that represents each kept index (lets the caller fetch rows it stored per candidate instead of going
 *   back to the sequence); only available for n <= ASPA_MERGE_POS_MAX. */
#define ASPA_MERGE_POS_MAX 65536
int64_t aspa_merge_finalise_scratch(int64_t seq_len);
int aspa_merge_finalise(const float* scores, const int64_t* indices, int64_t n, int64_t seq_len,
                        int max_tokens, void* table, int64_t* keep_idx, float* keep_scores, int64_t* keep_pos,
                        int32_t* keep_count, void* stream);

/* Gather rows src[idx[i], :] -> dst[i, :] (cs.py:688-689); a negative index gives a row of zeros; rows
 * i >= *count_dev (when count_dev is given) are left untouched.  row_bytes multiple of 16. */
int aspa_gather_rows(const void* src, const int64_t* idx, const int32_t* count_dev, int64_t max_rows,
                     int64_t row_bytes, void* dst, void* stream);

/* Ordered compaction of a byte mask (n): kept_idx (capacity) int64 gets the indices i with mask[i] != 0 in
 * ascending order, padded with n; slot_of (n) int32 gets the position of every kept index in kept_idx (entries of
 * dropped indices are left unwritten; slot_of may be NULL); count (1) int32 the number kept.  Indices beyond `capacity` are dropped
 * (count still reports all of them).  scratch: aspa_compact_mask_scratch(n) bytes.  No reference counterpart
 * (the reference uses boolean indexing, aspa.py:1715-1721). */
int64_t aspa_compact_mask_scratch(int64_t n);
int aspa_compact_mask(const uint8_t* mask, int64_t n, int64_t capacity, int64_t* kept_idx, int32_t* slot_of,
                      int32_t* count, void* scratch, void* stream);

/* dst (n, row_bytes): row i = src[slot_of[i]] where mask[i] != 0, else `fill` (one row of row_bytes, NULL =
 * zeros).  Rebuilds a full-length result from rows computed for kept tokens only; with fill = the projection
 * bias it equals projecting an all-zero row (aspa.py:1854).  row_bytes multiple of 16. */
int aspa_scatter_rows_fill(const void* src, const int32_t* slot_of, const uint8_t* mask, const void* fill, int64_t n,
                           int64_t row_bytes, void* dst, void* stream);

/* One fp64 record of a layer call for a single device-to-host copy (the reference reads these values with
 * some twenty .item() calls, aspa.py:1560-1640, 1856-1916):
 *   [row_offsets (n_offsets) | kept (n_kept) | k, adaptive k | selected-score sum, entropy sum |
 *    prototype similarity sum, blend sum, blended-token count | router status]
 * kept NULL -> kept_fill; k_dev NULL -> k_fill (both entries); head_partials (2 * head_blocks) and
 * proto_partials (3 * proto_blocks, may be NULL -> zeros) are the per-block partial sums written by
 * aspa_head_select and the router; status (1) int32 or NULL.  record: n_offsets + n_kept + 8 doubles. */
int aspa_stats_record(const int32_t* row_offsets, int n_offsets, const int32_t* kept, int n_kept, double kept_fill,
                      const int32_t* k_dev, double k_fill, const float* head_partials, int64_t head_blocks,
                      const float* proto_partials, int64_t proto_blocks, const int32_t* status, double* record,
                      void* stream);

/* Deterministic sum of per-block partials: out[j] = sum_i partials[j * n_blocks + i]. */
int aspa_reduce_partials(const float* partials, int n_series, int64_t n_blocks, float* out, void* stream);

/* Key/value memory bank (reference models/aspa.py:932-969, _update_memory_bank).  mem_keys / mem_values (H, slots, D),
 * mem_counts (H, slots) fp32 and mem_ptr (H) int64 are the layer's buffers.  For every (batch, head) pair with packed
 * rows, in batch order per head: the head's bank is multiplied by `decay`, the mean key and mean value over the
 * pair's rows (k, v of dtype `dtype`, read through kv_layout or head-major (B*H, T, D) when NULL) go into the slot under
 * the ring pointer with the row count beside them, and the pointer advances.  decay >= 1 writes nothing, as the
 * reference does.  head_dim <= 256. */
int aspa_memory_update(const void* k, const void* v, int dtype, const aspa_kv_layout* kv_layout, int B, int H, int T,
                       int D, const int32_t* row_offsets, const int32_t* token_idx, float decay, float* mem_keys,
                       float* mem_values, float* mem_counts, int64_t* mem_ptr, int slots, void* stream);
/* INT8 side of _prepare_memory_candidates (aspa.py:971-1013, 1262-1272): the reference quantises k and v with the
 * ring appended, so the per-head amax covers the appended rows (the first c rows of the ring read from the pointer on,
 * c = slots with a positive count, values rounded to `dtype`).  Folds that into amax_k / amax_v (B*H) for the pairs
 * that have packed rows.  The appended rows never reach the attention: the candidate builder clamps their ids onto
 * the row's own token (sa.py:570-571). */
int aspa_memory_fold_amax(const float* mem_keys, const float* mem_values, const float* mem_counts,
                          const int64_t* mem_ptr, int B, int H, int slots, int D, int dtype,
                          const int32_t* row_offsets, float* amax_k, float* amax_v, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ASPA_B200_H */
