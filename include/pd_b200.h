/* C ABI of the B200 paged split-KV flash-decoding engine (libpd_b200.so).
 *
 * This is the drop-in boundary for the decode hot path of emaanh/paged-attention.
 * The reference exposes that path only as C++ (namespace decode::); every entry
 * point here names the C++ declaration it stands in for, by the file's path in
 * the reference project.  Plain pointers and sizes only; all device pointers are
 * CUDA device pointers of the current device; `stream` is a cudaStream_t passed
 * as void* (NULL = default stream).
 *
 * Error model: every function that can fail returns a pd_status.  Nothing here
 * aborts the process, throws across the boundary or traps on the device.  The
 * message of the calling thread's last failure is pd_last_error().  The C++
 * wrappers (paged_attention_b200/include) turn PD_INVALID_ARGUMENT into
 * std::invalid_argument and PD_LENGTH_ERROR into std::length_error, as the
 * reference throws them.
 *
 * Threading: as in the reference, one host thread drives one cache / plan at a
 * time; objects carry no locks.  One-time kernel configuration is thread-safe.
 */
#ifndef PD_B200_H
#define PD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pd_status {
    PD_OK               = 0,
    PD_INVALID_ARGUMENT = 1,  /* std::invalid_argument in the reference */
    PD_LENGTH_ERROR     = 2,  /* std::length_error in the reference */
    PD_CUDA_ERROR       = 3,  /* the reference prints and abort()s (include/cuda_check.hpp:9-17) */
    PD_OUT_OF_PAGES     = 4,  /* append returned false in the reference */
    PD_KERNEL_TIMEOUT   = 5,  /* a bounded device-side wait expired; see pd_kernel_status */
    PD_INTERNAL         = 6
} pd_status;

/* decode::KVDtype (src/decode/decode_types.hpp:8) */
typedef enum pd_kv_dtype { PD_FP16 = 0, PD_FP8_E4M3 = 1 } pd_kv_dtype;

/* decode::DecodeParams (src/decode/decode_types.hpp:14-45), field for field and
 * in the same order, so a decode::DecodeParams can be passed as a pd_params. */
typedef struct pd_params {
    const void* q;              /* half [batch][num_q_heads][head_dim] */
    void*       out;            /* half [batch][num_q_heads][head_dim] */
    const void* k_cache;        /* [num_pages][num_kv_heads][page_size][head_dim], fp16 or e4m3 */
    const void* v_cache;
    const int*  block_table;    /* [num_slots][block_table_stride] physical page ids */
    const int*  seq_lens;       /* [num_slots] */
    const int*  slot_ids;       /* [batch] cache slot per batch row; NULL = identity */
    int         block_table_stride;
    int         batch;
    int         num_q_heads;
    int         num_kv_heads;
    int         head_dim;
    int         page_size;
    float       sm_scale;
    float       k_scale;
    float       v_scale;
    const void* segments;       /* int4 (row, kv head, token begin, token end) per segment */
    const int*  cta_seg_begin;  /* [num_ctas + 1] */
    const int*  item_seg_begin; /* [batch * num_kv_heads + 1] */
    int         num_ctas;
    int         needs_merge;
    float*      partial_out;    /* [num_segments][group][head_dim] */
    float*      partial_lse;    /* [num_segments][group] */
} pd_params;

/* PagedKVCache::Config (src/decode/paged_kv_cache.hpp:19-29) */
typedef struct pd_cache_config {
    int   num_pages;
    int   page_size;
    int   num_kv_heads;
    int   head_dim;
    int   max_slots;
    int   max_pages_per_slot;
    int   dtype;      /* pd_kv_dtype */
    float k_scale;    /* stored = value / scale (FP8 only) */
    float v_scale;
} pd_cache_config;

typedef struct pd_plan        pd_plan;         /* decode::DecodePlan  (src/decode/decode.hpp:21-27) */
typedef struct pd_device_plan pd_device_plan;  /* decode::DevicePlan  (src/decode/decode.hpp:44-62) */
typedef struct pd_cache       pd_cache;        /* decode::PagedKVCache (src/decode/paged_kv_cache.hpp:17-93) */

/* Message of this thread's most recent failure ("" if none). */
const char* pd_last_error(void);
/* Library version string. */
const char* pd_version(void);

/* kv_dtype_bytes / kv_dtype_name (src/decode/decode_types.hpp:10-11) */
int         pd_kv_dtype_bytes(int dtype);
const char* pd_kv_dtype_name(int dtype);

/* decode::tile_tokens / wave_ctas / default_ctas (src/decode/decode.hpp:30-35).
 * tile_tokens needs no GPU; the other two query the current device. */
int pd_tile_tokens(int dtype, int head_dim, int group, int* out);
int pd_wave_ctas(int dtype, int head_dim, int group, int* out);
int pd_default_ctas(int dtype, int head_dim, int group, int* out);

/* Tuning knob without a counterpart in the reference.  Layers with exactly 8 kv heads whose plan came from
 * pd_make_plan (directly or through the cache) normally run the "head-fused" schedule: the device plan also
 * carries the step cut by rows, a tile is 16 tokens (fp16 cache) or 32 tokens (e4m3 cache) of all 8 kv heads
 * (one 32 KB / 16 KB box per page and pool instead of eight boxes fetched by different CTAs at different
 * times), one consumer warp per kv head, no cross-warp merge.  The plan object and pd_params keep the
 * reference's (row, kv head) format either way.  Modes: 0 never (environment PD_B200_NO_HEAD_FUSED=1 also
 * selects it); 1, the default, where it wins: steps whose rows are cut in at most 4 pieces each over the
 * one-CTA-per-SM grid (batches of about 64 rows and more; with fewer rows every row is spread over dozens of
 * CTAs and the (row, kv head) schedule, which has 8 times as many work items, is faster); 2 whenever the
 * layer allows it (used by tests).  Takes effect at the next decode call. */
int pd_set_head_fused(int mode);
int pd_head_fused(void);
/* Second knob without a counterpart in the reference: the adaptive cut.  SMs of one GPU do not stream at
 * the same rate, and CTA c of a grid always runs on the same SM, so with the planner's equal shares the
 * slower SMs finish tens of microseconds after the others.  While this is on (default; environment
 * PD_B200_NO_ADAPTIVE=1 switches it off) every decode launch leaves (busy time, tiles) per CTA in a host
 * table, and pd_device_plan_upload cuts the step, inside the device plan, in shares proportional to the
 * rates seen so far for that kernel and grid; the plan object a caller holds keeps the reference's equal
 * cut.  Outputs stay within the path's tolerance but their last bits follow the cut, so a caller that
 * needs bit-identical results from step to step switches it off.  pd_adaptive_cut_reset forgets the rates. */
int pd_set_adaptive_cut(int on);
int pd_adaptive_cut(void);
int pd_adaptive_cut_reset(void);
/* Folds the latest per-CTA readings of the current device into the weights (what pd_device_plan_upload
 * and pd_device_plan_build do on their own); for callers that replay a CUDA graph holding a device-side
 * plan and therefore never come through those calls.  Does not wait for the device. */
int pd_adaptive_cut_refresh(void* stream);
/* Introspection: the index-th rate table (no particular order).  Returns its grid size (0: no such table)
 * and fills, up to cap CTAs, weights[c] (relative share of CTA c, mean 1) and record[2c], record[2c+1] (total
 * busy nanoseconds and tiles of CTA c at the last reading), record[2 * grid] launches; either may be NULL,
 * record needs 2 * cap + 1 entries. */
int pd_adaptive_cut_table(int index, float* weights, unsigned long long* record, int cap);

/* decode::make_plan (src/decode/decode.hpp:38-39).  num_ctas <= 0 uses
 * pd_default_ctas (needs a GPU).  The plan is a host object; free it with
 * pd_plan_free.  PD_INVALID_ARGUMENT if num_q_heads is not a multiple of
 * num_kv_heads or a sequence length is <= 0. */
int pd_make_plan(int dtype, const int* seq_lens, int batch, int num_q_heads, int num_kv_heads,
                 int head_dim, int num_ctas, pd_plan** out);
/* The same cut with an explicit tile size (tokens per work unit) instead of the
 * kernel's own; pure host arithmetic.  Used to check the planner against the
 * reference's published (ctas, segments) pairs, which were made at tile 64. */
int pd_make_plan_tiled(int tile, const int* seq_lens, int batch, int num_q_heads, int num_kv_heads,
                       int num_ctas, pd_plan** out);
/* The planner's segment rules with unequal shares (no counterpart in the reference): CTA c owns the work
 * units [B_c, B_c+1), B_c = round(total * (w_0 + .. + w_c-1) / sum(w)).  This is the cut the adaptive
 * schedule uses inside the device plan; exposed so that it can be checked on the host.  Pure host
 * arithmetic. */
int pd_make_plan_weighted(int tile, const int* seq_lens, int batch, int num_q_heads, int num_kv_heads,
                          const float* weights, int num_ctas, pd_plan** out);
/* A plan object from arrays the caller already holds: a decode::DecodePlan filled in by
 * the caller (src/decode/decode.hpp:21-27 is a plain struct that callers may build or edit
 * themselves before DevicePlan::upload).  The tables are checked for consistency
 * (monotone, covering the segments, token ranges non-empty and tile-aligned);
 * PD_INVALID_ARGUMENT otherwise.  segments holds 4 ints per segment. */
int pd_plan_from_arrays(int num_ctas, int tile, const int* segments, int num_segments, const int* cta_seg_begin,
                        const int* item_seg_begin, int num_items, pd_plan** out);
void       pd_plan_free(pd_plan* plan);
int        pd_plan_num_ctas(const pd_plan* plan);
int        pd_plan_tile(const pd_plan* plan);
int        pd_plan_num_segments(const pd_plan* plan);
int        pd_plan_num_items(const pd_plan* plan);
const int* pd_plan_segments(const pd_plan* plan);        /* 4 ints per segment */
const int* pd_plan_cta_seg_begin(const pd_plan* plan);   /* num_ctas + 1 */
const int* pd_plan_item_seg_begin(const pd_plan* plan);  /* num_items + 1 */

/* decode::DevicePlan (src/decode/decode.hpp:44-62): device copy of a plan plus the
 * partial-result workspace, grow-only. */
int  pd_device_plan_create(pd_device_plan** out);
void pd_device_plan_destroy(pd_device_plan* dp);
int  pd_device_plan_upload(pd_device_plan* dp, const pd_plan* plan, int group, int head_dim, void* stream);
int  pd_device_plan_bind(const pd_device_plan* dp, pd_params* p);
/* No counterpart in the reference, whose kernels have no bounded waits.  After pd_kernel_status has reported
 * PD_KERNEL_TIMEOUT, the CTA that gave up has skipped its arrivals, so the arrival counters of the in-kernel
 * merge inside this device plan may hold partial counts; a later launch of the same plan would merge rows too
 * early or never.  This call clears them (stream-ordered memsets); the next pd_device_plan_upload / _build
 * does so too. */
int  pd_device_plan_reset(pd_device_plan* dp, void* stream);

/* Device-side planner.  No counterpart in the reference, whose plan is always cut on the host from host
 * lengths (src/decode/decode.cu:65-108) and copied over (decode.cu:112-156); its README lists a
 * device-side, graph-capturable planner as future work.  pd_device_plan_build cuts the same plan with one
 * small kernel from lengths that already live on the device (row b has seq_lens[slot_ids ? slot_ids[b] : b]):
 * the segment, CTA and item arrays it leaves in the device plan are bit-identical to pd_make_plan's for
 * the same lengths and grid.  The call never waits for the device and copies nothing from the host; its
 * buffers only grow (sized for batch * num_kv_heads + grid segments), so once it has run with the
 * largest batch it allocates nothing and may be captured into a CUDA graph together with the decode that
 * follows.  num_ctas <= 0: pd_default_ctas.  The launch grid is num_ctas; CTAs the cut does not need idle.
 * pd_device_plan_bind then sets needs_merge = 3: rows cut in at most 4 pieces are merged inside the decode
 * kernel, the others by the merge kernel, which is always launched (the host cannot know).  For fp16
 * layers with 8 kv heads and at least a third as many rows as the one-CTA-per-SM grid has CTAs, a second
 * launch of the same planner also cuts the step by rows for the head-fused schedule (pd_set_head_fused).
 * With the adaptive cut on, the planner reads the per-CTA shares the host has derived so far from a
 * device array with a stable address (grids up to 1024 CTAs, steps with at least 8 work units per CTA;
 * otherwise the equal cut) and produces the cut of pd_make_plan_weighted for them; the call folds new
 * readings in unless the stream is being captured, and a caller that replays a captured step calls
 * pd_adaptive_cut_refresh between replays.  A length <= 0 gives that row no work and is reported by
 * pd_device_plan_info (the host planner refuses such a batch).
 * pd_device_plan_info (waits for the stream): out[0] CTAs with work, out[1] segments, out[2] most pieces
 * any (row, kv head) was cut in, out[3] 1 + first row with a length <= 0 (0: none).
 * pd_device_plan_fetch (waits for the stream): the plan as a host object, for inspection and tests. */
int  pd_device_plan_build(pd_device_plan* dp, int dtype, const int* d_seq_lens, const int* d_slot_ids, int batch,
                          int num_q_heads, int num_kv_heads, int head_dim, int num_ctas, void* stream);
int  pd_device_plan_info(const pd_device_plan* dp, int* out, void* stream);
int  pd_device_plan_fetch(const pd_device_plan* dp, pd_plan** out, void* stream);

/* decode::paged_decode (src/decode/decode.hpp:66): the split kernel and, if any
 * (row, head) was split across CTAs, the merge.  head_dim 128; group 1, 2, 4, 8.
 * num_pages > 0 bounds the page coordinate of the TMA descriptors (page ids
 * outside [0, num_pages) then read as zeros instead of touching memory);
 * pd_paged_decode passes "unknown". */
int pd_paged_decode(int dtype, const pd_params* p, void* stream);
int pd_paged_decode_bounded(int dtype, const pd_params* p, int num_pages, void* stream);
/* No counterpart in the reference, which has one dequantisation scale per tensor (DecodeParams::k_scale,
 * v_scale; its README notes that per-head scales would help fp8 accuracy).  The same decode with one
 * scale per kv head: d_k_scales / d_v_scales are device arrays of num_kv_heads floats that replace
 * p->k_scale / p->v_scale (either may be NULL: the per-tensor value then applies). */
int pd_paged_decode_scaled(int dtype, const pd_params* p, int num_pages, const float* d_k_scales,
                           const float* d_v_scales, void* stream);

/* What a decode of these params would launch (no counterpart in the reference, which has one kernel shape):
 * out[0] schedule (0 the caller's plan as bound, 1 the same step cut by rows for the head-fused kernel,
 * 2 the caller's plan cut in unequal shares by the adaptive cut), out[1] grid, out[2] tokens per tile,
 * out[3] kv heads per tile, out[4] consumer warps per CTA, out[5] pipeline stages, out[6] CTAs per SM the
 * shape is made for, out[7] needs_merge of that schedule (0 none, 1 merge kernel, 2 merged inside the decode
 * kernel, 3 per row).  Pure host lookup; launches nothing. */
int pd_describe_launch(int dtype, const pd_params* p, int* out);

/* No counterpart in the reference (its DevicePlan always allocates, src/decode/decode.cu:131-141).
 * The same decode + merge as pd_paged_decode_bounded, for callers that cannot allow a device
 * allocation: a server that has already given all free HBM to its KV pool, so that a workspace
 * cudaMalloc at step time would fail, or a step loop that forbids cudaMalloc/cudaFree because
 * they stall the whole device.  This call, including its first use, performs no cudaMalloc,
 * cudaFree or other allocating call.
 *   - p->partial_out / p->partial_lse are ignored: the workspace for rows split across CTAs is
 *     an 8 MiB array built into the library (each GPU that loads the library carries it until
 *     the process exits).  num_segments is the plan's segment count (pd_plan_num_segments); a plan
 *     that needs more than 8 MiB, i.e. num_segments * group * (head_dim + 1) * 4 bytes, is refused
 *     with PD_INVALID_ARGUMENT and nothing is launched.  Headline shapes need 0.4 - 1.6 MiB.
 *     The count is also checked on the device against the plan the kernels walk: if the bound plan
 *     has more segments than declared (a count left over from an earlier plan, say), the CTAs whose
 *     segments lie beyond it store nothing, the status word receives code 6 and the rows of those
 *     CTAs stay unwritten; nothing is ever stored outside the array.
 *   - d_status: device word the kernel writes if a bounded wait expires; the caller zeroes it and
 *     reads it back when it wants to know.  NULL selects a built-in word that nothing reads.
 *   - The first call on each device looks up the built-in arrays' device addresses
 *     (cudaGetSymbolAddress) and raises the kernel's shared-memory limit; make that first call
 *     during start-up, with the intended device current and before any stream capture begins.
 *   - All calls on a device share the one workspace and it keeps whatever the previous call left
 *     there.  Nothing in it has to start at zero (every slot the merge reads was written by the
 *     decode kernel of the same call), but two calls that overlap on the GPU - different streams,
 *     or one stream without ordering between them - overwrite each other's partials.  Order them. */
int pd_paged_decode_static(int dtype, const pd_params* p, int num_segments, int num_pages,
                           unsigned* d_status, void* stream);

/* Device status word of the last decode launched by this thread's library state:
 * 0 = every bounded wait completed.  Reads it back (synchronises `stream`).
 * Nonzero encodes (code << 24 | cta) of the first wait that gave up. */
int pd_kernel_status(void* stream, unsigned* status);

/* Multi-GPU (no counterpart in the reference, which is single-GPU): the decode layer sharded over
 * the GPUs of one node, one process per GPU, with the output all-gather done by the decode
 * kernel itself.  Every rank owns gathered-output buffers; the kernel's epilogue (and its
 * in-kernel merge) stores each output row into the step's buffer on EVERY peer with plain 16-byte
 * peer stores over NVLink.  The kernel neither fences nor signals; a one-warp kernel launched right
 * behind it as a programmatic dependent raises this rank's flag on every peer once the decode grid has
 * completed, and pd_gather_wait / pd_gather_wait_epoch enqueue a one-warp kernel that waits (bounded,
 * ~1 s, then PD_KERNEL_TIMEOUT via pd_kernel_status) until all ranks' flags of the step have arrived.
 * No collective library call is involved.  Four buffers are used in rotation (step e fills buffer
 * e mod 4), so a caller may launch step e+1's decode before it waits for step e: the wait then
 * overlaps the next decode.  Rule for such callers: wait for step e and finish reading its buffer
 * before launching step e+2.
 *   pd_gather_create   allocates this rank's block (four output buffers in rotation + flags)
 *   pd_gather_export   writes the block's CUDA IPC handle (pd_gather_handle_bytes() bytes)
 *   pd_gather_connect  takes all ranks' handles, rank-major, and maps the peers' blocks
 *   pd_paged_decode_gather  pd_paged_decode_bounded with gathered output: this rank's
 *       [batch][num_q_heads] rows land at row `row_offset`, head `head_offset` of rows of
 *       `row_stride_heads` heads (kv-head sharding: offset = rank * local heads; batch sharding:
 *       row_offset = first global row).  p->out is ignored.  Plans with split rows must be
 *       bound by pd_device_plan_bind (in-kernel merge).
 *   pd_paged_decode_gather_sync  the same, and the kernel behind the decode also waits (bounded) for all
 *       ranks' flags of this step: when it has run, the whole gathered layer is in the local buffer.  One
 *       dependent launch instead of two (announcement + pd_gather_wait), for callers that do not overlap
 *       the wait with anything.
 *   pd_gather_buffer   the local gathered buffer number `which` (0..3: step mod 4; -1 = last step)
 *   pd_gather_wait     the wait for the last step; pd_gather_wait_epoch for a step the caller names
 *       (steps are numbered 1, 2, ... by pd_gather_epoch).  Waiting for a step that no peer ever
 *       signals ends after the bounded ~1 s with PD_KERNEL_TIMEOUT in pd_kernel_status; the context
 *       stays usable and nothing in the group needs resetting (flags carry step numbers). */
typedef struct pd_gather_group pd_gather_group;
int      pd_gather_create(int world, int rank, size_t out_bytes, pd_gather_group** out);
void     pd_gather_destroy(pd_gather_group* g);
int      pd_gather_handle_bytes(void);
int      pd_gather_export(const pd_gather_group* g, unsigned char* handle);
int      pd_gather_connect(pd_gather_group* g, const unsigned char* all_handles);
void*    pd_gather_buffer(const pd_gather_group* g, int which);
unsigned pd_gather_epoch(const pd_gather_group* g);
int      pd_paged_decode_gather(int dtype, const pd_params* p, int num_pages, pd_gather_group* g,
                                int row_stride_heads, int head_offset, int row_offset, void* stream);
int      pd_paged_decode_gather_sync(int dtype, const pd_params* p, int num_pages, pd_gather_group* g,
                                     int row_stride_heads, int head_offset, int row_offset, void* stream);
int      pd_gather_wait(pd_gather_group* g, void* stream);
int      pd_gather_wait_epoch(pd_gather_group* g, unsigned epoch, void* stream);

/* read_kernel of the reference's benchmark (bench/bench_decode.cu:69-78, "copy" mode
 * :224-240): a read-only streaming pass over `bytes` of device memory with `blocks`
 * CTAs of 512 threads; the attainable HBM read rate decode is compared with. */
int pd_stream_read(const void* d_buf, size_t bytes, int blocks, void* stream);

/* append_kernel<KV> (src/decode/paged_kv_cache.cu:25-39) on caller-owned buffers:
 * scatter n tokens of fp16 K/V ([n][num_kv_heads][head_dim], device) into the
 * pools through one slot's block-table row (device), quantising to E4M3 with
 * value * (1/scale) when dtype is FP8. */
int pd_append_tokens(int dtype, const void* d_k, const void* d_v, void* k_cache, void* v_cache,
                     const int* d_block_table_row, int start_pos, int n, int num_kv_heads,
                     int head_dim, int page_size, float k_scale, float v_scale, void* stream);
/* The same with one quantisation scale per kv head (device arrays of num_kv_heads floats; NULL: the
 * per-tensor scale): byte = e4m3(value * (1 / scale[head])), reciprocal correctly rounded.  No
 * counterpart in the reference. */
int pd_append_tokens_scaled(int dtype, const void* d_k, const void* d_v, void* k_cache, void* v_cache,
                            const int* d_block_table_row, int start_pos, int n, int num_kv_heads,
                            int head_dim, int page_size, float k_scale, float v_scale,
                            const float* d_k_scales, const float* d_v_scales, void* stream);

/* decode::PagedKVCache (src/decode/paged_kv_cache.hpp:31-73). */
size_t pd_cache_bytes_per_page(const pd_cache_config* cfg);
int    pd_cache_pages_for_budget(const pd_cache_config* cfg, size_t budget_bytes);
int    pd_cache_create(const pd_cache_config* cfg, pd_cache** out);
void   pd_cache_destroy(pd_cache* c);
int    pd_cache_admit(pd_cache* c);   /* slot, or -1 when every slot is in use */
/* PD_OK, PD_OUT_OF_PAGES (nothing changed), PD_INVALID_ARGUMENT, PD_LENGTH_ERROR */
int    pd_cache_append(pd_cache* c, int slot, const void* d_k, const void* d_v, int n, void* stream);
/* PagedKVCache::append (src/decode/paged_kv_cache.cu:95-136) for a whole decode step: `count` slots,
 * slot i receives n[i] tokens from d_k[i] / d_v[i].  Allocator decisions are those of `count`
 * single appends in the given order; one packed host->device copy and two launches instead of one
 * copy, one launch and one stream synchronisation per slot; all-or-nothing on PD_OUT_OF_PAGES /
 * PD_LENGTH_ERROR / PD_INVALID_ARGUMENT (a slot may appear once).  Stream-ordered: it does not
 * wait, and the sources must stay valid until the stream has consumed them. */
int    pd_cache_append_batch(pd_cache* c, int count, const int* slots, const void* const* d_k,
                             const void* const* d_v, const int* n, void* stream);
int    pd_cache_release(pd_cache* c, int slot);
/* Per-kv-head scales for an fp8 cache (host arrays of num_kv_heads positive floats; both NULL: back to
 * the per-tensor scales of the config).  Every later append quantises and every later run dequantises
 * with them.  Only while the cache holds no tokens.  No counterpart in the reference. */
int    pd_cache_set_head_scales(pd_cache* c, const float* k_scales, const float* v_scales);
void   pd_cache_shuffle_free_pages(pd_cache* c, unsigned seed);
int    pd_cache_plan(pd_cache* c, const int* slots, int num_slots, int num_q_heads, int num_ctas, void* stream);
/* plan() through the device-side planner (pd_device_plan_build) from the cache's own device lengths, which
 * appends update in stream order.  d_slot_ids: device array of `batch` slot numbers that stays valid until
 * the last run() of this plan, or NULL for slots 0..batch-1.  pd_cache_last_plan returns NULL afterwards.
 * No counterpart in the reference. */
int    pd_cache_plan_device(pd_cache* c, const int* d_slot_ids, int batch, int num_q_heads, int num_ctas, void* stream);
int    pd_cache_run(pd_cache* c, const void* d_q, void* d_out, void* stream);
int    pd_cache_decode(pd_cache* c, const void* d_q, void* d_out, int batch, int num_q_heads,
                       int num_ctas, void* stream);
/* pd_describe_launch for the cache's current plan: what the next run() launches.  No counterpart in the reference. */
int    pd_cache_describe_launch(const pd_cache* c, int* out);
const pd_plan* pd_cache_last_plan(const pd_cache* c);  /* borrowed; valid until the next plan */
int    pd_cache_params(const pd_cache* c, pd_params* out);
int    pd_cache_seq_len(const pd_cache* c, int slot);
int    pd_cache_occupied(const pd_cache* c, int slot);
int    pd_cache_free_pages(const pd_cache* c);
int    pd_cache_max_seq_len(const pd_cache* c);
size_t pd_cache_total_bytes(const pd_cache* c);
int    pd_cache_config_of(const pd_cache* c, pd_cache_config* out);
/* Host copy of a slot's page ids; returns the count and writes up to cap of them. */
int    pd_cache_block_table(const pd_cache* c, int slot, int* out, int cap);
/* Free list, back = next page handed out; returns the count. */
int    pd_cache_free_list(const pd_cache* c, int* out, int cap);

#ifdef __cplusplus
}
#endif
#endif /* PD_B200_H */
