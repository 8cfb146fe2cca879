/*
 * hiscache_b200.h -- C ABI of libhiscache_b200.so
 *
 * B200 (sm_100a) kernels for the data-parallel hot path of HisCache:
 * history-aware CSR gather-reduce aggregation (forward / backward), the
 * gradient-based admission with history writeback, used-mask propagation,
 * cache lookup + feature-row assembly (host-resident rows included), and the
 * bucket / un-permute steps either side of the multi-GPU table exchange.
 *
 * This library replaces the pybind11 module `hiscache_backend` of the
 * reference (src/cpp/python_bindings/binding.cpp:9-19) and the torch index
 * arithmetic of hiscache/history_cache.py / hiscache/history_table.py that sits
 * on the same path.  Every entry point cites the reference interface it
 * replaces.
 *
 * Conventions
 *   - plain C: raw device pointers, sizes, a CUDA stream passed as `void*`
 *     (a `cudaStream_t`; NULL = the legacy default stream);
 *   - indices are int64 as in the reference (`using Index = int64_t`,
 *     src/cpp/include/common.h:11); -1 means "no entry";
 *   - every function returns an int: 0 = ok, negative = HC_ERR_* argument
 *     error detected before any launch, positive = the `cudaError_t` of the
 *     failing runtime call.  Nothing here exits, aborts, resets the device or
 *     traps (the reference does: common.h:13-34);
 *   - nothing is allocated unless the function says so; the caller owns every
 *     buffer; launches are asynchronous on the given stream;
 *   - row storage dtype is HC_F32 or HC_F16, accumulation is always fp32.
 */
#ifndef HISCACHE_B200_H
#define HISCACHE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HC_ABI_VERSION 1

/* storage dtypes */
#define HC_F32 0
#define HC_F16 1

/* argument errors (returned negated: e.g. -HC_ERR_NULL) */
#define HC_ERR_NULL 1      /* a required pointer is NULL                      */
#define HC_ERR_SIZE 2      /* a size / count / stride is out of range         */
#define HC_ERR_DTYPE 3     /* unknown dtype code                              */
#define HC_ERR_ALIGN 4     /* pointer not aligned to its element type         */
#define HC_ERR_UNSUPPORTED 5 /* combination of options not implemented        */
#define HC_ERR_STRUCT 6    /* args->struct_size does not match this build     */
#define HC_ERR_LIMIT 7     /* more rows than a fixed-capacity entry point takes */
#define HC_ERR_RANGE 8     /* an index of the block is outside its table (checked build) */

/* score kinds */
#define HC_SCORE_L2 0 /* sqrt(sum x^2): HistoryCache.update_history, history_cache.py:205 */
#define HC_SCORE_L1 1 /* sum |x|     : HistoryTable.record_history, history_table.py:161 */

int hc_abi_version(void);
/* Human-readable text for a return code of any function below. The pointer is
 * static storage (negative codes) or CUDA's own string (positive codes). */
const char* hc_error_string(int code);

/* ------------------------------------------------------------------------ */
/* Aggregation                                                              */
/* ------------------------------------------------------------------------ */

/*
 * One descriptor serves forward and backward so that both see the same block.
 * Set struct_size = sizeof(hc_aggr_args) and zero the rest before filling.
 *
 * A "target" is a (destination row, head) pair; num_head == 1 gives one target
 * per row.  Source row s, head h starts at input + (s*num_head + h)*feat when
 * in_stride == num_head*feat (the only layout the reference has).
 */
typedef struct hc_aggr_args {
  uint32_t struct_size;
  /* CSR block over destination rows */
  const int64_t* ptr;      /* [num_node + 1]                                 */
  const int64_t* idx;      /* [ptr[num_node]] local source ids               */
  int64_t num_node;        /* destination rows to process                    */
  /* source rows */
  const void* input;       /* [n_src, num_head, feat]                        */
  int32_t in_dtype;        /* HC_F32 | HC_F16                                */
  int32_t feat;            /* F, columns per (row, head)                     */
  int32_t num_head;        /* >= 1                                           */
  int64_t n_src;           /* rows of input (size of grad_input)             */
  int64_t in_stride;       /* elements between source rows; 0 = num_head*feat*/
  /* optional per-source select made inside the gather: when src_map is not
   * NULL and src_map[s] != -1, source s is read from row src_map[s] of
   * src_alt instead of from input, and receives no gradient in backward.    */
  const int64_t* src_map;  /* [n_src] or NULL                                */
  const void* src_alt;     /* [*, num_head*feat] rows, stride alt_stride     */
  int32_t alt_dtype;
  int64_t alt_stride;      /* elements; 0 = num_head*feat                    */
  /* NULL => mean over neighbours; else weighted sum with edge_value[e] or
   * edge_value[e*num_head + h] (no division; written for empty rows too)     */
  const float* edge_value;
  /* optional per-destination history override: hmap[r] != -1 => the output
   * row is a copy of a history row and nothing flows to its neighbours.      */
  const int64_t* hmap;     /* [num_node] or NULL                             */
  const void* hbuf;        /* history rows, stride hsize elements            */
  int32_t h_dtype;
  int32_t h_indexed;       /* 0: read row r (reference layout, row-aligned
                              buffer); 1: read row hmap[r] of the table       */
  int64_t hsize;           /* == feat, or == num_head*feat (per-head rows)   */
  /* row counts of the two optional tables, used only by the index checks of a
   * library built with HC_CHECK_BOUNDS (0 = unknown, not checked)            */
  int64_t h_rows;          /* rows of hbuf                                   */
  int64_t alt_rows;        /* rows of src_alt                                */
} hc_aggr_args;

/*
 * out[t, :] (fp32, [num_node, num_head, feat]) for every target t.  Every
 * element of out is written (empty rows get zeros), so out need not be
 * cleared.  Replaces aggr_forward_history / aggr_forward_history_edge_value
 * (src/cpp/src/history_aggr.cu:598-617; kernels :7-125; launcher :399-473).
 * With hmap == NULL it is the plain mean aggregation the reference takes from
 * cxgnncomp.sage_mean_forward (hiscache/history_model.py:90).
 */
int hc_aggr_fwd(const hc_aggr_args* a, float* out, void* stream);

/*
 * Transposed scatter of grad_out (fp32 [num_node, num_head, feat]).
 *   grad_input  fp32 [n_src, num_head, feat] or NULL: miss rows add
 *               grad_out[t]/deg (or * edge_value) to every neighbour's row.
 *               zero_grad_input != 0 clears it first (cudaMemsetAsync).
 *   grad_history fp32, stride hsize, rows [0, num_node), or NULL: hit rows
 *               receive grad_out[t]; miss rows are written as zeros
 *               (row-aligned, as zeros_like(history_buffer) in the reference).
 *   edge_grad   fp32 [E(, num_head)] or NULL: <grad_out[t], source row>.
 *   row_score   fp32 [num_node] or NULL (num_head must be 1): the admission
 *               score of grad_out[r, :] (score_kind), computed in the same
 *               pass in the library's fixed reduction order (see hc_score_rows).
 * Replaces AggrHistoryFunction::backward / historyBackwardImpl
 * (history_aggr.cu:493-596; kernels :127-397) and, with row_score, the
 * `grad.norm(dim=1)` of hiscache/history_cache.py:205.
 */
int hc_aggr_bwd(const hc_aggr_args* a, const float* grad_out, float* grad_input,
                int32_t zero_grad_input, float* grad_history, float* edge_grad,
                float* row_score, int32_t score_kind, void* stream);

/*
 * Index checks (a library built with -DHC_CHECK_BOUNDS, libhiscache_b200_checked.so).
 *
 * The aggregation kernels trust ptr, idx, src_map and hmap; the reference does too, and a value
 * outside its table is an out-of-range access on the device (its 32-bit index arithmetic,
 * history_aggr.cu:34-35, was one way to get there).  In the checked build hc_aggr_fwd and
 * hc_aggr_bwd first run a validation kernel over the block: ptr must be non-decreasing from a
 * non-negative start, idx[e] in [0, n_src), src_map[s] in [-1, alt_rows), hmap[r] in
 * [-1, h_rows) when h_indexed (row-aligned: num_node <= h_rows).  The first violation is
 * recorded in a status word on the device and the operator's kernels then return without
 * touching memory: nothing faults, nothing traps, out / gradients are left as they were.
 *   hc_last_status: waits for `stream`, then out[0] = 0 (clean) or HC_ERR_RANGE, out[1] = which
 *     array (1 ptr, 2 idx, 3 src_map, 4 hmap), out[2] = position in it, out[3] = the offending
 *     value; clear != 0 resets the word (a set word blocks every later aggregation call).
 *     In the regular build it returns -HC_ERR_UNSUPPORTED.
 */
int hc_last_status(int64_t out[4], int32_t clear, void* stream);

/*
 * Backward as a gather over the transposed block (mean aggregation, one head,
 * no edge values): the alternative to the atomic scatter of hc_aggr_bwd, with
 * no atomics on the data, no zero-fill and a bit-reproducible result.  No
 * reference counterpart (the reference only scatters, history_aggr.cu:127-168).
 *   hc_transpose_block: a stable radix sort of the block's edge slots
 *     [0, n_edges) by source (n_edges >= ptr[num_node]; slots behind it are
 *     ignored).  t_ptr [n_src+1], t_dst / t_w [n_edges]: for every source s the
 *     ascending list of destination rows r < num_node with hmap[r] == -1 that
 *     have s as a neighbour (once per edge) and, beside each, the weight
 *     1/deg(r); sources with src_map[s] != -1 are left empty.  The cost does
 *     not depend on the skew of the source popularity.
 *     scratch >= hc_transpose_scratch_bytes(n_src, n_edges).
 *   hc_aggr_bwd_gather: grad_input[s, :] = sum over that list of
 *     t_w * grad_out[r, :] for s < n_src; every row of grad_input is written
 *     (zeros for empty lists), so it needs no clearing.  The lists may come
 *     from a transposition of a LARGER block that has this one as a prefix
 *     (the layers of a sampled batch share one CSR): entries with
 *     r >= num_node or hmap[r] != -1 are skipped, as are sources with
 *     src_map[s] != -1.  Lists longer than 64 entries take a thread block
 *     each; lists longer than 2048 are split into chunks over several blocks
 *     and their chunk sums added in chunk order.
 *     feat must be a multiple of 4 and <= 1024; t_n_src / n_edges: the n_src
 *     and n_edges the transposition was built with (a->n_src <= t_n_src, else
 *     HC_ERR_SIZE); scratch >= hc_gather_scratch_bytes(n_edges, feat),
 *     16-byte aligned (may be NULL when n_edges <= 64).
 */
int64_t hc_transpose_scratch_bytes(int64_t n_src, int64_t n_edges);
int hc_transpose_block(const hc_aggr_args* a, int64_t n_edges, int64_t* t_ptr, int64_t* t_dst,
                       float* t_w, void* scratch, void* stream);
int64_t hc_gather_scratch_bytes(int64_t n_edges, int32_t feat);
int hc_aggr_bwd_gather(const hc_aggr_args* a, const int64_t* t_ptr, const int64_t* t_dst,
                       const float* t_w, int64_t t_n_src, int64_t n_edges, const float* grad_out,
                       float* grad_input, void* scratch, void* stream);

/* ------------------------------------------------------------------------ */
/* Scores and thresholds                                                    */
/* ------------------------------------------------------------------------ */

/*
 * score[r] = L2 or L1 norm of x[r, 0:feat] (fp32, row stride `stride`
 * elements).  Fixed order, restated by the oracle bit for bit: element e
 * goes to lane (e/4) mod 32; each lane adds its terms in increasing e with
 * separately rounded multiply and add; the 32 partial sums are combined by
 * an xor butterfly (16, 8, 4, 2, 1); L2 takes a correctly rounded sqrt.
 * Replaces grad.norm(dim=1) (history_cache.py:205) and sum(|grad|, 1)
 * (history_table.py:161,219).
 */
int hc_score_rows(const float* x, int64_t n, int32_t feat, int64_t stride,
                  int32_t kind, float* score, void* stream);

/*
 * thres[0] = torch.quantile(score, q) with linear interpolation
 * (history_cache.py:211, history_table.py:173,230): rank = fp32(q)*(n-1)
 * computed in fp32, the two neighbouring order statistics found by an exact
 * radix select, combined as fma(w, hi-lo, lo) for w < 0.5 and
 * fma(-(hi-lo), 1-w, hi) otherwise (torch's lerp, whose multiply-add is fused
 * in its CPU and CUDA builds).  NaN in score gives NaN.
 * n == 0 is HC_ERR_SIZE.  Up to 49 152 scores are staged in shared memory by
 * one thread block (one pass over global memory); more take four passes of a
 * multi-block digit histogram with state in scratch: device, 8-byte aligned,
 * >= hc_select_scratch_bytes(n) (0 bytes, and scratch may be NULL, for the
 * small form).
 */
int64_t hc_select_scratch_bytes(int64_t n);
int hc_select_threshold(const float* score, int64_t n, float q, float* thres,
                        void* scratch, void* stream);
/*
 * The same quantile over the n_valid[0] (device int64) smallest of the n
 * scores, for batches padded to a fixed shape: the caller sets the scores of
 * padding rows to +inf.  Nothing about the size has to be known on the host.
 */
int hc_select_threshold_counted(const float* score, int64_t n, const int64_t* n_valid, float q,
                                float* thres, void* scratch, void* stream);

/* ------------------------------------------------------------------------ */
/* Admission and eviction                                                   */
/* ------------------------------------------------------------------------ */

/* Device scratch needed by the two admission entry points for n candidates. */
int64_t hc_admit_scratch_bytes(int64_t n);

/*
 * Ring-buffer admission of the per-layer table path; deterministic
 * restatement of record_history (src/cpp/src/grad_check.cu:6-68).  Row `sub`
 * of buffer_new is admitted iff sub_to_history[sub] == -1 and not
 * (thres[0] != 0 and score[sub] > thres[0]) and used_mask[sub] (NULL = all
 * used).  Admitted rows take consecutive ring slots in ascending `sub`
 * starting at header[0] (the reference takes them in warp-scheduling order,
 * grad_check.cu:25); a slot's previous owner g is unmapped only while
 * full_to_history[g] still equals that slot; the row is copied (converted to
 * table_dtype); full_to_history[sub_to_full[sub]], history_to_full[slot] and
 * checkin_iter[slot] are set; header[0] advances modulo capacity.  If more
 * rows are admitted than the table holds, the result equals applying them one
 * by one.  n_admitted (device int64[1], may be NULL) receives the count.
 */
int hc_record_history(const float* buffer_new, int64_t new_stride, int64_t n,
                      void* buffer_all, int32_t table_dtype, int64_t capacity,
                      int32_t history_size, const uint8_t* used_mask,
                      const int64_t* sub_to_full, const int64_t* sub_to_history,
                      int64_t* history_to_full, int64_t* full_to_history,
                      int64_t* header, const float* score, const float* thres,
                      int64_t* checkin_iter, int64_t glb_iter,
                      int64_t* n_admitted, void* scratch, void* stream);

/*
 * hc_record_history for callers that cannot allocate device memory.  (No
 * counterpart in the reference, whose op allocates nothing because its kernel
 * takes slots with an atomic counter.)  Who needs it: a plain-C / cgo / JNI
 * host that only holds the buffers it was handed and has no way to reach the
 * framework's device allocator for the scratch argument, and loops whose
 * device memory is wholly owned by a caching allocator, where a raw
 * cudaMalloc / cudaFree would fail or stall the device.  Same arguments and
 * result as hc_record_history minus `scratch`: the scratch is a 16 KB array
 * inside the library image (each GPU that loads the library holds it until
 * exit).  Limits and rules:
 *   - n <= HC_NOALLOC_MAX_ROWS (hc_noalloc_max_rows()); more returns
 *     -HC_ERR_LIMIT and nothing is launched;
 *   - calls no cudaMalloc / cudaFree / allocating routine;
 *   - the first call on a device looks the array's device address up
 *     (cudaGetSymbolAddress, with the caller's current device) and remembers
 *     it; make that first call with the right device current and before any
 *     stream capture begins;
 *   - all calls on one device share the array: two calls whose kernels can
 *     overlap on the GPU (different streams) race; serialise them.  Nothing
 *     in the array needs clearing between calls.
 */
#define HC_NOALLOC_MAX_ROWS (1 << 20)
int64_t hc_noalloc_max_rows(void);
int hc_record_history_noalloc(const float* buffer_new, int64_t new_stride, int64_t n,
                              void* buffer_all, int32_t table_dtype, int64_t capacity,
                              int32_t history_size, const uint8_t* used_mask,
                              const int64_t* sub_to_full, const int64_t* sub_to_history,
                              int64_t* history_to_full, int64_t* full_to_history,
                              int64_t* header, const float* score, const float* thres,
                              int64_t* checkin_iter, int64_t glb_iter,
                              int64_t* n_admitted, void* stream);

/*
 * Admission of the unified-buffer cache path; restatement of
 * HistoryCache.update_history (hiscache/history_cache.py:211-254) with the
 * write position kept on the device.  Row r of produced ([n, hidden] fp32) is
 * admitted iff score[r] < thres[0] and sub2embed[r] == -1; admitted rows are
 * appended in ascending r at embedding slots header[0].. ; raw-feature slots
 * overlapped by the new rows lose their mapping through feat2full; previous
 * owners of the overwritten embedding slots are unmapped only if their map
 * still points into the overwritten range; then full2embed / embed2full are
 * set and header[0] advances.  Unlike the reference, rows that would run past
 * embed_capacity are not admitted.  reset_header != 0 sets header[0] = 0
 * first (the ring restart of history_cache.py:190-192).  valid (bytes [n],
 * may be NULL): rows with valid[r] == 0 are never admitted (padding rows of
 * fixed-shape batches).
 * full2embed has 2*total_num_node + 1 entries (history_cache.py:42-46).
 */
int hc_cache_admit(const float* produced, int64_t prod_stride, int64_t n,
                   void* buffer, int32_t buf_dtype, int32_t hidden,
                   int32_t in_feat, int64_t embed_capacity,
                   const int64_t* sub_to_full, const int64_t* sub2embed,
                   const float* score, const float* thres, int64_t* full2embed,
                   int64_t total_num_node, int64_t* embed2full,
                   const int64_t* feat2full, int64_t feat2full_len,
                   int64_t* header, int32_t reset_header, const uint8_t* valid,
                   int64_t* n_admitted, void* scratch, void* stream);

/*
 * Staleness eviction: every slot with -1 < checkin_iter[s] <= glb_iter - limit
 * is cleared in checkin_iter, history_to_full and full_to_history
 * (hiscache/history_table.py:189-200, :244-251).
 */
int hc_evict_stale(int64_t* checkin_iter, int64_t* history_to_full,
                   int64_t* full_to_history, int64_t capacity, int64_t glb_iter,
                   int64_t limit, void* stream);

/*
 * The iteration number kept in device memory (int64[1]), for steps replayed
 * from a CUDA graph, where it cannot be a launch argument:
 * hc_evict_stale_dev is hc_evict_stale with glb_iter read from glb_iter_dev[0];
 * hc_stamp_checkin replaces every checkin_iter[s] == marker by glb_iter_dev[0]
 * (call hc_record_history with glb_iter = marker, a value no iteration takes,
 * then stamp).
 */
int hc_evict_stale_dev(int64_t* checkin_iter, int64_t* history_to_full,
                       int64_t* full_to_history, int64_t capacity,
                       const int64_t* glb_iter_dev, int64_t limit, void* stream);
int hc_stamp_checkin(int64_t* checkin_iter, int64_t capacity, int64_t marker,
                     const int64_t* glb_iter_dev, void* stream);

/*
 * Score eviction: for r < n with score[r] >= thres[0] and
 * sub_to_history[r] != -1 the slot is cleared in all three arrays
 * (hiscache/history_table.py:234-241).
 */
int hc_evict_by_score(const int64_t* sub_to_history, const float* score,
                      const float* thres, int64_t n, int64_t* checkin_iter,
                      int64_t* history_to_full, int64_t* full_to_history,
                      void* stream);

/* ------------------------------------------------------------------------ */
/* Receptive-field bookkeeping                                              */
/* ------------------------------------------------------------------------ */

/*
 * masks: num_layer+1 consecutive byte masks of num_node entries each
 * (masks[k] at masks + k*num_node), all written here.  masks[num_layer] is
 * the seed level, masks[0] gates raw-feature loading; a row with
 * history_map[r] != -1 stops the propagation at the second step only.
 * Replaces count_history_reconstruct (grad_check.cu:70-130).  ptr has
 * ptr_rows+1 entries; history_map may be NULL or have >= the number of rows
 * that can be live at the second step.
 */
int hc_used_masks(const int64_t* ptr, const int64_t* idx, int64_t ptr_rows,
                  const int64_t* history_map, int64_t history_map_len,
                  int64_t num_node, int64_t num_seed, int32_t num_layer,
                  uint8_t* masks, void* stream);

/*
 * Level-synchronous form of get_graph_structure_score (grad_check.cu:132-163):
 * seeds get 1; at each of num_layer steps an unset neighbour takes
 * score(parent)*deg(parent) of its lowest-numbered parent that was set before
 * the step.  output: int64 [num_node], written here.  scratch: int64
 * [num_node].
 */
int hc_structure_score(const int64_t* ptr, const int64_t* idx, int64_t ptr_rows,
                       int64_t num_node, int64_t num_seed, int32_t num_layer,
                       int64_t* output, int64_t* scratch, void* stream);

/*
 * output[v] (int32 [mmax+1], cleared here) = number of i with arr[i] == v,
 * except that value 0 is never counted (count_num, grad_check.cu:165-182).
 * Values outside [0, mmax] are ignored.
 */
int hc_count_num(const int64_t* arr, int64_t n, int64_t mmax, int32_t* output,
                 void* stream);

/* ------------------------------------------------------------------------ */
/* Lookup and feature-row assembly                                          */
/* ------------------------------------------------------------------------ */

/*
 * out[i] = map[ids[i] + offset] for i < n (negative positions wrap from the
 * end as torch indexing does).  The two lookups of lookup_and_load
 * (history_cache.py:310,315) are this with offset 0 / total_num_node.
 * force_miss_below: entries i < force_miss_below are set to -1 (the
 * seeds-are-never-history rule of history_table.py:106).
 */
int hc_map_lookup(const int64_t* map, int64_t map_len, const int64_t* ids,
                  int64_t n, int64_t offset, int64_t force_miss_below,
                  int64_t* out, void* stream);

/*
 * out[i, :] = table[rows[i], :] for i < n; rows[i] == -1 reads the last row
 * (torch negative indexing, which history_cache.py:312-313 relies on), unless
 * zero_missing != 0, in which case the output row is zeros.  Output dtype may
 * differ from the table's.
 */
int hc_gather_rows(const void* table, int32_t table_dtype, int64_t table_rows,
                   int64_t table_stride, int32_t feat, const int64_t* rows,
                   int64_t n, int32_t zero_missing, void* out, int32_t out_dtype,
                   int64_t out_stride, void* stream);

/*
 * Assembles batch.x in one pass (history_cache.py:327-350 and :276-288):
 *   load_mask[i] = (used == NULL || used[i]) && sub2feat[i] == -1
 *   x[i] = load_mask[i] ? host_table[sub_to_full[i]]
 *        : sub2feat[i] != -1 ? feat_cache[sub2feat[i]] : 0
 * host_table may be device memory or mapped pinned host memory (history_uvm
 * mode): rows are fetched by the kernel itself over the host link and staged
 * through shared memory.  load_mask_out (bytes, may be NULL) receives the
 * mask; stats (int64[2], may be NULL) accumulates {rows from host_table, rows
 * from the feature cache}.
 */
int hc_load_rows(const void* host_table, int32_t host_dtype, int64_t host_rows,
                 int64_t host_stride, const void* feat_cache, int32_t cache_dtype,
                 int64_t cache_rows, int64_t cache_stride, int32_t feat,
                 const int64_t* sub_to_full, const int64_t* sub2feat,
                 const uint8_t* used, int64_t n, void* x, int32_t x_dtype,
                 int64_t x_stride, uint8_t* load_mask_out, int64_t* stats,
                 void* stream);

/*
 * hc_load_rows for a batch whose host rows were (partly) fetched ahead of the
 * step.  staged_rows is [n, feat] in device memory, dtype x_dtype, contiguous;
 * where staged_mask[i] != 0 it holds host_table[sub_to_full[i]] and a row that
 * hc_load_rows would read from host_table is read from there instead:
 *   x[i] = !load_mask[i] ? (as hc_load_rows)
 *        : staged_mask[i] ? staged_rows[i] : host_table[sub_to_full[i]]
 * The result equals hc_load_rows' for any staged_mask (host rows never change);
 * only the bytes that cross the host link during the step differ.  stats is
 * int64[3] here: {rows from host_table, rows from the feature cache, rows from
 * staged_rows}.  The reference loads in the step only (history_cache.py:
 * 327-350) and has no counterpart.
 */
int hc_load_rows_staged(const void* host_table, int32_t host_dtype,
                        int64_t host_rows, int64_t host_stride,
                        const void* feat_cache, int32_t cache_dtype,
                        int64_t cache_rows, int64_t cache_stride, int32_t feat,
                        const int64_t* sub_to_full, const int64_t* sub2feat,
                        const uint8_t* used, int64_t n, void* x, int32_t x_dtype,
                        int64_t x_stride, uint8_t* load_mask_out, int64_t* stats,
                        const void* staged_rows, const uint8_t* staged_mask,
                        void* stream);

/*
 * The staging for hc_load_rows_staged; on any stream, at any time before the
 * step that consumes it:
 *   staged_mask[i] = (consider == NULL || consider[i]) && (sub2feat == NULL || sub2feat[i] == -1)
 *   staged_rows[i] = host_table[ids[i]]      where staged_mask[i]
 * Rows whose mask is 0 are left unspecified (they may or may not be written).
 * staged_rows is [n, feat] of host_dtype, contiguous.  stats (int64[3], may be
 * NULL): [0] += rows copied, [1] += rows skipped because sub2feat[i] != -1.
 * The call is meant to run beside a training step and therefore uses a small
 * grid (the more host reads are outstanding, the more the step's own kernels
 * are slowed down); max_blocks > 0 overrides the default number of thread
 * blocks (16).
 */
int hc_stage_host_rows(const void* host_table, int32_t host_dtype,
                       int64_t host_rows, int64_t host_stride, int32_t feat,
                       const int64_t* ids, const int64_t* sub2feat,
                       const uint8_t* consider, int64_t n, void* staged_rows,
                       uint8_t* staged_mask, int64_t* stats, int32_t max_blocks,
                       void* stream);

/* ------------------------------------------------------------------------ */
/* Multi-GPU table exchange helpers                                         */
/* ------------------------------------------------------------------------ */

/* owner(id) = hc_mix64(id) mod world; the partition function of the sharded
 * history table (the reference has none: its only sharding attempt splits the
 * feature axis, history_cache.py:72-78). Host-callable. */
uint64_t hc_mix64(uint64_t x);

/*
 * Stable bucket sort of ids by owner: counts[w] (int64 [world]) = ids owned by
 * w; perm[k] (int64 [n]) = position in ids of the k-th element in bucket
 * order (buckets ascending, original order inside a bucket);
 * bucketed[k] = ids[perm[k]].  keep (bytes, may be NULL): entries with
 * keep[i] == 0 are left out (counts exclude them; the tail of perm/bucketed is
 * unspecified).  Replaces the per-(src,dst) index_select of prepare_transfer
 * (hiscache/comm.py:132-143).  scratch >= hc_bucket_scratch_bytes(n, world).
 */
int64_t hc_bucket_scratch_bytes(int64_t n, int32_t world);
int hc_bucket_by_owner(const int64_t* ids, const uint8_t* keep, int64_t n,
                       int32_t world, int64_t* counts, int64_t* perm,
                       int64_t* bucketed, void* scratch, void* stream);

/*
 * Fixed-shape form of the exchange, which needs no sizes on the host: every
 * (source, destination) pair carries exactly `slots` ids.
 * hc_bucket_pad: out[w*slots + p] = p-th id of bucket w (bucket order and
 *   counts from hc_bucket_by_owner) or -1; ids beyond `slots` in a bucket are
 *   dropped and added to overflow[0] (device int64, may be NULL).
 * hc_unpad_hits: for bucket-order entry k < n (position p in bucket w):
 *   slot_of[perm[k]] = w*slots + p (or -1 if dropped); hit_out[perm[k]] = that
 *   row when flags_back[row] != 0, else -1.  Entries past the sum of counts
 *   (left out by the keep mask) are not written.
 * hc_last_occurrence: winners[k] = 1 iff ids[k] >= 0 and no later entry of ids
 *   has the same value (the admissions of one step: last copy wins).  claim:
 *   int32 [map_len], all -1 on entry and again on return.  n < 2^31.
 * No reference counterpart (the reference's exchange is one-process peer copies,
 * hiscache/comm.py:48-85).
 */
int hc_bucket_pad(const int64_t* bucketed, const int64_t* counts, int64_t n, int32_t world,
                  int64_t slots, int64_t* out, int64_t* overflow, void* stream);
int hc_unpad_hits(const int64_t* perm, const int64_t* counts, int64_t n, int32_t world,
                  int64_t slots, const uint8_t* flags_back, int64_t* hit_out, int64_t* slot_of,
                  void* stream);
int hc_last_occurrence(const int64_t* ids, int64_t n, int32_t* claim, int64_t map_len,
                       uint8_t* winners, void* stream);

/*
 * dst[perm[k], :] = src[k, :] for k < n where flags == NULL or flags[k] != 0
 * (post_transfer of hiscache/comm.py:146-151, by rows instead of by feature
 * slices).  hit_out (int64 [*], may be NULL): hit_out[perm[k]] = flags[k] ?
 * k : -1, the row-aligned history map the aggregation consumes.
 */
int hc_unpermute_rows(const void* src, int32_t dtype, int64_t src_stride,
                      int32_t feat, const int64_t* perm, const uint8_t* flags,
                      int64_t n, void* dst, int64_t dst_stride, int64_t* hit_out,
                      void* stream);

/*
 * Owner-side lookup for the exchange: for k < n, slot = map[ids[k]] (ids are
 * global node ids this rank owns); flags[k] = slot != -1; rows_out[k, :] =
 * table[slot, :] when hit (left untouched otherwise).
 */
int hc_owner_lookup(const int64_t* map, int64_t map_len, const int64_t* ids,
                    int64_t n, const void* table, int32_t dtype,
                    int64_t table_rows, int64_t table_stride, int32_t feat,
                    void* rows_out, int64_t out_stride, uint8_t* flags,
                    void* stream);

/* ------------------------------------------------------------------------ */
/* History exchange over peer memory (one process per GPU, NVLink loads)    */
/* ------------------------------------------------------------------------ */

/*
 * Replaces the p2psend / all2all path of src/cpp/src/comm.cu:5-29 and
 * hiscache/comm.py:8-151 for the node-partitioned history (owner(id) =
 * hc_mix64(id) mod world).  Every rank keeps its shard (id -> slot map, rows)
 * and a "published candidates" area (ids, fp32 rows, count) in ONE allocation
 * made by hc_peer_alloc, exports it with hc_peer_export, and maps the other
 * ranks' allocations with hc_peer_open.  The pointer tables below are HOST
 * arrays of `world` device pointers, entry r = rank r's copy (own memory for
 * r == me).  Only plain loads cross the link; nothing is written to a peer.
 * No kernel waits for another GPU: the caller orders the ranks with the
 * collectives its step already has (a lookup may not overlap an admission on
 * the owner; a pull may not start before every rank published).
 *
 *   hc_peer_alloc / hc_peer_free : cudaMalloc'd, zero-filled region (the one
 *       place this library allocates: an exported region must be an allocation
 *       of its own).  hc_peer_export writes HC_PEER_HANDLE_BYTES bytes that
 *       another process of the same box passes to hc_peer_open (mapped with
 *       lazily enabled peer access); hc_peer_close unmaps.
 *   hc_peer_lookup : for i < n: slot = peer_maps[owner(ids[i])][ids[i]]; on a
 *       hit (0 <= slot < table_rows) rows_out[i,:] = peer_tables[owner][slot,:]
 *       and hit_map[i] = i, else hit_map[i] = -1 and the row is left untouched.
 *       Rows must be multiples of 16 bytes (else -HC_ERR_UNSUPPORTED).
 *   hc_peer_publish: pub_n[0] = n; for i < n: row i is published when mask[i] != 0
 *       (mask NULL = all) and score[i] < thres[0] (score NULL = no test; the
 *       admission test of grad_check.cu:31-33 made where the candidates are
 *       written) and present[i] == -1 (present NULL = no test; rows that were
 *       served from history are not admitted again).  pub_ids[i] = ids[i] or -1,
 *       pub_rows[i,:] = rows[i,:] for published rows.  n > max_ids is
 *       -HC_ERR_LIMIT.
 *   hc_peer_pull   : scans every rank's published ids in (rank, row) order, keeps
 *       those this rank owns, and writes them to got_ids[0..cap) / got_rows
 *       (fp32 [cap, feat], contiguous) in that order; the tail of got_ids is -1;
 *       candidates beyond cap are dropped and counted in *overflow (may be
 *       NULL).  scratch >= hc_peer_pull_scratch_bytes(world, max_ids).
 */
#define HC_MAX_PEERS 32
#define HC_PEER_HANDLE_BYTES 64
int hc_peer_alloc(int64_t bytes, void** ptr);
int hc_peer_free(void* ptr);
int hc_peer_export(const void* ptr, void* handle);
int hc_peer_open(const void* handle, void** ptr);
int hc_peer_close(void* ptr);
int hc_peer_lookup(const void* const* peer_maps, const void* const* peer_tables, int32_t world,
                   int64_t map_len, int32_t dtype, int64_t table_rows, int64_t table_stride,
                   int32_t feat, const int64_t* ids, int64_t n, void* rows_out, int64_t out_stride,
                   int64_t* hit_map, void* stream);
int hc_peer_publish(const int64_t* ids, const uint8_t* mask, const float* score,
                    const float* thres, const int64_t* present, int64_t n, const float* rows,
                    int64_t row_stride, int32_t feat, int64_t* pub_ids, float* pub_rows,
                    int64_t* pub_n, int64_t max_ids, void* stream);
int64_t hc_peer_pull_scratch_bytes(int32_t world, int64_t max_ids);
int hc_peer_pull(const void* const* peer_pub_ids, const void* const* peer_pub_rows,
                 const void* const* peer_pub_n, int32_t world, int32_t me, int64_t max_ids,
                 int32_t feat, int64_t* got_ids, float* got_rows, int64_t cap, int64_t* overflow,
                 void* scratch, void* stream);

/*
 * One rank's shard of the node-partitioned history, as hc_peer_admit needs it
 * (the members of hiscache/history_table.py:33-61 for one table, plus the
 * device-side iteration counter).  struct_size = sizeof(hc_shard).
 */
typedef struct hc_shard {
  uint32_t struct_size;
  int64_t* full_to_slot;   /* [map_len] node id -> slot or -1                  */
  int64_t map_len;
  int64_t* slot_to_full;   /* [capacity]                                       */
  int64_t* checkin;        /* [capacity] iteration of admission, -1 = free     */
  int64_t capacity;
  void* table;             /* [capacity, feat] rows, dtype                     */
  int32_t dtype;
  int32_t feat;
  int64_t* header;         /* [1] ring header                                  */
  int64_t* iter_dev;       /* [1] current iteration                            */
  int32_t* claim;          /* [map_len] int32, all -1 between calls            */
  int64_t staleness;       /* entries older than this leave; <= 0: never       */
  int64_t* n_admitted;     /* [1] rows admitted by the call, may be NULL       */
} hc_shard;

/*
 * The owner-side admission of one step in one call, on one stream:
 *   evict (when evict != 0 and staleness > 0; hc_evict_stale_dev), hc_peer_pull,
 *   last copy of an id wins (hc_last_occurrence), ids the shard already holds
 *   are skipped, ring admission with writeback (hc_record_history), check-in
 *   stamp (hc_stamp_checkin), and iter_dev[0] += 1 when advance_iter != 0.
 * got_ids [cap] / got_rows [cap, feat] fp32 are the candidate list (left
 * filled for inspection).  scratch >= hc_peer_admit_scratch_bytes(world,
 * max_ids, cap).  The ordering rules of the peer exchange apply: every rank has
 * published and finished its lookups before this call, and no rank looks up
 * again before every rank has returned from it (stream order + a collective).
 */
int64_t hc_peer_admit_scratch_bytes(int32_t world, int64_t max_ids, int64_t cap);
int hc_peer_admit(const hc_shard* shard, const void* const* peer_pub_ids,
                  const void* const* peer_pub_rows, const void* const* peer_pub_n, int32_t world,
                  int32_t me, int64_t max_ids, int64_t* got_ids, float* got_rows, int64_t cap,
                  int64_t* overflow, int32_t evict, int32_t advance_iter, void* scratch,
                  void* stream);

/* ------------------------------------------------------------------------ */
/* Neighbour sampling (stand-in for the external loader)                    */
/* ------------------------------------------------------------------------ */

/*
 * The reference takes its batches from cxgnndl.get_loader
 * (hiscache/history_trainer.py:19), a project of its own.  These entry points
 * produce the batch layout the hot path consumes (hiscache/history_model.py:
 * 120-153): uniform sampling with replacement of min(fanout, degree) neighbours
 * per frontier node, then relabelling into batch-local ids in order of first
 * occurrence.  gptr / gidx: the full graph in CSR.  Draw j of frontier position
 * i is gidx[gptr[v] + mix64(seed ^ mix64((base+i)*fanout + j)) mod deg(v)].
 *   hc_sample_counts: counts[i] = min(fanout, deg(frontier[i])).
 *   hc_sample_picks : nbr[out_ptr[i] + j] for j < out_ptr[i+1]-out_ptr[i]
 *                     (out_ptr = exclusive scan of counts).
 *   local_map: int32 [num_nodes], INT32_MIN for nodes outside the batch.
 *   hc_relabel_seed : local_map[seeds[i]] = i.
 *   hc_relabel      : nodes of nbr without a local id get n_total, n_total+1, ..
 *                     in order of first occurrence; new_nodes[r] (capacity m) and
 *                     n_new[0] (device) receive them; out_idx[p] = local id of
 *                     nbr[p].  scratch >= hc_relabel_scratch_bytes(m).
 *   hc_relabel_reset: local_map[nodes[i]] = INT32_MIN (end of a batch).
 */
int hc_sample_counts(const int64_t* gptr, const int64_t* frontier, int64_t nf, int32_t fanout,
                     int64_t* counts, void* stream);
int hc_sample_picks(const int64_t* gptr, const int64_t* gidx, const int64_t* frontier, int64_t nf,
                    int32_t fanout, const int64_t* out_ptr, uint64_t seed, int64_t base,
                    int64_t* nbr, void* stream);
int hc_relabel_seed(const int64_t* seeds, int64_t n, int32_t* local_map, void* stream);
int hc_relabel_reset(const int64_t* nodes, int64_t n, int32_t* local_map, void* stream);
int64_t hc_relabel_scratch_bytes(int64_t m);
int hc_relabel(const int64_t* nbr, int64_t m, int32_t* local_map, int64_t n_total,
               int64_t* new_nodes, int64_t* n_new, int64_t* out_idx, void* scratch, void* stream);

/*
 * A whole sampled batch in a fixed shape, with no device->host read (see the hc_sample_* notes
 * above for the draws and the layout).  caps[k] = rows of layer k (caps[0] >= number of seeds;
 * the new nodes of hop h take rows [caps[h], caps[h+1])), fanout[h] draws per node of hop h's
 * frontier, edge_cap entries of idx.  Outputs, all device: ptr int64 [caps[L-1] + 1], idx int64
 * [edge_cap] (zero behind the last edge), sub_to_full int64 [caps[L]] and mask uint8 [caps[L]]
 * (padding rows: node 0, mask 0, no neighbours), counters int64[4] = real nodes, real edges, new
 * nodes cut because their layer was full, edges cut because idx was full.  A cut node gets no row
 * and the edges to it become self loops of their destination row; a batch that fits its caps
 * (counters[2] == counters[3] == 0) equals the one hc_sample_counts / hc_sample_picks / hc_relabel
 * build for the same seeds and batch number.  seeds: n_seeds distinct nodes.  batch_no: device
 * int64, read for the draws' seed and advanced by one.  local_map as for hc_relabel; it is restored
 * before the call returns.  scratch >= hc_sample_fixed_scratch_bytes(b).
 */
typedef struct hc_fixed_batch {
  uint32_t struct_size;
  int32_t num_hops;          /* L, 1..8 */
  int32_t fanout[8];
  int64_t caps[9];
  int64_t edge_cap;
  int64_t* ptr;
  int64_t* idx;
  int64_t* sub_to_full;
  uint8_t* mask;
  int64_t* counters;
} hc_fixed_batch;
int64_t hc_sample_fixed_scratch_bytes(const hc_fixed_batch* b);
int hc_sample_fixed(const int64_t* gptr, const int64_t* gidx, const int64_t* seeds, int64_t n_seeds,
                    int32_t* local_map, uint64_t seed, int64_t* batch_no, const hc_fixed_batch* b,
                    void* scratch, void* stream);

/* ---------------------------------------------------------------------------
 * Dense epilogue of a layer: batch norm (training statistics) + ReLU + dropout.
 *
 * Replaces, for the training step, the three torch modules the reference's
 * models apply after every hidden conv (hiscache/history_model.py:141-143 for
 * SAGE, :383-385 for RGCN): y = dropout(relu(batch_norm(x))).  Forward and
 * backward are two kernels each, with no stored masks: ReLU's mask is
 * recomputed from x, dropout's from (seed, step counter, element).
 *   x [n, feat] fp32 (row stride x_stride, 0 = feat); valid: optional uint8 [n],
 *   rows with 0 stay out of the statistics and give zeros (padding rows of
 *   fixed-shape batches).  weight / bias [feat] or NULL (1 / 0).
 *   running_mean / running_var: updated as torch.nn.BatchNorm1d does
 *   (momentum, unbiased variance) or both NULL.
 *   state: device int64[4], zeroed ONCE by the caller and private to one layer:
 *     [0] dropout step counter (advanced by every forward with drop_p > 0),
 *     [1] the step the last forward used (read by its backward), [2] internal.
 *   save_mean / save_rstd [feat], save_count [1]: written by the forward, read
 *   by the backward of the same call.
 *   Column statistics are reproducible (fixed-order reduction in double).
 *   feat % 4 == 0, feat <= 1024; x, y, grads 16-byte aligned.
 *   scratch >= hc_norm_scratch_bytes(feat), 16-byte aligned; the same scratch
 *   may serve every layer (calls on one stream).
 * hc_norm_act_bwd: grad_x [n, feat]; grad_weight / grad_bias [feat] or NULL.
 */
typedef struct hc_norm_args {
  uint32_t struct_size;    /* = sizeof(hc_norm_args) */
  const float* x;
  int64_t n;
  int32_t feat;
  int64_t x_stride;
  const uint8_t* valid;
  const float* weight;
  const float* bias;
  float* running_mean;
  float* running_var;
  float momentum;
  float eps;
  float drop_p;            /* 0 <= p < 1; 0 = no dropout */
  int32_t relu;            /* 0 = identity instead of ReLU */
  uint64_t seed;
  int64_t* state;
  float* save_mean;
  float* save_rstd;
  float* save_count;
} hc_norm_args;
int64_t hc_norm_scratch_bytes(int32_t feat);
int hc_norm_act_fwd(const hc_norm_args* a, float* y, void* scratch, void* stream);
int hc_norm_act_bwd(const hc_norm_args* a, const float* grad_y, float* grad_x, float* grad_weight,
                    float* grad_bias, void* scratch, void* stream);

/* ---------------------------------------------------------------------------
 * Heterogeneous (RGCN) layers: edge types and the relation-segmented block.
 *
 * hc_edge_types: etype[e] = rel_table[type(dst) * n_types + type(src)] for the
 *   edges of rows [0, rows), where a node's type is the range of type_bounds
 *   (HOST int64 [n_types + 1], ascending) its GLOBAL id sub_to_full[.] falls
 *   in; rel_table: HOST int32 [n_types * n_types]; n_types <= 8.  Stand-in for
 *   cxgnncomp_backend.gen_edge_type_mag240m(ptr, idx, sub_to_full)
 *   (hiscache/history_model.py:354-357), which is not part of the reference.
 *
 * hc_rgcn_group: what MyRGCNConvHistory2.forward does with torch.sort before it
 *   calls RGCNOP_sorted (hiscache/history_model.py:244-266).  Edge e of row d
 *   (e in [ptr[d], ptr[d+1]), d < num_node; slots up to n_edges) keeps its
 *   relation etype[e] unless its source is unused (used_src[idx[e]] == 0, :250),
 *   d is served from history (hmap[d] != -1, optional) or etype[e] is outside
 *   [0, num_rel): then it gets num_rel and drops out.  The edges are sorted by
 *   relation with ONE stable radix pass, so inside a relation they stay in
 *   destination order.  Outputs:
 *     ptr2 int64 [num_rel * num_node + 1], idx2 int64 [n_edges], w2 fp32
 *       [n_edges]: a CSR whose row r * num_node + d lists the sources of d's
 *       relation-r edges with the weight 1 / (ptr[d+1] - ptr[d]) beside each
 *       (the reference divides by the total in-degree, :245,272);
 *       ptr2[num_rel * num_node] = number of edges kept;
 *     perm int64 [n_edges] or NULL: the sorted order (torch.sort's indices);
 *     rel_out int64 [n_edges] or NULL: the relation of every edge after
 *       pruning, in edge order (the array the reference passes to count_num).
 *   num_rel <= 255.  scratch >= hc_rgcn_group_scratch_bytes(n_edges).
 */
int hc_edge_types(const int64_t* ptr, const int64_t* idx, const int64_t* sub_to_full, int64_t rows,
                  int32_t n_types, const int64_t* type_bounds, const int32_t* rel_table,
                  int64_t* etype, void* stream);
int64_t hc_rgcn_group_scratch_bytes(int64_t n_edges);
int hc_rgcn_group(const int64_t* ptr, const int64_t* idx, const int64_t* etype, int64_t num_node,
                  int64_t n_edges, int32_t num_rel, const uint8_t* used_src, const int64_t* hmap,
                  int64_t* ptr2, int64_t* idx2, float* w2, int64_t* perm, int64_t* rel_out,
                  void* scratch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HISCACHE_B200_H */
