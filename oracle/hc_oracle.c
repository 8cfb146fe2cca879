/*
 * hc_oracle.c -- CPU restatement of the HisCache hot path.  TEST INFRASTRUCTURE.
 *
 * This file is the checker for libhiscache_b200: the parity tests, the smoke
 * check and the bench's CPU-baseline leg call it; the product library and the
 * `hiscache` package never do.  Each function restates one piece of the
 * reference (file:line given per function; paths are relative to the
 * reference project) as plain sequential C.  The *_omp variants add OpenMP
 * over independent rows and exist only to be timed as the CPU baseline.
 *
 * Parity pinning: the reference holds no golden vectors and has no CPU
 * implementation of these kernels.  The restatement is pinned (a) by running
 * the reference's own Python methods (HistoryCache.update_history /
 * lookup_and_load, HistoryTable.lookup / evict_*) on CPU tensors and
 * committing their outputs as fixtures, and (b) on a GPU, by comparing with
 * the reference's CUDA operators compiled unmodified for sm_100a.
 *
 * Build: gcc -O2 -fopenmp -fPIC -shared -std=c11 -ffp-contract=off
 * (-ffp-contract=off matters: the score reduction is defined with separately
 * rounded multiply and add; the quantile lerp calls fmaf explicitly).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* Aggregation forward: src/cpp/src/history_aggr.cu:7-125 (kernels),         */
/* :399-473 (launcher: output zero-filled, num_node default, head layout).  */
/* Extensions restated here because the CUDA library offers them: a         */
/* per-source select map (hiscache/history_cache.py:343-350 does it in      */
/* torch) and indexed history rows (hbuf[hmap[r]] instead of hbuf[r]).      */
/* acc64 != 0 accumulates in double (tolerance reference); acc64 == 0 adds  */
/* in fp32 in edge order exactly as the reference loop does.                */
/* ------------------------------------------------------------------------ */
static void aggr_fwd_row(int64_t t, const int64_t* ptr, const int64_t* idx, const float* input,
                         int64_t in_stride, int feat, int num_head, const int64_t* src_map,
                         const float* src_alt, int64_t alt_stride, const float* edge_value,
                         const int64_t* hmap, const float* hbuf, int64_t hsize, int h_indexed,
                         int acc64, float* out) {
  const int64_t r = t / num_head;
  const int h = (int)(t % num_head);
  float* orow = out + t * feat;
  if (hmap && hmap[r] != -1) {
    /* history_aggr.cu:21-25 (single head), :96-107 (multi head) */
    const int64_t hrow = h_indexed ? hmap[r] : r;
    const float* src = hbuf + hrow * hsize + (hsize == feat ? 0 : (int64_t)h * feat);
    memcpy(orow, src, sizeof(float) * (size_t)feat);
    return;
  }
  const int64_t begin = ptr[r], end = ptr[r + 1];
  for (int c = 0; c < feat; ++c) {
    double acc_d = 0.0;
    float acc_f = 0.0f;
    for (int64_t e = begin; e < end; ++e) {
      const int64_t s = idx[e];
      const int64_t al = src_map ? src_map[s] : -1;
      const float x = al != -1 ? src_alt[al * alt_stride + (int64_t)h * feat + c]
                               : input[s * in_stride + (int64_t)h * feat + c];
      const float w = edge_value ? edge_value[e * num_head + h] : 1.0f;
      if (acc64) acc_d += (double)w * (double)x;
      else acc_f = edge_value ? acc_f + x * w : acc_f + x;
    }
    if (edge_value) {
      orow[c] = acc64 ? (float)acc_d : acc_f; /* :77, :124: written even for empty rows */
    } else if (end > begin) {
      orow[c] = acc64 ? (float)(acc_d / (double)(end - begin)) : acc_f / (float)(end - begin); /* :38-39 */
    } else {
      orow[c] = 0.0f; /* output comes from new_zeros, :423-426 */
    }
  }
}

ORC_API void orc_aggr_fwd(const int64_t* ptr, const int64_t* idx, int64_t num_node,
                          const float* input, int64_t in_stride, int feat, int num_head,
                          const int64_t* src_map, const float* src_alt, int64_t alt_stride,
                          const float* edge_value, const int64_t* hmap, const float* hbuf,
                          int64_t hsize, int h_indexed, int acc64, int use_omp, float* out) {
  const int64_t targets = num_node * num_head;
  if (use_omp) {
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t t = 0; t < targets; ++t)
      aggr_fwd_row(t, ptr, idx, input, in_stride, feat, num_head, src_map, src_alt, alt_stride,
                   edge_value, hmap, hbuf, hsize, h_indexed, acc64, out);
  } else {
    for (int64_t t = 0; t < targets; ++t)
      aggr_fwd_row(t, ptr, idx, input, in_stride, feat, num_head, src_map, src_alt, alt_stride,
                   edge_value, hmap, hbuf, hsize, h_indexed, acc64, out);
  }
}

/* ------------------------------------------------------------------------ */
/* Aggregation backward: history_aggr.cu:127-397 (kernels), :493-580        */
/* (grad_input / grad_history / edge_grad are zero-filled there).           */
/* Sequential, accumulates in double, rounds once at the end.               */
/* grad_input_acc: caller-provided double scratch [n_src*num_head*feat].    */
/* ------------------------------------------------------------------------ */
ORC_API void orc_aggr_bwd(const int64_t* ptr, const int64_t* idx, int64_t num_node,
                          const float* input, int64_t in_stride, int feat, int num_head,
                          int64_t n_src, const int64_t* src_map, const float* src_alt,
                          int64_t alt_stride, const float* edge_value, const int64_t* hmap,
                          int64_t hsize, const float* grad_out, double* grad_input_acc,
                          float* grad_input, float* grad_history, float* edge_grad) {
  const int64_t row = (int64_t)num_head * feat;
  if (grad_input) memset(grad_input_acc, 0, sizeof(double) * (size_t)(n_src * row));
  if (grad_history) memset(grad_history, 0, sizeof(float) * (size_t)(num_node * hsize));
  for (int64_t t = 0; t < num_node * num_head; ++t) {
    const int64_t r = t / num_head;
    const int h = (int)(t % num_head);
    const float* g = grad_out + t * feat;
    if (hmap && hmap[r] != -1) {
      /* :143-149: no division, nothing flows to neighbours */
      if (grad_history) {
        float* dst = grad_history + r * hsize + (hsize == feat ? 0 : (int64_t)h * feat);
        for (int c = 0; c < feat; ++c) dst[c] += g[c];
      }
      continue;
    }
    const int64_t begin = ptr[r], end = ptr[r + 1];
    for (int64_t e = begin; e < end; ++e) {
      const int64_t s = idx[e];
      const int64_t al = src_map ? src_map[s] : -1;
      double dot = 0.0;
      for (int c = 0; c < feat; ++c) {
        if (grad_input && al == -1) {
          const double v = edge_value ? (double)g[c] * (double)edge_value[e * num_head + h]
                                      : (double)g[c] / (double)(end - begin);
          grad_input_acc[s * row + (int64_t)h * feat + c] += v;
        }
        if (edge_grad) {
          const float x = al != -1 ? src_alt[al * alt_stride + (int64_t)h * feat + c]
                                   : input[s * in_stride + (int64_t)h * feat + c];
          dot += (double)g[c] * (double)x; /* :246, :373 */
        }
      }
      if (edge_grad) edge_grad[e * num_head + h] = (float)dot;
    }
  }
  if (grad_input)
    for (int64_t k = 0; k < n_src * row; ++k) grad_input[k] = (float)grad_input_acc[k];
}

/* fp32 OpenMP form of the same scatter, only for CPU-baseline timing */
ORC_API void orc_aggr_bwd_omp(const int64_t* ptr, const int64_t* idx, int64_t num_node, int feat,
                              int64_t n_src, const int64_t* hmap, const float* grad_out,
                              float* grad_input) {
  memset(grad_input, 0, sizeof(float) * (size_t)(n_src * feat));
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t r = 0; r < num_node; ++r) {
    if (hmap && hmap[r] != -1) continue;
    const int64_t begin = ptr[r], end = ptr[r + 1];
    if (end == begin) continue;
    const float inv = 1.0f / (float)(end - begin);
    for (int64_t e = begin; e < end; ++e) {
      float* dst = grad_input + idx[e] * feat;
      const float* g = grad_out + r * feat;
      for (int c = 0; c < feat; ++c) {
#pragma omp atomic
        dst[c] += g[c] * inv;
      }
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Row scores: grad.norm(dim=1) of hiscache/history_cache.py:205 (kind 0)   */
/* and torch.sum(torch.abs(grad), 1) of hiscache/history_table.py:161       */
/* (kind 1), in the reduction order the CUDA library fixes: element e goes  */
/* to lane (e/4) mod 32, lanes add in increasing e with separately rounded  */
/* multiply and add, then an xor butterfly 16,8,4,2,1, then sqrt.           */
/* ------------------------------------------------------------------------ */
ORC_API void orc_score_rows(const float* x, int64_t n, int feat, int64_t stride, int kind,
                            float* score) {
  for (int64_t r = 0; r < n; ++r) {
    const float* row = x + r * stride;
    float p[32], q[32];
    for (int l = 0; l < 32; ++l) p[l] = 0.0f;
    for (int c0 = 0; c0 < feat; c0 += 128)
      for (int l = 0; l < 32; ++l)
        for (int k = 0; k < 4; ++k) {
          const int e = c0 + 4 * l + k;
          if (e < feat) {
            const float v = row[e];
            const float term = kind == 0 ? v * v : fabsf(v);
            p[l] = p[l] + term;
          }
        }
    for (int off = 16; off > 0; off >>= 1) {
      for (int l = 0; l < 32; ++l) q[l] = p[l] + p[l ^ off];
      memcpy(p, q, sizeof(p));
    }
    score[r] = kind == 0 ? sqrtf(p[0]) : p[0];
  }
}

/* ------------------------------------------------------------------------ */
/* torch.quantile(score, q) with linear interpolation, as called at          */
/* hiscache/history_cache.py:211 and hiscache/history_table.py:173,230:     */
/* rank = fp32(q)*(n-1) in fp32; below = trunc(rank); above = ceil(rank);   */
/* w = rank - below; result = lerp(sorted[below], sorted[above], w) with    */
/* torch's two-sided lerp, whose multiply-add is fused in torch's CPU (AVX2  */
/* and up) and CUDA builds: w < 0.5 ? fma(w, hi-lo, lo) : fma(-(hi-lo), 1-w, */
/* hi).  Checked bit for bit against torch.quantile on CPU by the tests.     */
/* Any NaN gives NaN.                                                        */
/* ------------------------------------------------------------------------ */
static int cmp_float_nan_last(const void* a, const void* b) {
  const float x = *(const float*)a, y = *(const float*)b;
  const int xn = x != x, yn = y != y;
  if (xn || yn) return xn - yn;
  return (x > y) - (x < y);
}

ORC_API float orc_quantile(const float* score, int64_t n, float q) {
  if (n <= 0) return NAN;
  float* s = (float*)malloc(sizeof(float) * (size_t)n);
  memcpy(s, score, sizeof(float) * (size_t)n);
  qsort(s, (size_t)n, sizeof(float), cmp_float_nan_last);
  float result;
  if (s[n - 1] != s[n - 1]) {
    result = NAN;
  } else {
    const float pos = q * (float)(n - 1);
    int64_t lo = (int64_t)pos, hi = (int64_t)ceilf(pos);
    if (lo > n - 1) lo = n - 1;
    if (hi > n - 1) hi = n - 1;
    const float w = pos - (float)lo;
    const float a = s[lo], b = s[hi];
    const float diff = b - a;
    result = fabsf(w) < 0.5f ? fmaf(w, diff, a) : fmaf(-diff, 1.0f - w, b);
  }
  free(s);
  return result;
}

/* ------------------------------------------------------------------------ */
/* Per-layer table admission: record_history_kernel_used_mask,              */
/* src/cpp/src/grad_check.cu:6-46, applied to the candidate rows one by one */
/* in ascending row order (the kernel takes ring slots with atomicInc in    */
/* scheduling order, :25; ascending order is one of its possible outcomes   */
/* and the one the CUDA library fixes).  Returns the number admitted.       */
/* ------------------------------------------------------------------------ */
ORC_API int64_t orc_record_history(const float* buffer_new, int64_t new_stride, int64_t n,
                                   float* buffer_all, int64_t capacity, int history_size,
                                   const uint8_t* used_mask, const int64_t* sub_to_full,
                                   const int64_t* sub_to_history, int64_t* history_to_full,
                                   int64_t* full_to_history, int64_t* header, const float* score,
                                   float thres, int64_t* checkin_iter, int64_t glb_iter) {
  int64_t admitted = 0;
  if (capacity <= 0) return 0;
  for (int64_t sub = 0; sub < n; ++sub) {
    /* :17-21 */
    if (sub_to_history[sub] != -1 || (thres != 0.0f && score[sub] > thres) ||
        (used_mask && used_mask[sub] == 0))
      continue;
    /* :25 atomicInc(header, history_num - 1): returns old, wraps to 0 */
    const int64_t slot = header[0];
    header[0] = (slot >= capacity - 1) ? 0 : slot + 1;
    /* :26-30 unmap the previous owner only if it still points here */
    const int64_t old = history_to_full[slot];
    if (old != -1 && full_to_history[old] == slot) full_to_history[old] = -1;
    /* :34-38 */
    memcpy(buffer_all + slot * history_size, buffer_new + sub * new_stride,
           sizeof(float) * (size_t)history_size);
    /* :40-45 */
    const int64_t full = sub_to_full[sub];
    full_to_history[full] = slot;
    history_to_full[slot] = full;
    checkin_iter[slot] = glb_iter;
    ++admitted;
  }
  return admitted;
}

/* ------------------------------------------------------------------------ */
/* Unified-buffer admission: hiscache/history_cache.py:213-254, statement   */
/* by statement (the vectorised torch ops become loops; reads of the maps   */
/* happen before the writes of the same statement, as in torch).  One       */
/* deviation, shared with the CUDA library: rows that would run past        */
/* embed_capacity are not admitted (the reference has no bound check).      */
/* full2embed has 2*N+1 entries; index -1 is its last entry (:42-46).       */
/* ------------------------------------------------------------------------ */
ORC_API int64_t orc_cache_admit(const float* produced, int64_t prod_stride, int64_t n,
                                float* buffer, int hidden, int in_feat, int64_t embed_capacity,
                                const int64_t* sub_to_full, const int64_t* sub2embed,
                                const float* score, float thres, int64_t* full2embed,
                                int64_t total_num_node, int64_t* embed2full,
                                const int64_t* feat2full, int64_t feat2full_len, int64_t* header,
                                int reset_header, uint8_t* record_mask_out) {
  const int64_t map_len = 2 * total_num_node + 1;
  if (reset_header) header[0] = 0; /* :190-192 */
  const int64_t h0 = header[0];
  /* :215 record_mask = (grad < thres) & (sub2embed == -1) */
  int64_t num = 0;
  const int64_t room = embed_capacity > h0 ? embed_capacity - h0 : 0;
  int64_t* rows = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1));
  for (int64_t r = 0; r < n; ++r) {
    const int m = (score[r] < thres) && (sub2embed[r] == -1) && (num < room);
    if (record_mask_out) record_mask_out[r] = (uint8_t)m;
    if (m) rows[num++] = r;
  }
  /* :219-221 append rows at [header, header+num) of the [-1, hidden] view */
  for (int64_t k = 0; k < num; ++k)
    memcpy(buffer + (h0 + k) * hidden, produced + rows[k] * prod_stride,
           sizeof(float) * (size_t)hidden);
  /* :223-226 raw-feature slots overlapped by the new rows lose their mapping */
  {
    int64_t begin = h0 * hidden / in_feat;
    int64_t end = ((h0 + num) * hidden + in_feat - 1) / in_feat;
    if (end > feat2full_len) end = feat2full_len; /* python slice clipping */
    for (int64_t k = begin; k < end; ++k) full2embed[feat2full[k]] = -1;
  }
  /* :230-240 previous owners of the overwritten embedding slots */
  for (int64_t k = 0; k < num; ++k) {
    int64_t g = embed2full[h0 + k];
    if (g < 0) g += map_len; /* -1 -> the dummy last entry */
    const int64_t cur = full2embed[g];
    if (cur >= h0 && cur < h0 + num) full2embed[g] = -1;
  }
  /* :243-254 */
  for (int64_t k = 0; k < num; ++k) {
    const int64_t id = sub_to_full[rows[k]];
    full2embed[id] = h0 + k;
    embed2full[h0 + k] = id;
  }
  header[0] = h0 + num;
  free(rows);
  return num;
}

/* hiscache/history_table.py:189-200 (and :244-251) */
ORC_API void orc_evict_stale(int64_t* checkin, int64_t* h2f, int64_t* f2h, int64_t capacity,
                             int64_t glb_iter, int64_t limit) {
  const int64_t stale = glb_iter - limit;
  for (int64_t s = 0; s < capacity; ++s)
    if (checkin[s] > -1 && checkin[s] <= stale) {
      const int64_t full = h2f[s];
      checkin[s] = -1;
      h2f[s] = -1;
      if (full != -1) f2h[full] = -1;
    }
}

/* hiscache/history_table.py:234-241 */
ORC_API void orc_evict_by_score(const int64_t* sub_to_history, const float* score, float thres,
                                int64_t n, int64_t* checkin, int64_t* h2f, int64_t* f2h) {
  for (int64_t r = 0; r < n; ++r) {
    const int64_t slot = sub_to_history[r];
    if (slot == -1 || !(score[r] >= thres)) continue;
    const int64_t full = h2f[slot];
    if (full != -1) f2h[full] = -1;
    h2f[slot] = -1;
    checkin[slot] = -1;
  }
}

/* ------------------------------------------------------------------------ */
/* Used masks: count_history_reconstruct / count_history_kernel,            */
/* src/cpp/src/grad_check.cu:70-130.  masks: (num_layer+1) x num_node       */
/* bytes, masks[k] at masks + k*num_node.                                   */
/* ------------------------------------------------------------------------ */
/* one launch of count_history_kernel (:70-101); seeds_first marks rows < num_seed in `in` */
ORC_API void orc_used_mask_step(const int64_t* ptr, const int64_t* idx, int64_t ptr_rows,
                                const int64_t* hmap, int64_t hmap_len, uint8_t* in, uint8_t* out,
                                int64_t num_seed, int seeds_first) {
  for (int64_t row = 0; row < ptr_rows; ++row) {
    if (seeds_first && row < num_seed) in[row] = 1; /* :79-82 */
    else if (in[row] != 1) continue;
    if (hmap && row < hmap_len && hmap[row] != -1) continue; /* :87-90 */
    out[row] = 1;                                            /* :92-94 */
    for (int64_t e = ptr[row]; e < ptr[row + 1]; ++e) out[idx[e]] = 1;
  }
}

ORC_API void orc_used_masks(const int64_t* ptr, const int64_t* idx, int64_t ptr_rows,
                            const int64_t* history_map, int64_t history_map_len,
                            int64_t num_node, int64_t num_seed, int num_layer, uint8_t* masks) {
  memset(masks, 0, (size_t)((num_layer + 1) * num_node));
  for (int i = 0; i < num_layer; ++i) {
    uint8_t* in = masks + (int64_t)(num_layer - i) * num_node;
    uint8_t* out = masks + (int64_t)(num_layer - 1 - i) * num_node;
    /* the history map is passed to the second launch only (:122-124) */
    orc_used_mask_step(ptr, idx, ptr_rows, (i == 1) ? history_map : NULL, history_map_len, in,
                       out, num_seed, i == 0);
  }
}

/* ------------------------------------------------------------------------ */
/* Structure score: get_graph_structure_score, grad_check.cu:132-163.  The  */
/* reference propagates in place with racing warps; this is its             */
/* level-synchronous reading: a node unset before a step takes              */
/* score(parent)*deg(parent) of its lowest-numbered parent set before it.   */
/* ------------------------------------------------------------------------ */
ORC_API void orc_structure_score(const int64_t* ptr, const int64_t* idx, int64_t ptr_rows,
                                 int64_t num_node, int64_t num_seed, int num_layer,
                                 int64_t* output) {
  memset(output, 0, sizeof(int64_t) * (size_t)num_node);
  if (num_layer <= 0) return;
  int64_t* prev = (int64_t*)malloc(sizeof(int64_t) * (size_t)(num_node > 0 ? num_node : 1));
  for (int64_t r = 0; r < num_seed && r < ptr_rows; ++r) output[r] = 1;
  for (int i = 0; i < num_layer; ++i) {
    memcpy(prev, output, sizeof(int64_t) * (size_t)num_node);
    for (int64_t row = 0; row < ptr_rows; ++row) {
      if (prev[row] == 0) continue;
      const int64_t deg = ptr[row + 1] - ptr[row];
      for (int64_t e = ptr[row]; e < ptr[row + 1]; ++e) {
        const int64_t v = idx[e];
        /* ascending rows: the first parent to reach v is its lowest-numbered one */
        if (prev[v] == 0 && output[v] == 0) output[v] = prev[row] * deg;
      }
    }
  }
  free(prev);
}

/* count_num, grad_check.cu:165-182: value 0 is never counted (:169) */
ORC_API void orc_count_num(const int64_t* arr, int64_t n, int64_t mmax, int32_t* output) {
  memset(output, 0, sizeof(int32_t) * (size_t)(mmax + 1));
  for (int64_t i = 0; i < n; ++i)
    if (arr[i] != 0 && arr[i] > 0 && arr[i] <= mmax) output[arr[i]] += 1;
}

/* splitmix64 finaliser, the owner hash of the sharded table (no reference   */
/* counterpart: hiscache/history_cache.py:72-78 splits the feature axis).    */
ORC_API uint64_t orc_mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
