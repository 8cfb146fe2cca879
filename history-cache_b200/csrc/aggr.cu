// History-aware CSR gather-reduce (forward) and transposed scatter (backward).
//
// Replaces the eight kernels of the reference's src/cpp/src/history_aggr.cu
// (:7-397) and their launchers (:399-596).  The reference splits one row over
// F/32 warps of scalar 4-byte lanes, each re-reading ptr / idx / hmap; here
// one warp owns a whole destination row, every lane moves 16 bytes per
// request, narrow rows are shared by several edges per request, and the
// choice between a fresh source row, an alternative (cached) source row and a
// history row is made inside the gather.  Memory bound: no tensor cores.
#include "common.cuh"

namespace hc {

// ---------------------------------------------------------------------------
// index checks of the HC_CHECK_BOUNDS build: a validation pass over the block records the first
// index that lies outside its table; while the status word is set the operator kernels return at
// once, so no out-of-range access is ever made and nothing traps.
// ---------------------------------------------------------------------------
#ifdef HC_CHECK_BOUNDS
static __device__ unsigned long long g_status[4];   // code, which array, position, value

__device__ __forceinline__ void status_set(int which, int64_t pos, int64_t value) {
  if (atomicCAS(&g_status[0], 0ull, (unsigned long long)HC_ERR_RANGE) == 0ull) {
    g_status[1] = (unsigned long long)which;
    g_status[2] = (unsigned long long)pos;
    g_status[3] = (unsigned long long)value;
  }
}

__global__ void __launch_bounds__(256) aggr_check_kernel(const hc_aggr_args a) {
  constexpr int G = 8;
  const int gl = threadIdx.x & (G - 1);
  const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (r >= a.num_node) return;
  const int64_t b = a.ptr[r], e_end = a.ptr[r + 1];
  if (gl == 0) {
    if (b < 0 || e_end < b) status_set(1, r, e_end < b ? e_end : b);
    if (a.hmap) {
      const int64_t h = a.hmap[r];
      const int64_t rows = a.h_rows;
      if (h < -1 || (a.h_indexed && rows > 0 && h >= rows) || (!a.h_indexed && h != -1 && rows > 0 && r >= rows))
        status_set(4, r, h);
    }
  }
  if (b < 0 || e_end < b) return;
  for (int64_t e = b + gl; e < e_end; e += G) {
    const int64_t s = a.idx[e];
    if (s < 0 || s >= a.n_src) {
      status_set(2, e, s);
      continue;
    }
    if (a.src_map) {
      const int64_t m = a.src_map[s];
      if (m < -1 || (a.alt_rows > 0 && m >= a.alt_rows)) status_set(3, s, m);
    }
  }
}
#define HC_BAIL_IF_BAD() \
  if (g_status[0] != 0ull) return;
#else
#define HC_BAIL_IF_BAD()
#endif

// ---------------------------------------------------------------------------
// history row -> fp32 output row
// ---------------------------------------------------------------------------
__device__ __forceinline__ void copy_history_row(const hc_aggr_args& a, int64_t hrow, int head,
                                                 float* __restrict__ orow, int lane, int h_vec) {
  const int F = a.feat;
  const int64_t off = hrow * a.hsize + (a.hsize == F ? 0 : (int64_t)head * F);
  if (h_vec) {
    if (a.h_dtype == HC_F32) {
      const float* src = reinterpret_cast<const float*>(a.hbuf) + off;
      for (int v = lane; v < (F >> 2); v += kWarp)
        reinterpret_cast<uint4*>(orow)[v] = ldg16(src + 4 * v);
    } else {
      const __half* src = reinterpret_cast<const __half*>(a.hbuf) + off;
      for (int v = lane; v < (F >> 3); v += kWarp) {
        float f[8];
        Vec16<__half>::unpack(ldg16(src + 8 * v), f);
        reinterpret_cast<float4*>(orow)[2 * v] = make_float4(f[0], f[1], f[2], f[3]);
        reinterpret_cast<float4*>(orow)[2 * v + 1] = make_float4(f[4], f[5], f[6], f[7]);
      }
    }
  } else {
    for (int c = lane; c < F; c += kWarp) orow[c] = load_as_f32(a.hbuf, a.h_dtype, off + c);
  }
}

// ---------------------------------------------------------------------------
// forward, 16-byte vector path (num_head == 1)
//   T   storage type of source rows
//   G   lanes that share one source row (G < 32: 32/G edges per request)
//   V   16-byte vectors per lane
//   EV  weighted sum with edge values instead of mean
//   IDX32  source ids fit 31 bits (n_src < 2^31): they travel in one shuffle
// ---------------------------------------------------------------------------
// Tuning, measured on B200 with 2 M x 10-neighbour blocks larger than L2: throughput follows
// the bytes in flight per SM (resident warps x U x 16 B per lane).  Six independent loads
// per lane cover a sampled row (<= 12 edges of 256 B, <= 6 of 512 B) in one batch, and 48
// registers keep five blocks resident; more unrolling or forcing more blocks spills and
// loses (U=4: 4.3 TB/s, U=6 @5 blocks: 5.1 TB/s, U=8: 3.8 TB/s for fp16 dim-128 rows).
// Two other layouts were built and measured on the same block and lost: staging each block's
// idx slice in shared memory with one lane group per row (3.7 TB/s), and fetching every
// source row with the bulk-copy engine into a double-buffered shared-memory ring (4.1 TB/s:
// the engine tops out near 13 G row copies/s, below the 16 G rows/s the register path moves).
#ifndef HC_FWD_MINBLOCKS
#define HC_FWD_MINBLOCKS 5
#endif
#ifndef HC_FWD_U1
#define HC_FWD_U1 6
#endif
//   MH  several heads: a warp owns one (row, head) target; with MH == false the head arithmetic
//       folds away and the kernel is the single-head one
template <typename T, int G, int V, bool EV, bool IDX32, bool MH = false>
__global__ void __launch_bounds__(256, HC_FWD_MINBLOCKS)
    aggr_fwd_vec_kernel(const hc_aggr_args a, float* __restrict__ out, const int nvec,
                        const int h_vec) {
  HC_BAIL_IF_BAD()
  constexpr int EL = Vec16<T>::kElems;
  constexpr int EPW = kWarp / G;
  constexpr int U = V == 1 ? HC_FWD_U1 : (V == 2 ? 4 : (V <= 4 ? 2 : 1));
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int H = MH ? a.num_head : 1;
  if (t >= a.num_node * H) return;
  const int64_t r = MH ? t / H : t;
  const int h = MH ? (int)(t - r * H) : 0;
  const int F = a.feat;
  float* __restrict__ orow = out + t * F;

  const int64_t hid = a.hmap ? a.hmap[r] : -1;
  if (hid != -1) {
    copy_history_row(a, a.h_indexed ? hid : r, h, orow, lane, h_vec);
    return;
  }

  const int sub = lane / G, gl = lane % G;
  float acc[V][EL];
#pragma unroll
  for (int k = 0; k < V; ++k)
#pragma unroll
    for (int e = 0; e < EL; ++e) acc[k][e] = 0.f;

  const int64_t begin = a.ptr[r], end = a.ptr[r + 1];
  const T* __restrict__ in = reinterpret_cast<const T*>(a.input) + (MH ? (int64_t)h * F : 0);
  const T* __restrict__ alt = reinterpret_cast<const T*>(a.src_alt) + (MH ? (int64_t)h * F : 0);
  const bool has_map = a.src_map != nullptr;

  for (int64_t i = begin; i < end; i += kWarp) {
    int64_t my_s = 0, my_alt = -1;
    float my_w = 0.f;
    if (i + lane < end) {
      my_s = a.idx[i + lane];
      if (has_map) my_alt = a.src_map[my_s];
      if (EV) my_w = MH ? a.edge_value[(i + lane) * H + h] : a.edge_value[i + lane];
    }
    const int cnt = (int)((end - i) < (int64_t)kWarp ? (end - i) : (int64_t)kWarp);
    for (int j = 0; j < cnt; j += EPW * U) {
      uint4 buf[U][V];
      float w[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int jj = j + u * EPW + sub;
        const int from = jj & 31;
        const int64_t s = IDX32 ? (int64_t)__shfl_sync(kFull, (int)my_s, from) : shfl64(my_s, from);
        const int64_t al = has_map ? shfl64(my_alt, from) : -1;
        w[u] = EV ? __shfl_sync(kFull, my_w, from) : 1.f;
        const bool ok = jj < cnt;
        if (EV && !ok) w[u] = 0.f;
        const T* row = (al != -1) ? alt + al * a.alt_stride : in + s * a.in_stride;
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int v = gl + k * G;
          buf[u][k] = (ok && v < nvec) ? ldg16(row + v * EL) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (j + u * EPW < cnt) {  // warp-uniform: slots past the end of the chunk do nothing
#pragma unroll
          for (int k = 0; k < V; ++k) {
            if (EV) {
              float f[EL];
              Vec16<T>::unpack(buf[u][k], f);
#pragma unroll
              for (int e = 0; e < EL; ++e) acc[k][e] = fmaf(w[u], f[e], acc[k][e]);
            } else {
              accumulate_vec<T>(acc[k], buf[u][k]);
            }
          }
        }
      }
    }
  }

  if (EPW > 1) {
#pragma unroll
    for (int off = G; off < kWarp; off <<= 1)
#pragma unroll
      for (int k = 0; k < V; ++k)
#pragma unroll
        for (int e = 0; e < EL; ++e) acc[k][e] += __shfl_xor_sync(kFull, acc[k][e], off);
  }
  if (sub != 0) return;

  const int64_t deg = end - begin;
  if (!EV && deg > 0) {
    const float inv = __frcp_rn((float)deg);  // one correctly rounded reciprocal per row
#pragma unroll
    for (int k = 0; k < V; ++k)
#pragma unroll
      for (int e = 0; e < EL; ++e) acc[k][e] *= inv;
  }
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int v = gl + k * G;
    if (v < nvec) {
      float4* dst = reinterpret_cast<float4*>(orow + v * EL);
      dst[0] = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
      if (EL == 8) dst[1] = make_float4(acc[k][EL - 4], acc[k][EL - 3], acc[k][EL - 2], acc[k][EL - 1]);
    }
  }
}

// ---------------------------------------------------------------------------
// forward, generic path: any F, any dtype mix, multi-head
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    aggr_fwd_generic_kernel(const hc_aggr_args a, float* __restrict__ out) {
  HC_BAIL_IF_BAD()
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int H = a.num_head, F = a.feat;
  if (t >= a.num_node * H) return;
  const int64_t r = t / H;
  const int h = (int)(t % H);
  float* __restrict__ orow = out + t * F;
  const int64_t hid = a.hmap ? a.hmap[r] : -1;
  if (hid != -1) {
    copy_history_row(a, a.h_indexed ? hid : r, h, orow, lane, 0);
    return;
  }
  const int64_t begin = a.ptr[r], end = a.ptr[r + 1];
  const int64_t deg = end - begin;
  const bool ev = a.edge_value != nullptr;
  for (int c0 = 0; c0 < F; c0 += 128) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t e = begin; e < end; ++e) {
      const int64_t s = a.idx[e];
      const int64_t al = a.src_map ? a.src_map[s] : -1;
      const float w = ev ? a.edge_value[e * H + h] : 1.f;
      const void* base = al != -1 ? a.src_alt : a.input;
      const int dt = al != -1 ? a.alt_dtype : a.in_dtype;
      const int64_t off = (al != -1 ? al * a.alt_stride : s * a.in_stride) + (int64_t)h * F;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + lane + 32 * k;
        if (c < F) acc[k] = fmaf(w, load_as_f32(base, dt, off + c), acc[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + lane + 32 * k;
      if (c < F) orow[c] = (!ev && deg > 0) ? __fdiv_rn(acc[k], (float)deg) : acc[k];
    }
  }
}

// ---------------------------------------------------------------------------
// backward, 16-byte vector path
//   MH  several heads (one warp per (row, head) target; fp32 source rows)
//   EG  also the gradient of the edge values: edge_grad[e(, h)] = <grad_out[t], source row>, the
//       dot product taken by the G lanes that share the row and written once (every edge of every
//       head belongs to exactly one target, so no atomics)
// ---------------------------------------------------------------------------
template <int G, int V, bool EV, bool MH = false, bool EG = false>
__global__ void __launch_bounds__(256)
    aggr_bwd_vec_kernel(const hc_aggr_args a, const float* __restrict__ grad_out,
                        float* __restrict__ grad_input, float* __restrict__ grad_history,
                        float* __restrict__ row_score_out, const int score_kind, const int nvec,
                        const int64_t gi_stride, float* __restrict__ edge_grad) {
  HC_BAIL_IF_BAD()
  constexpr int EPW = kWarp / G;
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int H = MH ? a.num_head : 1;
  if (t >= a.num_node * H) return;
  const int64_t r = MH ? t / H : t;
  const int h = MH ? (int)(t - r * H) : 0;
  const int F = a.feat;
  const int sub = lane / G, gl = lane % G;

  float4 g[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int v = gl + k * G;
    g[k] = v < nvec ? __ldg(reinterpret_cast<const float4*>(grad_out + t * F) + v)
                    : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  if (!MH && row_score_out) {
    float p = 0.f;
    if (sub == 0) {
#pragma unroll
      for (int k = 0; k < V; ++k) {
        p = score_term(p, g[k].x, score_kind);
        p = score_term(p, g[k].y, score_kind);
        p = score_term(p, g[k].z, score_kind);
        p = score_term(p, g[k].w, score_kind);
      }
    }
    p = score_finish(p, score_kind);
    if (lane == 0) row_score_out[r] = p;
  }

  const int64_t hid = a.hmap ? a.hmap[r] : -1;
  if (grad_history && sub == 0) {
    // per-head history rows (hsize == num_head * feat) or a single head
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    float* hrow = grad_history + r * a.hsize + (MH ? (int64_t)h * F : 0);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int v = gl + k * G;
      if (v < nvec) reinterpret_cast<float4*>(hrow)[v] = hid != -1 ? g[k] : z;
    }
  }
  const int64_t begin = a.ptr[r], end = a.ptr[r + 1];
  if (hid != -1) {
    // edges of a history row carry no gradient (zeros_like in the reference, :536)
    if (EG)
      for (int64_t e = begin + lane; e < end; e += kWarp) edge_grad[MH ? e * H + h : e] = 0.f;
    return;
  }
  if (grad_input == nullptr && !EG) return;
  const int64_t deg = end - begin;
  if (deg == 0) return;
  if (!EV) {
    const float inv = __frcp_rn((float)deg);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      g[k].x *= inv;
      g[k].y *= inv;
      g[k].z *= inv;
      g[k].w *= inv;
    }
  }
  const bool has_map = a.src_map != nullptr;
  const float* __restrict__ in = reinterpret_cast<const float*>(a.input) + (MH ? (int64_t)h * F : 0);
  const float* __restrict__ alt = reinterpret_cast<const float*>(a.src_alt) + (MH ? (int64_t)h * F : 0);
  for (int64_t i = begin; i < end; i += kWarp) {
    int64_t my_s = 0, my_alt = -1;
    float my_w = 0.f;
    if (i + lane < end) {
      my_s = a.idx[i + lane];
      if (has_map) my_alt = a.src_map[my_s];
      if (EV) my_w = MH ? a.edge_value[(i + lane) * H + h] : a.edge_value[i + lane];
    }
    const int cnt = (int)((end - i) < (int64_t)kWarp ? (end - i) : (int64_t)kWarp);
    for (int j = 0; j < cnt; j += EPW) {
      const int jj = j + sub;
      const int from = jj & 31;
      const int64_t s = shfl64(my_s, from);
      const int64_t al = has_map ? shfl64(my_alt, from) : -1;
      const float w = EV ? __shfl_sync(kFull, my_w, from) : 1.f;
      const bool ok = jj < cnt;
      if (EG) {
        float dot = 0.f;
        if (ok) {
          const float* row = al != -1 ? alt + al * a.alt_stride : in + s * a.in_stride;
#pragma unroll
          for (int k = 0; k < V; ++k) {
            const int v = gl + k * G;
            if (v < nvec) {
              const float4 x = __ldg(reinterpret_cast<const float4*>(row) + v);
              dot = fmaf(g[k].x, x.x, dot);
              dot = fmaf(g[k].y, x.y, dot);
              dot = fmaf(g[k].z, x.z, dot);
              dot = fmaf(g[k].w, x.w, dot);
            }
          }
        }
#pragma unroll
        for (int off = 1; off < G; off <<= 1) dot += __shfl_xor_sync(kFull, dot, off);
        if (ok && gl == 0) edge_grad[MH ? (i + jj) * H + h : (i + jj)] = dot;
      }
      if (ok && al == -1 && grad_input != nullptr) {
        float* dst = grad_input + s * gi_stride + (MH ? (int64_t)h * F : 0);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int v = gl + k * G;
          if (v < nvec) {
            if (EV)
              red_add_v4(dst + 4 * v, g[k].x * w, g[k].y * w, g[k].z * w, g[k].w * w);
            else
              red_add_v4(dst + 4 * v, g[k].x, g[k].y, g[k].z, g[k].w);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// backward, generic path: any F, multi-head, edge_grad
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    aggr_bwd_generic_kernel(const hc_aggr_args a, const float* __restrict__ grad_out,
                            float* __restrict__ grad_input, float* __restrict__ grad_history,
                            float* __restrict__ edge_grad, float* __restrict__ row_score_out,
                            const int score_kind, const int64_t gi_stride) {
  HC_BAIL_IF_BAD()
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int H = a.num_head, F = a.feat;
  if (t >= a.num_node * H) return;
  const int64_t r = t / H;
  const int h = (int)(t % H);
  const float* __restrict__ grow = grad_out + t * F;
  if (row_score_out && H == 1) {
    const float s = row_score(grow, F, score_kind, lane);
    if (lane == 0) row_score_out[r] = s;
  }
  const int64_t hid = a.hmap ? a.hmap[r] : -1;
  const bool heads_share_history = H > 1 && a.hsize == F;
  if (grad_history) {
    float* dst = grad_history + r * a.hsize + (a.hsize == F ? 0 : (int64_t)h * F);
    if (heads_share_history) {
      // all heads of a hit row add into one row; the launcher cleared it
      if (hid != -1)
        for (int c = lane; c < F; c += kWarp) atomicAdd(dst + c, grow[c]);
    } else {
      for (int c = lane; c < F; c += kWarp) dst[c] = hid != -1 ? grow[c] : 0.f;
    }
  }
  const int64_t begin = a.ptr[r], end = a.ptr[r + 1];
  if (hid != -1) {
    // edges of a history row carry no gradient (zeros_like in the reference, :536)
    if (edge_grad)
      for (int64_t e = begin + lane; e < end; e += kWarp) edge_grad[e * H + h] = 0.f;
    return;
  }
  if (grad_input == nullptr && edge_grad == nullptr) return;
  const int64_t deg = end - begin;
  const bool ev = a.edge_value != nullptr;
  for (int64_t e = begin; e < end; ++e) {
    const int64_t s = a.idx[e];
    const int64_t al = a.src_map ? a.src_map[s] : -1;
    const float w = ev ? a.edge_value[e * H + h] : 1.f;
    float dot = 0.f;
    for (int c = lane; c < F; c += kWarp) {
      const float gv = grow[c];
      if (grad_input && al == -1) {
        const float val = ev ? gv * w : __fdiv_rn(gv, (float)deg);
        atomicAdd(grad_input + s * gi_stride + (int64_t)h * F + c, val);
      }
      if (edge_grad) {
        const void* base = al != -1 ? a.src_alt : a.input;
        const int dt = al != -1 ? a.alt_dtype : a.in_dtype;
        const int64_t off = (al != -1 ? al * a.alt_stride : s * a.in_stride) + (int64_t)h * F;
        dot = fmaf(gv, load_as_f32(base, dt, off + c), dot);
      }
    }
    if (edge_grad) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(kFull, dot, off);
      if (lane == 0) edge_grad[e * H + h] = dot;
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int validate(const hc_aggr_args* a, hc_aggr_args* n) {
  HC_REQUIRE(a != nullptr, HC_ERR_NULL);
  HC_REQUIRE(a->struct_size == sizeof(hc_aggr_args), HC_ERR_STRUCT);
  *n = *a;
  HC_REQUIRE(n->num_node >= 0 && n->feat > 0 && n->num_head >= 1 && n->n_src >= 0, HC_ERR_SIZE);
  if (n->num_node == 0) return 0;
  HC_REQUIRE(n->ptr && n->idx && n->input, HC_ERR_NULL);
  HC_REQUIRE(dtype_size(n->in_dtype) != 0, HC_ERR_DTYPE);
  const int64_t row = (int64_t)n->num_head * n->feat;
  if (n->in_stride == 0) n->in_stride = row;
  HC_REQUIRE(n->in_stride >= row, HC_ERR_SIZE);
  HC_REQUIRE(aligned_to(n->ptr, 8) && aligned_to(n->idx, 8), HC_ERR_ALIGN);
  HC_REQUIRE(aligned_to(n->input, dtype_size(n->in_dtype)), HC_ERR_ALIGN);
  if (n->src_map) {
    HC_REQUIRE(n->src_alt != nullptr, HC_ERR_NULL);
    HC_REQUIRE(dtype_size(n->alt_dtype) != 0, HC_ERR_DTYPE);
    if (n->alt_stride == 0) n->alt_stride = row;
    HC_REQUIRE(n->alt_stride >= row, HC_ERR_SIZE);
  }
  if (n->hmap) {
    HC_REQUIRE(n->hbuf != nullptr, HC_ERR_NULL);
    HC_REQUIRE(dtype_size(n->h_dtype) != 0, HC_ERR_DTYPE);
    // history rows are either shared by the heads or one segment per head
    // (the reference asserts on the device: history_aggr.cu:97-106)
    HC_REQUIRE(n->hsize >= n->feat, HC_ERR_SIZE);
    HC_REQUIRE(n->num_head == 1 || n->hsize == n->feat || n->hsize == row, HC_ERR_SIZE);
  }
  return 0;
}

static int vec_shape(int nvec, int* G, int* V) {
  if (nvec <= 8) { *G = 8; *V = 1; }
  else if (nvec <= 16) { *G = 16; *V = 1; }
  else if (nvec <= 32) { *G = 32; *V = 1; }
  else if (nvec <= 64) { *G = 32; *V = 2; }
  else if (nvec <= 96) { *G = 32; *V = 3; }
  else if (nvec <= 128) { *G = 32; *V = 4; }
  else if (nvec <= 192) { *G = 32; *V = 6; }
  else if (nvec <= 256) { *G = 32; *V = 8; }
  else return 0;
  return 1;
}

// several heads (edge-weighted sums only; source ids must fit 31 bits)
template <typename T>
static void launch_fwd_heads(int G, int V, dim3 grid, cudaStream_t st, const hc_aggr_args& a,
                             float* out, int nvec, int h_vec) {
#define HC_FWD_CASE(g, v)                                                                          \
  if (G == g && V == v) {                                                                          \
    aggr_fwd_vec_kernel<T, g, v, true, true, true><<<grid, 256, 0, st>>>(a, out, nvec, h_vec);     \
    return;                                                                                        \
  }
  HC_FWD_CASE(8, 1) HC_FWD_CASE(16, 1) HC_FWD_CASE(32, 1) HC_FWD_CASE(32, 2)
  HC_FWD_CASE(32, 3) HC_FWD_CASE(32, 4) HC_FWD_CASE(32, 6) HC_FWD_CASE(32, 8)
#undef HC_FWD_CASE
}

template <typename T, bool EV>
static void launch_fwd_vec(int G, int V, dim3 grid, cudaStream_t st, const hc_aggr_args& a,
                           float* out, int nvec, int h_vec) {
  const bool idx32 = a.n_src < 0x7fffffffLL;
#define HC_FWD_CASE(g, v)                                                                     \
  if (G == g && V == v) {                                                                     \
    if (idx32) aggr_fwd_vec_kernel<T, g, v, EV, true><<<grid, 256, 0, st>>>(a, out, nvec, h_vec);  \
    else aggr_fwd_vec_kernel<T, g, v, EV, false><<<grid, 256, 0, st>>>(a, out, nvec, h_vec);  \
    return;                                                                                   \
  }
  HC_FWD_CASE(8, 1) HC_FWD_CASE(16, 1) HC_FWD_CASE(32, 1) HC_FWD_CASE(32, 2)
  HC_FWD_CASE(32, 3) HC_FWD_CASE(32, 4) HC_FWD_CASE(32, 6) HC_FWD_CASE(32, 8)
#undef HC_FWD_CASE
}

template <bool EV>
static void launch_bwd_vec(int G, int V, dim3 grid, cudaStream_t st, const hc_aggr_args& a,
                           const float* grad_out, float* grad_input, float* grad_history,
                           float* row_score, int score_kind, int nvec, int64_t gi_stride) {
#define HC_BWD_CASE(g, v)                                                                  \
  if (G == g && V == v) {                                                                  \
    aggr_bwd_vec_kernel<g, v, EV><<<grid, 256, 0, st>>>(a, grad_out, grad_input,           \
                                                        grad_history, row_score,           \
                                                        score_kind, nvec, gi_stride, nullptr); \
    return;                                                                                \
  }
  HC_BWD_CASE(8, 1) HC_BWD_CASE(16, 1) HC_BWD_CASE(32, 1) HC_BWD_CASE(32, 2)
  HC_BWD_CASE(32, 3) HC_BWD_CASE(32, 4) HC_BWD_CASE(32, 6) HC_BWD_CASE(32, 8)
#undef HC_BWD_CASE
}

// edge-weighted backward with several heads and / or the gradient of the edge values (fp32 rows)
template <bool MH, bool EG>
static void launch_bwd_heads(int G, int V, dim3 grid, cudaStream_t st, const hc_aggr_args& a,
                             const float* grad_out, float* grad_input, float* grad_history,
                             float* row_score, int score_kind, int nvec, int64_t gi_stride,
                             float* edge_grad) {
#define HC_BWD_CASE(g, v)                                                                          \
  if (G == g && V == v) {                                                                          \
    aggr_bwd_vec_kernel<g, v, true, MH, EG><<<grid, 256, 0, st>>>(a, grad_out, grad_input,         \
                                                                  grad_history, row_score,         \
                                                                  score_kind, nvec, gi_stride,     \
                                                                  edge_grad);                      \
    return;                                                                                        \
  }
  HC_BWD_CASE(8, 1) HC_BWD_CASE(16, 1) HC_BWD_CASE(32, 1) HC_BWD_CASE(32, 2)
  HC_BWD_CASE(32, 3) HC_BWD_CASE(32, 4) HC_BWD_CASE(32, 6) HC_BWD_CASE(32, 8)
#undef HC_BWD_CASE
}

}  // namespace hc

using namespace hc;

#ifdef HC_CHECK_BOUNDS
#define HC_CHECK_BLOCK(a, st)                                                                 \
  do {                                                                                        \
    const int64_t cb_ = ceil_div((a).num_node * 8, 256);                                      \
    HC_REQUIRE(cb_ <= 0x7fffffffLL, HC_ERR_SIZE);                                             \
    aggr_check_kernel<<<(unsigned)cb_, 256, 0, st>>>(a);                                      \
  } while (0)
#else
#define HC_CHECK_BLOCK(a, st)
#endif

extern "C" int hc_last_status(int64_t out[4], int32_t clear, void* stream) {
#ifdef HC_CHECK_BOUNDS
  HC_REQUIRE(out != nullptr, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  HC_CUDA(cudaStreamSynchronize(st));
  unsigned long long h[4];
  HC_CUDA(cudaMemcpyFromSymbol(h, g_status, sizeof(h)));
  for (int i = 0; i < 4; ++i) out[i] = (int64_t)h[i];
  if (clear) {
    const unsigned long long z[4] = {0, 0, 0, 0};
    HC_CUDA(cudaMemcpyToSymbol(g_status, z, sizeof(z)));
  }
  return 0;
#else
  (void)out; (void)clear; (void)stream;
  return -HC_ERR_UNSUPPORTED;
#endif
}

extern "C" int hc_aggr_fwd(const hc_aggr_args* args, float* out, void* stream) {
  hc_aggr_args a;
  int rc = validate(args, &a);
  if (rc) return rc;
  if (a.num_node == 0) return 0;
  HC_REQUIRE(out != nullptr, HC_ERR_NULL);
  HC_REQUIRE(aligned_to(out, 4), HC_ERR_ALIGN);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  HC_CHECK_BLOCK(a, st);
  const int s = dtype_size(a.in_dtype);
  const int64_t row_bytes = (int64_t)a.feat * s;
  const bool out_vec = aligned16(out) && a.feat % 4 == 0;
  int h_vec = 0;
  if (a.hmap) {
    const int hs = dtype_size(a.h_dtype);
    h_vec = out_vec && aligned16(a.hbuf) && (a.hsize * hs) % 16 == 0 && ((int64_t)a.feat * hs) % 16 == 0;
  }
  // several heads take the vector path when they are an edge-weighted sum (the only multi-head
  // operator of the reference, history_aggr.cu:80-125) and source ids fit 31 bits
  const bool heads = a.num_head > 1;
  bool vec = (!heads || (a.edge_value != nullptr && a.n_src < 0x7fffffffLL)) && out_vec &&
             row_bytes % 16 == 0 && aligned16(a.input) && (a.in_stride * s) % 16 == 0;
  if (vec && a.src_map)
    vec = a.alt_dtype == a.in_dtype && aligned16(a.src_alt) && (a.alt_stride * s) % 16 == 0;
  if (vec && a.edge_value) vec = aligned_to(a.edge_value, 4);
  int G = 0, V = 0;
  const int nvec = (int)(row_bytes / 16);
  if (vec) vec = vec_shape(nvec, &G, &V) != 0;
  const int64_t targets = a.num_node * a.num_head;
  const int64_t blocks = ceil_div(targets, 8);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  dim3 grid((unsigned)blocks);
  if (vec && heads) {
    if (a.in_dtype == HC_F32) launch_fwd_heads<float>(G, V, grid, st, a, out, nvec, h_vec);
    else launch_fwd_heads<__half>(G, V, grid, st, a, out, nvec, h_vec);
  } else if (vec) {
    if (a.in_dtype == HC_F32) {
      if (a.edge_value) launch_fwd_vec<float, true>(G, V, grid, st, a, out, nvec, h_vec);
      else launch_fwd_vec<float, false>(G, V, grid, st, a, out, nvec, h_vec);
    } else {
      if (a.edge_value) launch_fwd_vec<__half, true>(G, V, grid, st, a, out, nvec, h_vec);
      else launch_fwd_vec<__half, false>(G, V, grid, st, a, out, nvec, h_vec);
    }
  } else {
    aggr_fwd_generic_kernel<<<grid, 256, 0, st>>>(a, out);
  }
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_aggr_bwd(const hc_aggr_args* args, const float* grad_out, float* grad_input,
                           int32_t zero_grad_input, float* grad_history, float* edge_grad,
                           float* row_score, int32_t score_kind, void* stream) {
  hc_aggr_args a;
  int rc = validate(args, &a);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t row = (int64_t)a.num_head * a.feat;
  const int64_t gi_stride = row;  // grad_input is dense [n_src, num_head, feat]
  if (grad_input && zero_grad_input && a.n_src > 0)
    HC_CUDA(cudaMemsetAsync(grad_input, 0, (size_t)a.n_src * row * sizeof(float), st));
  if (a.num_node == 0) return 0;
  HC_REQUIRE(grad_out != nullptr, HC_ERR_NULL);
  HC_REQUIRE(score_kind == HC_SCORE_L2 || score_kind == HC_SCORE_L1, HC_ERR_SIZE);
  HC_CHECK_BLOCK(a, st);
  HC_REQUIRE(!(row_score && a.num_head != 1), HC_ERR_UNSUPPORTED);
  HC_REQUIRE(!(edge_grad && !a.edge_value), HC_ERR_UNSUPPORTED);
  HC_REQUIRE(!(grad_history && !a.hmap), HC_ERR_NULL);
  if (grad_history && a.num_head > 1 && a.hsize == a.feat)
    HC_CUDA(cudaMemsetAsync(grad_history, 0, (size_t)a.num_node * a.hsize * sizeof(float), st));

  const bool heads = a.num_head > 1;
  bool vec = a.feat % 4 == 0 && aligned16(grad_out) && (grad_input == nullptr || aligned16(grad_input)) &&
             (grad_history == nullptr || (aligned16(grad_history) && a.hsize % 4 == 0));
  // several heads / the gradient of the edge values: vector path for edge-weighted sums over fp32
  // rows, with per-head (or single-head) history rows
  const bool special = heads || edge_grad != nullptr;
  if (vec && special) {
    vec = a.edge_value != nullptr && a.in_dtype == HC_F32 && aligned16(a.input) && a.in_stride % 4 == 0 &&
          (!a.src_map || (a.alt_dtype == HC_F32 && aligned16(a.src_alt) && a.alt_stride % 4 == 0)) &&
          (grad_history == nullptr || !heads || a.hsize == row) &&
          (edge_grad == nullptr || aligned_to(edge_grad, 4));
  }
  int G = 0, V = 0;
  const int nvec = a.feat / 4;
  if (vec) vec = vec_shape(nvec, &G, &V) != 0;
  const int64_t targets = a.num_node * a.num_head;
  const int64_t blocks = ceil_div(targets, 8);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  dim3 grid((unsigned)blocks);
  if (vec && special) {
    if (heads && edge_grad)
      launch_bwd_heads<true, true>(G, V, grid, st, a, grad_out, grad_input, grad_history, row_score,
                                   score_kind, nvec, gi_stride, edge_grad);
    else if (heads)
      launch_bwd_heads<true, false>(G, V, grid, st, a, grad_out, grad_input, grad_history, row_score,
                                    score_kind, nvec, gi_stride, nullptr);
    else
      launch_bwd_heads<false, true>(G, V, grid, st, a, grad_out, grad_input, grad_history, row_score,
                                    score_kind, nvec, gi_stride, edge_grad);
  } else if (vec) {
    if (a.edge_value)
      launch_bwd_vec<true>(G, V, grid, st, a, grad_out, grad_input, grad_history, row_score,
                           score_kind, nvec, gi_stride);
    else
      launch_bwd_vec<false>(G, V, grid, st, a, grad_out, grad_input, grad_history, row_score,
                            score_kind, nvec, gi_stride);
  } else {
    aggr_bwd_generic_kernel<<<grid, 256, 0, st>>>(a, grad_out, grad_input, grad_history, edge_grad,
                                                  row_score, score_kind, gi_stride);
  }
  HC_LAUNCH_OK();
  return 0;
}
