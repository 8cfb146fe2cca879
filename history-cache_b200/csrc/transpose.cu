// Backward aggregation as a gather over the transposed block.
//
// The reference (and hc_aggr_bwd) push gradients to the sources with atomic adds
// (src/cpp/src/history_aggr.cu:127-168).  On blocks larger than L2 that scatter is
// bound by read-modify-write DRAM traffic: every reduction that misses L2 moves its
// line DRAM -> L2 -> DRAM, and grad_input needs a zero-fill first.  Here the block is
// transposed once (source -> list of destination rows, each list sorted, so the
// result is reproducible bit for bit) and every source row is then written exactly
// once as the sum of its destinations' gradient rows: no atomics on the data, no
// zero-fill, deterministic.
#include "common.cuh"
#include "radix.cuh"

namespace hc {

// ---------------------------------------------------------------------------
// Transposition = a stable sort of the block's edges by source.
//
// Edges are laid out by destination row (CSR), so a STABLE sort by source leaves every
// source's list in ascending destination order: no per-list sort, no atomics, and the cost
// does not depend on how skewed the source popularity is (a hub with 10^5 entries is just
// 10^5 keys).  The sort is a least-significant-digit radix sort with 8-bit digits over
// 32-bit keys (key = source, payload = destination row); edges that carry no gradient
// (history-hit rows, sources served from the alternative table, the unused tail of idx)
// get the key n_src and end up behind every real list.  ceil(bits(n_src)/8) passes of
//   digit histogram per 4096-key chunk -> exclusive scan (digit-major) -> stable scatter.
// ---------------------------------------------------------------------------
// key/payload of every edge slot in [0, n_edges)
__global__ void __launch_bounds__(256)
    tr_expand_kernel(const hc_aggr_args a, const int64_t n_edges, uint32_t* __restrict__ key,
                     uint32_t* __restrict__ val) {
  constexpr int G = 8;
  const int gl = threadIdx.x & (G - 1);
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = gtid / G;
  const uint32_t none = (uint32_t)a.n_src;
  if (r < a.num_node) {
    const bool row_counts = !(a.hmap && a.hmap[r] != -1);
    int64_t b = a.ptr[r], e_end = a.ptr[r + 1];
    if (e_end > n_edges) e_end = n_edges;
    for (int64_t e = b + gl; e < e_end; e += G) {
      const int64_t s = a.idx[e];
      const bool ok = row_counts && s >= 0 && s < a.n_src && !(a.src_map && a.src_map[s] != -1);
      key[e] = ok ? (uint32_t)s : none;
      val[e] = (uint32_t)r;
    }
  }
  // slots behind the last row's edges
  int64_t tail = a.num_node > 0 ? a.ptr[a.num_node] : 0;
  if (tail < 0) tail = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = tail + gtid; e < n_edges; e += stride) {
    key[e] = none;
    val[e] = 0;
  }
}

// list boundaries, destination rows and weights from the sorted (source, row) pairs
__global__ void __launch_bounds__(256)
    tr_finalize_kernel(const uint32_t* __restrict__ key, const uint32_t* __restrict__ val, int64_t n_edges,
                       int64_t n_src, const int64_t* __restrict__ ptr, int64_t* __restrict__ t_ptr,
                       int64_t* __restrict__ t_dst, float* __restrict__ t_w) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_edges) return;
  const int64_t k = key[i];
  const int64_t prev = i > 0 ? (int64_t)key[i - 1] : -1;
  for (int64_t s = prev + 1; s <= k && s <= n_src; ++s) t_ptr[s] = i;   // lists of s in (prev, k] start here
  if (i == n_edges - 1)
    for (int64_t s = k + 1; s <= n_src; ++s) t_ptr[s] = n_edges;
  if (k < n_src) {
    const int64_t r = val[i];
    t_dst[i] = r;
    t_w[i] = __frcp_rn((float)(ptr[r + 1] - ptr[r]));
  }
}

// grad_input[s, :] = sum over the transposed list of t_w * grad_out[r, :]; every row written once.
// A warp takes kSW consecutive sources: their lists are one contiguous slice of t_dst / t_w,
// fetched with one coalesced load when it has at most 32 entries, so that each source then
// costs a single round of row loads.
//
// The lists may belong to a LARGER block than the one being differentiated (one transposition
// of a batch's CSR serves every layer, because all layers share the CSR prefix): entries whose
// destination row is >= num_node, or is served from history (hmap[r] != -1), are skipped.
//
// Lists longer than kLongList entries (popular sources of a skewed block) are left to the
// block-per-list kernels below: one thread block per list of up to kChunk entries, hub lists
// split into chunks of kChunk whose sums are added in chunk order, so the result stays
// bit-reproducible.
constexpr int kSW = 8;
constexpr int kLongList = 64;     // longer lists take the block-per-list path
constexpr int kChunk = 2048;       // entries per work item of that path

__device__ __forceinline__ bool entry_counts(int64_t r, int64_t num_node, const int64_t* __restrict__ hmap) {
  return r < num_node && !(hmap && hmap[r] != -1);
}

template <int G, int V>
__global__ void __launch_bounds__(256)
    aggr_bwd_gather_kernel(const int64_t n_src, const int feat, const int64_t* __restrict__ t_ptr,
                           const int64_t* __restrict__ t_dst, const float* __restrict__ t_w,
                           const float* __restrict__ grad_out, float* __restrict__ grad_input,
                           const int nvec, const int64_t num_node, const int64_t* __restrict__ hmap,
                           const int64_t* __restrict__ src_map) {
  constexpr int EPW = kWarp / G;
  constexpr int U = V == 1 ? 4 : (V == 2 ? 2 : 1);
  const int lane = threadIdx.x & 31;
  const int64_t s0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kSW;
  if (s0 >= n_src) return;
  const int ns = (int)((n_src - s0) < kSW ? (n_src - s0) : kSW);
  const int sub = lane / G, gl = lane % G;
  const int64_t my_p = lane <= ns ? t_ptr[s0 + lane] : 0;
  const int64_t E0 = shfl64(my_p, 0), E1 = shfl64(my_p, ns);
  const bool one_chunk = (E1 - E0) <= kWarp;
  int64_t my_r = -1;
  float my_w = 0.f;
  if (one_chunk && E0 + lane < E1) {
    my_r = t_dst[E0 + lane];
    my_w = t_w[E0 + lane];
    if (!entry_counts(my_r, num_node, hmap)) my_r = -1;
  }
  for (int k = 0; k < ns; ++k) {
    const int64_t begin = shfl64(my_p, k);
    int64_t end = shfl64(my_p, k + 1);
    if (end - begin > kLongList) continue;   // warp-uniform: written by the long-list kernels
    if (src_map && src_map[s0 + k] != -1) end = begin;   // served from the other table: no gradient
    float4 acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t i = begin; i < end; i += EPW * U) {
      float4 buf[U][V];
      float w[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t jj = i + u * EPW + sub;
        bool ok = jj < end;
        int64_t r;
        if (one_chunk) {
          const int from = (int)(jj - E0) & 31;
          r = shfl64(my_r, from);
          w[u] = __shfl_sync(kFull, my_w, from);
          ok = ok && r >= 0;
        } else {
          r = ok ? t_dst[jj] : 0;
          w[u] = ok ? t_w[jj] : 0.f;
          ok = ok && entry_counts(r, num_node, hmap);
        }
        if (!ok) w[u] = 0.f;
#pragma unroll
        for (int q = 0; q < V; ++q) {
          const int v = gl + q * G;
          buf[u][q] = (ok && v < nvec) ? __ldg(reinterpret_cast<const float4*>(grad_out + r * feat) + v)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int q = 0; q < V; ++q) {
          acc[q].x = fmaf(w[u], buf[u][q].x, acc[q].x);
          acc[q].y = fmaf(w[u], buf[u][q].y, acc[q].y);
          acc[q].z = fmaf(w[u], buf[u][q].z, acc[q].z);
          acc[q].w = fmaf(w[u], buf[u][q].w, acc[q].w);
        }
    }
    if (EPW > 1) {
#pragma unroll
      for (int off = G; off < kWarp; off <<= 1)
#pragma unroll
        for (int q = 0; q < V; ++q) {
          acc[q].x += __shfl_xor_sync(kFull, acc[q].x, off);
          acc[q].y += __shfl_xor_sync(kFull, acc[q].y, off);
          acc[q].z += __shfl_xor_sync(kFull, acc[q].z, off);
          acc[q].w += __shfl_xor_sync(kFull, acc[q].w, off);
        }
    }
    if (sub == 0) {
#pragma unroll
      for (int q = 0; q < V; ++q) {
        const int v = gl + q * G;
        if (v < nvec) reinterpret_cast<float4*>(grad_input + (s0 + k) * feat)[v] = acc[q];
      }
    }
  }
}

// ---- long lists -----------------------------------------------------------
// work items (source, chunk).  A list of at most kChunk entries is one item that writes its
// grad_input row itself; a longer one is split into chunks whose items write partial[slot, :],
// added in chunk order by a last kernel.
struct LongWork {
  unsigned long long* counters;  // [0] items, [1] partial slots, [2] split sources
  int64_t* item_src;             // [max_items]
  int64_t* item_info;            // [max_items] chunk number << 32 | (partial slot + 1), 0 = direct
  int64_t* split_src;            // [max_split]
  int64_t* split_base;           // [max_split] first partial slot of the source
  float* partial;                // [max_slots, feat]
  int64_t max_items, max_slots, max_split;
};

__global__ void __launch_bounds__(256)
    long_collect_kernel(const int64_t n_src, const int64_t* __restrict__ t_ptr, LongWork w) {
  const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_src) return;
  const int64_t len = t_ptr[s + 1] - t_ptr[s];
  if (len <= kLongList) return;
  const int64_t chunks = ceil_div(len, kChunk);
  const int64_t first = (int64_t)atomicAdd(&w.counters[0], (unsigned long long)chunks);
  // the bounds hold by construction (lists are disjoint slices of the n_edges entries)
  if (first + chunks > w.max_items) return;
  if (chunks == 1) {
    w.item_src[first] = s;
    w.item_info[first] = 0;
    return;
  }
  const int64_t slot = (int64_t)atomicAdd(&w.counters[1], (unsigned long long)chunks);
  const int64_t li = (int64_t)atomicAdd(&w.counters[2], 1ull);
  if (slot + chunks > w.max_slots || li >= w.max_split) return;
  w.split_src[li] = s;
  w.split_base[li] = slot;
  for (int64_t c = 0; c < chunks; ++c) {
    w.item_src[first + c] = s;
    w.item_info[first + c] = (c << 32) | (slot + c + 1);
  }
}

// one block per item: warp q takes entries q*U.., (q+8)*U.. of the item with U row loads in
// flight per lane; the eight warp sums are added in warp order through shared memory
template <int V>
__global__ void __launch_bounds__(256)
    long_items_kernel(const int feat, const int nvec, const int64_t* __restrict__ t_ptr,
                      const int64_t* __restrict__ t_dst, const float* __restrict__ t_w,
                      const float* __restrict__ grad_out, LongWork w, float* __restrict__ grad_input,
                      const int64_t num_node, const int64_t* __restrict__ hmap,
                      const int64_t* __restrict__ src_map) {
  extern __shared__ __align__(16) float sh[];   // [8][feat]
  constexpr int U = V == 1 ? 4 : (V == 2 ? 2 : 1);
  int64_t n_items = (int64_t)w.counters[0];
  if (n_items > w.max_items) n_items = w.max_items;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int64_t s = w.item_src[item];
    const int64_t info = w.item_info[item];
    const int64_t chunk = info >> 32, slot = (info & 0xffffffffLL) - 1;
    const int64_t begin = t_ptr[s] + chunk * kChunk;
    int64_t end = begin + kChunk;
    if (end > t_ptr[s + 1]) end = t_ptr[s + 1];
    if (src_map && src_map[s] != -1) end = begin;
    float4 acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t j0 = begin + warp * U; j0 < end; j0 += 8 * U) {
      float4 buf[U][V];
      float wt[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t j = j0 + u;
        bool ok = j < end;
        const int64_t r = ok ? t_dst[j] : 0;
        wt[u] = ok ? t_w[j] : 0.f;
        ok = ok && entry_counts(r, num_node, hmap);
        if (!ok) wt[u] = 0.f;
#pragma unroll
        for (int q = 0; q < V; ++q) {
          const int v = lane + q * 32;
          buf[u][q] = (ok && v < nvec) ? __ldg(reinterpret_cast<const float4*>(grad_out + r * feat) + v)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int q = 0; q < V; ++q) {
          acc[q].x = fmaf(wt[u], buf[u][q].x, acc[q].x);
          acc[q].y = fmaf(wt[u], buf[u][q].y, acc[q].y);
          acc[q].z = fmaf(wt[u], buf[u][q].z, acc[q].z);
          acc[q].w = fmaf(wt[u], buf[u][q].w, acc[q].w);
        }
    }
#pragma unroll
    for (int q = 0; q < V; ++q) {
      const int v = lane + q * 32;
      if (v < nvec) reinterpret_cast<float4*>(sh + warp * feat)[v] = acc[q];
    }
    __syncthreads();
    float* dst = slot < 0 ? grad_input + s * feat : w.partial + slot * feat;
    for (int c = threadIdx.x; c < feat; c += blockDim.x) {
      float t = sh[c];
#pragma unroll
      for (int q = 1; q < 8; ++q) t += sh[q * feat + c];
      dst[c] = t;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
    long_reduce_kernel(const int feat, const int64_t* __restrict__ t_ptr, LongWork w,
                       float* __restrict__ grad_input) {
  int64_t n_split = (int64_t)w.counters[2];
  if (n_split > w.max_split) n_split = w.max_split;
  for (int64_t li = blockIdx.x; li < n_split; li += gridDim.x) {
    const int64_t s = w.split_src[li], base = w.split_base[li];
    const int64_t chunks = ceil_div(t_ptr[s + 1] - t_ptr[s], (int64_t)kChunk);
    for (int c = threadIdx.x; c < feat; c += blockDim.x) {
      float t = 0.f;
      for (int64_t k = 0; k < chunks; ++k) t += w.partial[(base + k) * feat + c];
      grad_input[s * feat + c] = t;
    }
  }
}

}  // namespace hc

using namespace hc;

static int radix_passes(int64_t n_src) {
  int bits = 1;
  while (bits < 32 && ((int64_t)1 << bits) <= n_src) ++bits;   // the key n_src itself must fit
  return (bits + 7) / 8;
}

extern "C" int64_t hc_transpose_scratch_bytes(int64_t n_src, int64_t n_edges) {
  (void)n_src;
  if (n_edges < 1) n_edges = 1;
  return (4 * n_edges + radix_hist_words(n_edges)) * (int64_t)sizeof(uint32_t);
}

static int check_simple(const hc_aggr_args* a) {
  HC_REQUIRE(a != nullptr, HC_ERR_NULL);
  HC_REQUIRE(a->struct_size == sizeof(hc_aggr_args), HC_ERR_STRUCT);
  HC_REQUIRE(a->num_node >= 0 && a->n_src >= 0 && a->feat > 0, HC_ERR_SIZE);
  HC_REQUIRE(a->num_head == 1 && a->edge_value == nullptr, HC_ERR_UNSUPPORTED);
  return 0;
}

extern "C" int hc_transpose_block(const hc_aggr_args* a, int64_t n_edges, int64_t* t_ptr,
                                  int64_t* t_dst, float* t_w, void* scratch, void* stream) {
  int rc = check_simple(a);
  if (rc) return rc;
  HC_REQUIRE(t_ptr != nullptr, HC_ERR_NULL);
  HC_REQUIRE(n_edges >= 0 && n_edges < 0x7fffffffLL && a->n_src < 0x7fffffffLL &&
                 a->num_node < 0x7fffffffLL, HC_ERR_SIZE);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->n_src == 0 || n_edges == 0 || a->num_node == 0) {
    HC_CUDA(cudaMemsetAsync(t_ptr, 0, (size_t)(a->n_src + 1) * sizeof(int64_t), st));
    return 0;
  }
  HC_REQUIRE(scratch != nullptr && aligned_to(scratch, 8), HC_ERR_NULL);
  HC_REQUIRE(a->ptr && a->idx && t_dst && t_w, HC_ERR_NULL);
  const int64_t nblk = ceil_div(n_edges, kRadixChunk);
  HC_REQUIRE(256 * nblk <= 0x7fffffffLL, HC_ERR_SIZE);
  uint32_t* key[2];
  uint32_t* val[2];
  key[0] = reinterpret_cast<uint32_t*>(scratch);
  key[1] = key[0] + n_edges;
  val[0] = key[1] + n_edges;
  val[1] = val[0] + n_edges;
  uint32_t* hist = val[1] + n_edges;
  // rows or leftover slots, whichever needs more threads (the tail loop is grid-strided)
  int64_t eb = ceil_div(a->num_node * 8, 256);
  const int64_t tail_b = ceil_div(n_edges, 256 * 8);
  if (tail_b > eb) eb = tail_b;
  HC_REQUIRE(eb <= 0x7fffffffLL, HC_ERR_SIZE);
  tr_expand_kernel<<<(unsigned)eb, 256, 0, st>>>(*a, n_edges, key[0], val[0]);
  const int cur = radix_sort_pairs(key, val, n_edges, radix_passes(a->n_src), hist, st);
  tr_finalize_kernel<<<(unsigned)ceil_div(n_edges, 256), 256, 0, st>>>(key[cur], val[cur], n_edges, a->n_src,
                                                                      a->ptr, t_ptr, t_dst, t_w);
  HC_LAUNCH_OK();
  return 0;
}

// every list longer than kLongList is at least one item; split lists add one item per chunk
static int64_t long_max_items(int64_t n_edges) { return n_edges / kLongList + n_edges / kChunk + 2; }
static int64_t long_max_slots(int64_t n_edges) { return 2 * (n_edges / kChunk) + 2; }
static int64_t long_max_split(int64_t n_edges) { return n_edges / kChunk + 1; }

extern "C" int64_t hc_gather_scratch_bytes(int64_t n_edges, int32_t feat) {
  if (n_edges < 0) n_edges = 0;
  return 256 + long_max_items(n_edges) * 16 + long_max_split(n_edges) * 16 +
         long_max_slots(n_edges) * (int64_t)feat * 4 + 64;
}

extern "C" int hc_aggr_bwd_gather(const hc_aggr_args* a, const int64_t* t_ptr, const int64_t* t_dst,
                                  const float* t_w, int64_t t_n_src, int64_t n_edges,
                                  const float* grad_out, float* grad_input, void* scratch,
                                  void* stream) {
  int rc = check_simple(a);
  if (rc) return rc;
  HC_REQUIRE(a->n_src <= t_n_src, HC_ERR_SIZE);   // t_ptr has t_n_src + 1 entries
  if (a->n_src == 0) return 0;
  HC_REQUIRE(t_ptr && grad_input, HC_ERR_NULL);
  HC_REQUIRE(a->num_node == 0 || (t_dst && t_w && grad_out), HC_ERR_NULL);
  HC_REQUIRE(a->feat % 4 == 0 && aligned16(grad_out) && aligned16(grad_input), HC_ERR_UNSUPPORTED);
  HC_REQUIRE(n_edges >= 0, HC_ERR_SIZE);
  const int nvec = a->feat / 4;
  int G, V;
  if (nvec <= 8) { G = 8; V = 1; }
  else if (nvec <= 16) { G = 16; V = 1; }
  else if (nvec <= 32) { G = 32; V = 1; }
  else if (nvec <= 64) { G = 32; V = 2; }
  else if (nvec <= 128) { G = 32; V = 4; }
  else if (nvec <= 256) { G = 32; V = 8; }
  else return -HC_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t blocks = ceil_div(ceil_div(a->n_src, kSW), 8);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  const unsigned g = (unsigned)blocks;
#define HC_GATHER_CASE(gg, vv)                                                                   \
  if (G == gg && V == vv)                                                                        \
    aggr_bwd_gather_kernel<gg, vv><<<g, 256, 0, st>>>(a->n_src, a->feat, t_ptr, t_dst, t_w, grad_out, \
                                                      grad_input, nvec, a->num_node, a->hmap,  \
                                                      a->src_map);
  HC_GATHER_CASE(8, 1) HC_GATHER_CASE(16, 1) HC_GATHER_CASE(32, 1) HC_GATHER_CASE(32, 2)
  HC_GATHER_CASE(32, 4) HC_GATHER_CASE(32, 8)
#undef HC_GATHER_CASE
  if (n_edges > kLongList) {   // only then can a list be long
    HC_REQUIRE(scratch != nullptr && aligned_to(scratch, 16), HC_ERR_NULL);
    LongWork w;
    w.max_items = long_max_items(n_edges);
    w.max_slots = long_max_slots(n_edges);
    w.max_split = long_max_split(n_edges);
    char* p = reinterpret_cast<char*>(scratch);
    w.counters = reinterpret_cast<unsigned long long*>(p); p += 256;
    w.item_src = reinterpret_cast<int64_t*>(p); p += w.max_items * 8;
    w.item_info = reinterpret_cast<int64_t*>(p); p += w.max_items * 8;
    w.split_src = reinterpret_cast<int64_t*>(p); p += w.max_split * 8;
    w.split_base = reinterpret_cast<int64_t*>(p); p += w.max_split * 8;
    w.partial = reinterpret_cast<float*>(p);
    HC_CUDA(cudaMemsetAsync(w.counters, 0, 32, st));
    long_collect_kernel<<<(unsigned)ceil_div(a->n_src, 256), 256, 0, st>>>(a->n_src, t_ptr, w);
    const unsigned ib = (unsigned)(w.max_items < 148 * 16 ? w.max_items : 148 * 16);
    const size_t smem = (size_t)8 * a->feat * sizeof(float);
    HC_REQUIRE(smem <= 48 * 1024, HC_ERR_UNSUPPORTED);
    const int LV = nvec <= 32 ? 1 : (nvec <= 64 ? 2 : (nvec <= 128 ? 4 : 8));
#define HC_LONG_CASE(vv)                                                                              \
  if (LV == vv)                                                                                       \
    long_items_kernel<vv><<<ib, 256, smem, st>>>(a->feat, nvec, t_ptr, t_dst, t_w, grad_out, w,       \
                                                 grad_input, a->num_node, a->hmap, a->src_map);
    HC_LONG_CASE(1) HC_LONG_CASE(2) HC_LONG_CASE(4) HC_LONG_CASE(8)
#undef HC_LONG_CASE
    const unsigned rb = (unsigned)(w.max_split < 148 * 4 ? w.max_split : 148 * 4);
    long_reduce_kernel<<<rb, 256, 0, st>>>(a->feat, t_ptr, w, grad_input);
  }
  HC_LAUNCH_OK();
  return 0;
}
