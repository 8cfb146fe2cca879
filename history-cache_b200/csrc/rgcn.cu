// Relation handling of the heterogeneous (RGCN) layers.
//
// The reference's MyRGCNConvHistory2.forward (hiscache/history_model.py:244-272) expands the CSR
// into (src, dst) pairs, gives edges whose source is not needed the relation number num_rel,
// sorts the edges by relation with torch.sort, counts them per relation (count_num) and hands
// (src[perm], dst[perm], count) to cxgnncomp.RGCNOP_sorted; edge types come from
// cxgnncomp_backend.gen_edge_type_mag240m (:354-357).  Neither operator is part of the project.
//
// Here one call builds the relation-segmented block directly on the device:
//   pruning (unused sources; optionally destinations served from history) -> ONE stable 8-bit
//   radix pass by relation (edges of a relation stay in destination order) -> a CSR over
//   num_rel * num_node rows, row r * num_node + d listing the sources of d's relation-r edges,
//   with the weight 1 / deg(d) beside each (the reference normalises by the total in-degree,
//   :245,272).
// The history-aware aggregation kernel then reads every source row exactly once per edge and
// produces the per-(relation, destination) sums that the grouped product consumes.
#include "common.cuh"
#include "radix.cuh"

namespace hc {

struct TypeTable {
  int n_types;
  int64_t bound[9];     // node type t owns global ids [bound[t], bound[t+1])
  int32_t rel[64];      // relation of an edge into a type-d node from a type-s node: rel[d * n_types + s]
};

__device__ __forceinline__ int node_type(const TypeTable& t, int64_t g) {
  int k = 0;
  while (k + 1 < t.n_types && g >= t.bound[k + 1]) ++k;
  return k;
}

__global__ void __launch_bounds__(256)
    edge_type_kernel(const int64_t* __restrict__ ptr, const int64_t* __restrict__ idx,
                     const int64_t* __restrict__ sub_to_full, int64_t rows, const TypeTable t,
                     int64_t* __restrict__ etype) {
  constexpr int G = 8;
  const int gl = threadIdx.x & (G - 1);
  const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (r >= rows) return;
  const int td = node_type(t, sub_to_full[r]);
  for (int64_t e = ptr[r] + gl; e < ptr[r + 1]; e += G)
    etype[e] = t.rel[td * t.n_types + node_type(t, sub_to_full[idx[e]])];
}

// key = relation (num_rel for pruned edges and for the slots behind the last row), payload = edge
__global__ void __launch_bounds__(256)
    rgcn_expand_kernel(const int64_t* __restrict__ ptr, const int64_t* __restrict__ idx,
                       const int64_t* __restrict__ etype, int64_t num_node, int64_t n_edges, int num_rel,
                       const uint8_t* __restrict__ used, const int64_t* __restrict__ hmap,
                       uint32_t* __restrict__ key, uint32_t* __restrict__ val, uint32_t* __restrict__ row_of,
                       int64_t* __restrict__ rel_out) {
  constexpr int G = 8;
  const int gl = threadIdx.x & (G - 1);
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = gtid / G;
  if (r < num_node) {
    const bool row_ok = !(hmap && hmap[r] != -1);
    int64_t e_end = ptr[r + 1];
    if (e_end > n_edges) e_end = n_edges;
    for (int64_t e = ptr[r] + gl; e < e_end; e += G) {
      int64_t rel = etype[e];
      if (!row_ok || rel < 0 || rel >= num_rel || (used && !used[idx[e]])) rel = num_rel;
      key[e] = (uint32_t)rel;
      val[e] = (uint32_t)e;
      row_of[e] = (uint32_t)r;
      if (rel_out) rel_out[e] = rel;
    }
  }
  int64_t tail = num_node > 0 ? ptr[num_node] : 0;
  if (tail < 0) tail = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = tail + gtid; e < n_edges; e += stride) {
    key[e] = (uint32_t)num_rel;
    val[e] = (uint32_t)e;
    row_of[e] = 0;
    if (rel_out) rel_out[e] = num_rel;
  }
}

// rows of the grouped CSR from the sorted (relation, edge) pairs
__global__ void __launch_bounds__(256)
    rgcn_finalize_kernel(const uint32_t* __restrict__ key, const uint32_t* __restrict__ val,
                         const uint32_t* __restrict__ row_of, int64_t n_edges, int64_t num_node, int num_rel,
                         const int64_t* __restrict__ ptr, const int64_t* __restrict__ idx,
                         int64_t* __restrict__ ptr2, int64_t* __restrict__ idx2, float* __restrict__ w2,
                         int64_t* __restrict__ perm) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_edges) return;
  const int64_t rows2 = (int64_t)num_rel * num_node;
  const int64_t e = val[i];
  const int64_t k = key[i] < (uint32_t)num_rel ? (int64_t)key[i] * num_node + row_of[e] : rows2;
  int64_t prev = -1;
  if (i > 0) {
    const int64_t pe = val[i - 1];
    prev = key[i - 1] < (uint32_t)num_rel ? (int64_t)key[i - 1] * num_node + row_of[pe] : rows2;
  }
  for (int64_t s = prev + 1; s <= k && s <= rows2; ++s) ptr2[s] = i;
  if (i == n_edges - 1)
    for (int64_t s = k + 1; s <= rows2; ++s) ptr2[s] = n_edges;
  if (perm) perm[i] = e;
  if (k < rows2) {
    const int64_t d = row_of[e];
    idx2[i] = idx[e];
    w2[i] = __frcp_rn((float)(ptr[d + 1] - ptr[d]));
  } else {
    idx2[i] = 0;
    w2[i] = 0.f;
  }
}

}  // namespace hc

using namespace hc;

extern "C" int hc_edge_types(const int64_t* ptr, const int64_t* idx, const int64_t* sub_to_full,
                             int64_t rows, int32_t n_types, const int64_t* type_bounds,
                             const int32_t* rel_table, int64_t* etype, void* stream) {
  HC_REQUIRE(rows >= 0, HC_ERR_SIZE);
  HC_REQUIRE(n_types >= 1 && n_types <= 8, HC_ERR_SIZE);
  HC_REQUIRE(type_bounds && rel_table, HC_ERR_NULL);
  if (rows == 0) return 0;
  HC_REQUIRE(ptr && idx && sub_to_full && etype, HC_ERR_NULL);
  TypeTable t;
  t.n_types = n_types;
  for (int k = 0; k <= n_types; ++k) t.bound[k] = type_bounds[k];     // host arrays
  for (int k = 0; k < n_types * n_types; ++k) t.rel[k] = rel_table[k];
  const int64_t blocks = ceil_div(rows * 8, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  edge_type_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ptr, idx, sub_to_full,
                                                                                         rows, t, etype);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int64_t hc_rgcn_group_scratch_bytes(int64_t n_edges) {
  if (n_edges < 1) n_edges = 1;
  return (5 * n_edges + radix_hist_words(n_edges)) * (int64_t)sizeof(uint32_t);
}

extern "C" int hc_rgcn_group(const int64_t* ptr, const int64_t* idx, const int64_t* etype,
                             int64_t num_node, int64_t n_edges, int32_t num_rel,
                             const uint8_t* used_src, const int64_t* hmap, int64_t* ptr2,
                             int64_t* idx2, float* w2, int64_t* perm, int64_t* rel_out,
                             void* scratch, void* stream) {
  HC_REQUIRE(num_node >= 0 && n_edges >= 0 && num_rel >= 1 && num_rel <= 255, HC_ERR_SIZE);
  HC_REQUIRE(n_edges < 0x7fffffffLL && num_node < 0x7fffffffLL, HC_ERR_SIZE);
  HC_REQUIRE(ptr2 != nullptr, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t rows2 = (int64_t)num_rel * num_node;
  if (n_edges == 0 || num_node == 0) {
    HC_CUDA(cudaMemsetAsync(ptr2, 0, (size_t)(rows2 + 1) * sizeof(int64_t), st));
    return 0;
  }
  HC_REQUIRE(ptr && idx && etype && idx2 && w2 && scratch, HC_ERR_NULL);
  HC_REQUIRE(aligned_to(scratch, 8), HC_ERR_NULL);
  uint32_t* key[2];
  uint32_t* val[2];
  key[0] = reinterpret_cast<uint32_t*>(scratch);
  key[1] = key[0] + n_edges;
  val[0] = key[1] + n_edges;
  val[1] = val[0] + n_edges;
  uint32_t* row_of = val[1] + n_edges;
  uint32_t* hist = row_of + n_edges;
  int64_t eb = ceil_div(num_node * 8, 256);
  const int64_t tail_b = ceil_div(n_edges, 256 * 8);
  if (tail_b > eb) eb = tail_b;
  HC_REQUIRE(eb <= 0x7fffffffLL, HC_ERR_SIZE);
  rgcn_expand_kernel<<<(unsigned)eb, 256, 0, st>>>(ptr, idx, etype, num_node, n_edges, num_rel, used_src, hmap,
                                                   key[0], val[0], row_of, rel_out);
  const int cur = radix_sort_pairs(key, val, n_edges, 1, hist, st);   // relations fit one 8-bit digit
  rgcn_finalize_kernel<<<(unsigned)ceil_div(n_edges, 256), 256, 0, st>>>(key[cur], val[cur], row_of, n_edges,
                                                                         num_node, num_rel, ptr, idx, ptr2,
                                                                         idx2, w2, perm);
  HC_LAUNCH_OK();
  return 0;
}
