// Receptive-field bookkeeping: used masks, structure score, relation histogram.
// Replaces count_history_kernel, get_graph_structure_score_kernel and
// count_kernel of the reference (src/cpp/src/grad_check.cu:70-182).
#include "common.cuh"

namespace hc {

// One propagation step.  `first` marks the step that starts from the seeds;
// hmap is passed for the second step only (grad_check.cu:122-124).
__global__ void __launch_bounds__(256)
    used_mask_step_kernel(const int64_t* __restrict__ ptr, const int64_t* __restrict__ idx,
                          const int64_t* __restrict__ hmap, int64_t hmap_len, uint8_t* use_in,
                          uint8_t* use_out, int64_t rows, int64_t num_seed, int first) {
  // 8 lanes per row: sampled rows have 5-25 neighbours
  constexpr int G = 8;
  const int gl = threadIdx.x & (G - 1);
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (row >= rows) return;
  if (first && row < num_seed) {
    if (gl == 0) use_in[row] = 1;
  } else if (use_in[row] != 1) {
    return;
  }
  if (hmap != nullptr && row < hmap_len && hmap[row] != -1) return;  // history hit: subtree not needed
  if (gl == 0) use_out[row] = 1;                                     // self loop
  const int64_t begin = ptr[row], end = ptr[row + 1];
  for (int64_t e = begin + gl; e < end; e += G) use_out[idx[e]] = 1;
}

__global__ void structure_seed_kernel(int64_t* out, int64_t num_node, int64_t rows, int64_t num_seed) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_node) return;
  out[i] = (i < num_seed && i < rows) ? 1 : 0;
}

__global__ void structure_claim_kernel(const int64_t* __restrict__ ptr, const int64_t* __restrict__ idx,
                                       const int64_t* __restrict__ out, long long* parent,
                                       int64_t rows) {
  constexpr int G = 8;
  const int gl = threadIdx.x & (G - 1);
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (row >= rows || out[row] == 0) return;
  const int64_t begin = ptr[row], end = ptr[row + 1];
  for (int64_t e = begin + gl; e < end; e += G) {
    const int64_t v = idx[e];
    if (out[v] == 0) atomicMin(parent + v, (long long)row);
  }
}

__global__ void structure_apply_kernel(const int64_t* __restrict__ ptr, int64_t* out,
                                       long long* parent, int64_t num_node) {
  const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= num_node) return;
  const long long p = parent[v];
  parent[v] = 0x7fffffffffffffffLL;
  if (p != 0x7fffffffffffffffLL && out[v] == 0) out[v] = out[p] * (ptr[p + 1] - ptr[p]);
}

__global__ void fill_i64_kernel(long long* p, int64_t n, long long v) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

__global__ void count_num_kernel(const int64_t* __restrict__ arr, int64_t n, int64_t mmax,
                                 int* output) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t a = arr[i];
  if (a != 0 && a > 0 && a <= mmax) atomicAdd(output + a, 1);  // value 0 is never counted
}

}  // namespace hc

using namespace hc;

extern "C" int hc_used_masks(const int64_t* ptr, const int64_t* idx, int64_t ptr_rows,
                             const int64_t* history_map, int64_t history_map_len,
                             int64_t num_node, int64_t num_seed, int32_t num_layer, uint8_t* masks,
                             void* stream) {
  HC_REQUIRE(ptr_rows >= 0 && num_node >= 0 && num_seed >= 0 && num_layer >= 0 &&
                 history_map_len >= 0,
             HC_ERR_SIZE);
  HC_REQUIRE(ptr_rows <= num_node && num_seed <= num_node, HC_ERR_SIZE);
  if (num_node == 0) return 0;
  HC_REQUIRE(masks != nullptr, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  HC_CUDA(cudaMemsetAsync(masks, 0, (size_t)(num_layer + 1) * num_node, st));
  if (ptr_rows == 0 || num_layer == 0) return 0;
  HC_REQUIRE(ptr && idx, HC_ERR_NULL);
  const int64_t blocks = ceil_div(ptr_rows * 8, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  for (int i = 0; i < num_layer; ++i) {
    uint8_t* in = masks + (int64_t)(num_layer - i) * num_node;
    uint8_t* out = masks + (int64_t)(num_layer - 1 - i) * num_node;
    used_mask_step_kernel<<<(unsigned)blocks, 256, 0, st>>>(
        ptr, idx, i == 1 ? history_map : nullptr, history_map_len, in, out, ptr_rows, num_seed,
        i == 0);
  }
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_structure_score(const int64_t* ptr, const int64_t* idx, int64_t ptr_rows,
                                  int64_t num_node, int64_t num_seed, int32_t num_layer,
                                  int64_t* output, int64_t* scratch, void* stream) {
  HC_REQUIRE(ptr_rows >= 0 && num_node >= 0 && num_seed >= 0 && num_layer >= 0, HC_ERR_SIZE);
  HC_REQUIRE(ptr_rows <= num_node, HC_ERR_SIZE);
  if (num_node == 0) return 0;
  HC_REQUIRE(output && scratch, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t nb = ceil_div(num_node, 256);
  HC_REQUIRE(nb <= 0x7fffffffLL, HC_ERR_SIZE);
  // the reference marks seeds inside every launch, so zero launches leave zeros
  structure_seed_kernel<<<(unsigned)nb, 256, 0, st>>>(output, num_node, ptr_rows,
                                                      num_layer > 0 ? num_seed : 0);
  if (ptr_rows > 0 && num_layer > 0) {
    HC_REQUIRE(ptr && idx, HC_ERR_NULL);
    long long* parent = reinterpret_cast<long long*>(scratch);
    fill_i64_kernel<<<(unsigned)nb, 256, 0, st>>>(parent, num_node, 0x7fffffffffffffffLL);
    const int64_t rb = ceil_div(ptr_rows * 8, 256);
    HC_REQUIRE(rb <= 0x7fffffffLL, HC_ERR_SIZE);
    for (int i = 0; i < num_layer; ++i) {
      structure_claim_kernel<<<(unsigned)rb, 256, 0, st>>>(ptr, idx, output, parent, ptr_rows);
      structure_apply_kernel<<<(unsigned)nb, 256, 0, st>>>(ptr, output, parent, num_node);
    }
  }
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_count_num(const int64_t* arr, int64_t n, int64_t mmax, int32_t* output,
                            void* stream) {
  HC_REQUIRE(n >= 0 && mmax >= 0, HC_ERR_SIZE);
  HC_REQUIRE(output != nullptr, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  HC_CUDA(cudaMemsetAsync(output, 0, (size_t)(mmax + 1) * sizeof(int32_t), st));
  if (n == 0) return 0;
  HC_REQUIRE(arr != nullptr, HC_ERR_NULL);
  const int64_t blocks = ceil_div(n, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  count_num_kernel<<<(unsigned)blocks, 256, 0, st>>>(arr, n, mmax, output);
  HC_LAUNCH_OK();
  return 0;
}
