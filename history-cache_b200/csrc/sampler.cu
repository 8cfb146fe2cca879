// Uniform neighbour sampling and batch relabelling on the device.
//
// Stand-in for the sampler of CxGNN-DL (`cxgnndl.get_loader`, the reference's
// hiscache/history_trainer.py:19), which is not part of the reference project.
// What the hot path needs from it is the batch layout (one CSR shared by all
// layers, nodes ordered seeds first then each hop's new nodes, batch-local ids):
// hiscache/history_model.py:120-153, hiscache/history_cache.py:307-324.
// Every draw is a pure function of (seed, frontier position, draw number), so the
// CPU oracle reproduces a batch bit for bit.
#include "common.cuh"

namespace hc {

constexpr int kAbsent = (int)0x80000000;  // local_map value of a node outside the batch
constexpr int kScanBlock = 1024;

__global__ void sample_counts_kernel(const int64_t* __restrict__ gptr, const int64_t* __restrict__ frontier,
                                     int64_t nf, int fanout, int64_t* __restrict__ counts) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nf) return;
  const int64_t v = frontier[i];
  const int64_t deg = gptr[v + 1] - gptr[v];
  counts[i] = deg < fanout ? deg : fanout;
}

// one thread per (frontier node, draw)
__global__ void sample_picks_kernel(const int64_t* __restrict__ gptr, const int64_t* __restrict__ gidx,
                                    const int64_t* __restrict__ frontier, int64_t nf, int fanout,
                                    const int64_t* __restrict__ out_ptr, uint64_t seed, int64_t base,
                                    int64_t* __restrict__ nbr) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t i = t / fanout;
  const int j = (int)(t % fanout);
  if (i >= nf) return;
  const int64_t o = out_ptr[i];
  if (j >= out_ptr[i + 1] - o) return;
  const int64_t v = frontier[i];
  const int64_t b = gptr[v];
  const uint64_t deg = (uint64_t)(gptr[v + 1] - b);
  const uint64_t u = mix64(seed ^ mix64((uint64_t)(base + i) * (uint64_t)fanout + (uint64_t)j));
  nbr[o + j] = gidx[b + (int64_t)(u % deg)];
}

__global__ void relabel_seed_kernel(const int64_t* __restrict__ seeds, int64_t n, int* local_map) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) local_map[seeds[i]] = (int)i;
}
__global__ void relabel_reset_kernel(const int64_t* __restrict__ nodes, int64_t n, int* local_map) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) local_map[nodes[i]] = kAbsent;
}

// position p claims node nbr[p] unless the node already has a local id; the lowest p wins
__global__ void relabel_claim_kernel(const int64_t* __restrict__ nbr, int64_t m, int* local_map) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p < m) atomicMax(local_map + nbr[p], -(int)(p + 2));
}

__device__ __forceinline__ bool is_first(const int64_t* nbr, const int* local_map, int64_t p, int64_t m) {
  return p < m && local_map[nbr[p]] == -(int)(p + 2);
}

__global__ void __launch_bounds__(kScanBlock)
    relabel_count_kernel(const int64_t* __restrict__ nbr, int64_t m, const int* __restrict__ local_map,
                         int64_t* __restrict__ block_counts) {
  const int64_t p = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  const int c = __syncthreads_count(is_first(nbr, local_map, p, m));
  if (threadIdx.x == 0) block_counts[blockIdx.x] = c;
}

__global__ void __launch_bounds__(1024)
    relabel_scan_kernel(int64_t* block_counts, int64_t nblocks, int64_t* n_new) {
  __shared__ int64_t carry;
  __shared__ int64_t part[1024];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < nblocks; base += 1024) {
    const int64_t b = base + threadIdx.x;
    const int64_t c = b < nblocks ? block_counts[b] : 0;
    part[threadIdx.x] = c;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int64_t v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
      __syncthreads();
      part[threadIdx.x] += v;
      __syncthreads();
    }
    if (b < nblocks) block_counts[b] = carry + part[threadIdx.x] - c;  // exclusive offset
    __syncthreads();
    if (threadIdx.x == 1023) carry += part[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) n_new[0] = carry;
}

// new nodes in order of first occurrence: new_nodes[rank] = node
__global__ void __launch_bounds__(kScanBlock)
    relabel_place_kernel(const int64_t* __restrict__ nbr, int64_t m, const int* __restrict__ local_map,
                         const int64_t* __restrict__ block_offsets, int64_t* __restrict__ new_nodes) {
  __shared__ int warp_sums[kScanBlock / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t p = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  const bool f = is_first(nbr, local_map, p, m);
  const unsigned bal = __ballot_sync(kFull, f);
  if (lane == 0) warp_sums[warp] = __popc(bal);
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += warp_sums[w];
  if (f) new_nodes[block_offsets[blockIdx.x] + before + __popc(bal & ((1u << lane) - 1u))] = nbr[p];
}

__global__ void relabel_assign_kernel(const int64_t* __restrict__ new_nodes, const int64_t* __restrict__ n_new,
                                      int64_t n_total, int* local_map) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r < n_new[0]) local_map[new_nodes[r]] = (int)(n_total + r);
}

__global__ void relabel_translate_kernel(const int64_t* __restrict__ nbr, int64_t m,
                                         const int* __restrict__ local_map, int64_t* __restrict__ out_idx) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p < m) out_idx[p] = local_map[nbr[p]];
}

}  // namespace hc

using namespace hc;

static inline unsigned blocks_for(int64_t n, int per) { return (unsigned)ceil_div(n > 0 ? n : 1, per); }

extern "C" int hc_sample_counts(const int64_t* gptr, const int64_t* frontier, int64_t nf, int32_t fanout,
                                int64_t* counts, void* stream) {
  HC_REQUIRE(nf >= 0 && fanout >= 1, HC_ERR_SIZE);
  if (nf == 0) return 0;
  HC_REQUIRE(gptr && frontier && counts, HC_ERR_NULL);
  sample_counts_kernel<<<blocks_for(nf, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      gptr, frontier, nf, fanout, counts);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_sample_picks(const int64_t* gptr, const int64_t* gidx, const int64_t* frontier,
                               int64_t nf, int32_t fanout, const int64_t* out_ptr, uint64_t seed,
                               int64_t base, int64_t* nbr, void* stream) {
  HC_REQUIRE(nf >= 0 && fanout >= 1 && base >= 0, HC_ERR_SIZE);
  if (nf == 0) return 0;
  HC_REQUIRE(gptr && gidx && frontier && out_ptr && nbr, HC_ERR_NULL);
  const int64_t threads = nf * fanout;
  HC_REQUIRE(ceil_div(threads, 256) <= 0x7fffffffLL, HC_ERR_SIZE);
  sample_picks_kernel<<<blocks_for(threads, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      gptr, gidx, frontier, nf, fanout, out_ptr, seed, base, nbr);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_relabel_seed(const int64_t* seeds, int64_t n, int32_t* local_map, void* stream) {
  HC_REQUIRE(n >= 0 && n < 0x7fffffffLL, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(seeds && local_map, HC_ERR_NULL);
  relabel_seed_kernel<<<blocks_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(seeds, n, local_map);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_relabel_reset(const int64_t* nodes, int64_t n, int32_t* local_map, void* stream) {
  HC_REQUIRE(n >= 0, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(nodes && local_map, HC_ERR_NULL);
  relabel_reset_kernel<<<blocks_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(nodes, n, local_map);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int64_t hc_relabel_scratch_bytes(int64_t m) {
  return (ceil_div(m > 0 ? m : 1, kScanBlock) + 1) * (int64_t)sizeof(int64_t);
}

extern "C" int hc_relabel(const int64_t* nbr, int64_t m, int32_t* local_map, int64_t n_total,
                          int64_t* new_nodes, int64_t* n_new, int64_t* out_idx, void* scratch,
                          void* stream) {
  HC_REQUIRE(m >= 0 && m < 0x7ffffff0LL && n_total >= 0 && n_total + m < 0x7fffffffLL, HC_ERR_SIZE);
  HC_REQUIRE(n_new != nullptr, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (m == 0) {
    HC_CUDA(cudaMemsetAsync(n_new, 0, sizeof(int64_t), st));
    return 0;
  }
  HC_REQUIRE(nbr && local_map && new_nodes && out_idx && scratch, HC_ERR_NULL);
  int64_t* block_counts = reinterpret_cast<int64_t*>(scratch);
  const unsigned nb = blocks_for(m, kScanBlock);
  relabel_claim_kernel<<<blocks_for(m, 256), 256, 0, st>>>(nbr, m, local_map);
  relabel_count_kernel<<<nb, kScanBlock, 0, st>>>(nbr, m, local_map, block_counts);
  relabel_scan_kernel<<<1, 1024, 0, st>>>(block_counts, nb, n_new);
  relabel_place_kernel<<<nb, kScanBlock, 0, st>>>(nbr, m, local_map, block_counts, new_nodes);
  relabel_assign_kernel<<<blocks_for(m, 256), 256, 0, st>>>(new_nodes, n_new, n_total, local_map);
  relabel_translate_kernel<<<blocks_for(m, 256), 256, 0, st>>>(nbr, m, local_map, out_idx);
  HC_LAUNCH_OK();
  return 0;
}
