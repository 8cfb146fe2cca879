// Owner bucketing for the node-partitioned history table, plus the small
// library-level entry points (version, error text, owner hash).
//
// The reference has no working sharded store: prepare_transfer
// (hiscache/comm.py:132-143) does one index_select per (src, dst) pair on a
// feature-axis split whose slice is empty (hiscache/history_cache.py:72-78).
// Here ids are bucketed by owner(id) = mix64(id) mod world in one stable pass
// so that a single all-to-all moves them.
#include "common.cuh"

namespace hc {

constexpr int kBucketBlock = 1024;
constexpr int kMaxWorld = 64;

__device__ __forceinline__ int owner_of(int64_t id, int world) {
  return (int)(mix64((uint64_t)id) % (uint64_t)world);
}

// per-block histogram: hist[b*world + w]
__global__ void __launch_bounds__(kBucketBlock)
    bucket_hist_kernel(const int64_t* __restrict__ ids, const uint8_t* __restrict__ keep, int64_t n,
                       int world, int64_t* __restrict__ hist) {
  __shared__ int cnt[kMaxWorld];
  if (threadIdx.x < kMaxWorld) cnt[threadIdx.x] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * kBucketBlock + threadIdx.x;
  if (i < n && (keep == nullptr || keep[i])) atomicAdd(&cnt[owner_of(ids[i], world)], 1);
  __syncthreads();
  if (threadIdx.x < world) hist[(int64_t)blockIdx.x * world + threadIdx.x] = cnt[threadIdx.x];
}

// one block: turns hist into start offsets (bucket-major) and writes counts
__global__ void __launch_bounds__(1024)
    bucket_scan_kernel(int64_t* hist, int64_t nblocks, int world, int64_t* counts) {
  __shared__ int64_t totals[kMaxWorld];
  __shared__ int64_t base[kMaxWorld];
  // each owner column is scanned by one thread (world <= 64, nblocks <= ~1e3)
  if (threadIdx.x < world) {
    int64_t run = 0;
    for (int64_t b = 0; b < nblocks; ++b) {
      const int64_t c = hist[b * world + threadIdx.x];
      hist[b * world + threadIdx.x] = run;
      run += c;
    }
    totals[threadIdx.x] = run;
    counts[threadIdx.x] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int64_t run = 0;
    for (int w = 0; w < world; ++w) {
      base[w] = run;
      run += totals[w];
    }
  }
  __syncthreads();
  for (int64_t k = threadIdx.x; k < nblocks * world; k += blockDim.x) hist[k] += base[k % world];
}

__global__ void __launch_bounds__(kBucketBlock)
    bucket_place_kernel(const int64_t* __restrict__ ids, const uint8_t* __restrict__ keep, int64_t n,
                        int world, const int64_t* __restrict__ hist, int64_t* __restrict__ perm,
                        int64_t* __restrict__ bucketed) {
  __shared__ int warp_cnt[kBucketBlock / 32][kMaxWorld];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t i = (int64_t)blockIdx.x * kBucketBlock + threadIdx.x;
  const bool on = i < n && (keep == nullptr || keep[i]);
  const int64_t id = on ? ids[i] : 0;
  const int own = on ? owner_of(id, world) : -1;
  // rank inside the warp among lanes with the same owner, and per-warp counts
  const unsigned peers = __match_any_sync(kFull, own);
  const int in_warp = __popc(peers & ((1u << lane) - 1u));
  for (int w = lane; w < world; w += 32) warp_cnt[warp][w] = 0;
  __syncwarp();
  if (on && in_warp == 0) warp_cnt[warp][own] = __popc(peers);
  __syncthreads();
  if (on) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w][own];
    const int64_t pos = hist[(int64_t)blockIdx.x * world + own] + before + in_warp;
    perm[pos] = i;
    if (bucketed) bucketed[pos] = id;
  }
}

}  // namespace hc

using namespace hc;

extern "C" int hc_abi_version(void) { return HC_ABI_VERSION; }

extern "C" const char* hc_error_string(int code) {
  if (code == 0) return "ok";
  if (code > 0) return cudaGetErrorString((cudaError_t)code);
  switch (-code) {
    case HC_ERR_NULL: return "hiscache_b200: a required pointer is NULL";
    case HC_ERR_SIZE: return "hiscache_b200: a size, count, stride or option is out of range";
    case HC_ERR_DTYPE: return "hiscache_b200: unknown dtype code";
    case HC_ERR_ALIGN: return "hiscache_b200: pointer not aligned to its element type";
    case HC_ERR_UNSUPPORTED: return "hiscache_b200: this combination of options is not implemented";
    case HC_ERR_STRUCT: return "hiscache_b200: struct_size does not match this build of the library";
    case HC_ERR_LIMIT: return "hiscache_b200: more rows than this fixed-scratch entry point accepts (see hc_noalloc_max_rows)";
    default: return "hiscache_b200: unknown error code";
  }
}

extern "C" uint64_t hc_mix64(uint64_t x) { return mix64(x); }

extern "C" int64_t hc_bucket_scratch_bytes(int64_t n, int32_t world) {
  const int64_t nb = n > 0 ? ceil_div(n, kBucketBlock) : 1;
  return nb * (world > 0 ? world : 1) * (int64_t)sizeof(int64_t);
}

extern "C" int hc_bucket_by_owner(const int64_t* ids, const uint8_t* keep, int64_t n, int32_t world,
                                  int64_t* counts, int64_t* perm, int64_t* bucketed, void* scratch,
                                  void* stream) {
  HC_REQUIRE(n >= 0 && world >= 1 && world <= kMaxWorld, HC_ERR_SIZE);
  HC_REQUIRE(counts != nullptr, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (n == 0) {
    HC_CUDA(cudaMemsetAsync(counts, 0, (size_t)world * sizeof(int64_t), st));
    return 0;
  }
  HC_REQUIRE(ids && perm && scratch, HC_ERR_NULL);
  const int64_t nb = ceil_div(n, kBucketBlock);
  HC_REQUIRE(nb <= 0x7fffffffLL, HC_ERR_SIZE);
  int64_t* hist = reinterpret_cast<int64_t*>(scratch);
  bucket_hist_kernel<<<(unsigned)nb, kBucketBlock, 0, st>>>(ids, keep, n, world, hist);
  bucket_scan_kernel<<<1, 1024, 0, st>>>(hist, nb, world, counts);
  bucket_place_kernel<<<(unsigned)nb, kBucketBlock, 0, st>>>(ids, keep, n, world, hist, perm,
                                                            bucketed);
  HC_LAUNCH_OK();
  return 0;
}
