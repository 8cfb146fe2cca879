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

// ---- fixed-shape exchange: every (source, destination) pair carries exactly `slots` ids ----

// ids in bucket order -> [world, slots] padded with -1; ids that do not fit are counted
__global__ void __launch_bounds__(256)
    bucket_pad_kernel(const int64_t* __restrict__ bucketed, const int64_t* __restrict__ counts,
                      int64_t n, int world, int64_t slots, int64_t* __restrict__ out,
                      unsigned long long* overflow) {
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= (int64_t)world * slots) return;
  const int b = (int)(k / slots);
  const int64_t pos = k % slots;
  int64_t start = 0;
  for (int w = 0; w < b; ++w) start += counts[w];
  const int64_t c = counts[b];
  out[k] = pos < c ? bucketed[start + pos] : -1;
  if (pos == 0 && c > slots && overflow) atomicAdd(overflow, (unsigned long long)(c - slots));
}

// hit_out[perm[k]] = row of the padded answer that holds bucket-order entry k, or -1
__global__ void __launch_bounds__(256)
    unpad_hits_kernel(const int64_t* __restrict__ perm, const int64_t* __restrict__ counts,
                      int64_t n_total, int world, int64_t slots,
                      const uint8_t* __restrict__ flags_back, int64_t* __restrict__ hit_out,
                      int64_t* __restrict__ slot_of) {
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n_total) return;
  int b = 0;
  int64_t start = 0;
  for (; b < world; ++b) {
    const int64_t c = counts[b];
    if (k < start + c) break;
    start += c;
  }
  if (b >= world) return;  // entry was left out of the buckets (keep mask)
  const int64_t pos = k - start;
  const int64_t where = (int64_t)b * slots + pos;
  const int64_t p = perm[k];
  if (slot_of) slot_of[p] = pos < slots ? where : -1;
  if (hit_out) hit_out[p] = (pos < slots && flags_back[where]) ? where : -1;
}

__global__ void last_claim_kernel(const int64_t* __restrict__ ids, int64_t n, int* claim, int64_t map_len) {
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int64_t id = ids[k];
  if (id >= 0 && id < map_len) atomicMax(claim + id, (int)k);
}
__global__ void last_mark_kernel(const int64_t* __restrict__ ids, int64_t n, const int* claim,
                                 int64_t map_len, uint8_t* winners) {
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int64_t id = ids[k];
  winners[k] = (id >= 0 && id < map_len && claim[id] == (int)k) ? 1 : 0;
}
__global__ void last_reset_kernel(const int64_t* __restrict__ ids, int64_t n, int* claim, int64_t map_len) {
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int64_t id = ids[k];
  if (id >= 0 && id < map_len) claim[id] = -1;
}

}  // namespace hc

using namespace hc;

extern "C" int hc_bucket_pad(const int64_t* bucketed, const int64_t* counts, int64_t n, int32_t world,
                             int64_t slots, int64_t* out, int64_t* overflow, void* stream) {
  HC_REQUIRE(n >= 0 && world >= 1 && world <= kMaxWorld && slots >= 1, HC_ERR_SIZE);
  HC_REQUIRE(counts && out && (bucketed || n == 0), HC_ERR_NULL);
  const int64_t total = (int64_t)world * slots;
  const int64_t blocks = ceil_div(total, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  bucket_pad_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      bucketed, counts, n, world, slots, out, reinterpret_cast<unsigned long long*>(overflow));
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_unpad_hits(const int64_t* perm, const int64_t* counts, int64_t n, int32_t world,
                             int64_t slots, const uint8_t* flags_back, int64_t* hit_out,
                             int64_t* slot_of, void* stream) {
  HC_REQUIRE(n >= 0 && world >= 1 && world <= kMaxWorld && slots >= 1, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(perm && counts && (hit_out || slot_of), HC_ERR_NULL);
  HC_REQUIRE(hit_out == nullptr || flags_back != nullptr, HC_ERR_NULL);
  const int64_t blocks = ceil_div(n, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  unpad_hits_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      perm, counts, n, world, slots, flags_back, hit_out, slot_of);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_last_occurrence(const int64_t* ids, int64_t n, int32_t* claim, int64_t map_len,
                                  uint8_t* winners, void* stream) {
  HC_REQUIRE(n >= 0 && n < 0x7fffffffLL && map_len >= 0, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(ids && claim && winners, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)ceil_div(n, 256);
  last_claim_kernel<<<blocks, 256, 0, st>>>(ids, n, claim, map_len);
  last_mark_kernel<<<blocks, 256, 0, st>>>(ids, n, claim, map_len, winners);
  last_reset_kernel<<<blocks, 256, 0, st>>>(ids, n, claim, map_len);
  HC_LAUNCH_OK();
  return 0;
}

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
    case HC_ERR_RANGE: return "hiscache_b200: an index of the block lies outside its table (see hc_last_status)";
    case HC_ERR_LIMIT: return "hiscache_b200: more rows than this entry point's fixed capacity (hc_noalloc_max_rows, or max_ids of a published area)";
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
