// Least-significant-digit radix sort of (32-bit key, 32-bit payload) pairs, 8-bit digits, STABLE:
// per pass a digit histogram per 4096-key chunk, an exclusive scan in digit-major order and a
// scatter in which a key goes to (scanned start of its digit for its chunk) + (keys of that digit
// in lower warps of the chunk) + (its rank among its warp's earlier keys).  No atomics decide a
// position, so equal keys keep their input order and the result is reproducible.
// Used by the block transposition (keys = sources) and the relation grouping of RGCN layers.
#pragma once
#include "common.cuh"

namespace hc {

constexpr int kRadixWarps = 8;
constexpr int kRadixIters = 16;                                   // keys per lane and pass
constexpr int kRadixChunk = kRadixWarps * kRadixIters * kWarp;    // 4096 keys per block
constexpr int kTScan = 1024;

// per-warp digit counts of this block's chunk, in shared memory cnt[warp][digit]
static __device__ __forceinline__ void radix_count(const uint32_t* __restrict__ key, int64_t n, int shift,
                                            uint32_t (*cnt)[256]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kRadixWarps * 256; i += blockDim.x) (&cnt[0][0])[i] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kRadixChunk + (int64_t)warp * (kRadixIters * kWarp);
#pragma unroll 4
  for (int it = 0; it < kRadixIters; ++it) {
    const int64_t i = base + it * kWarp + lane;
    if (i < n) atomicAdd(&cnt[warp][(key[i] >> shift) & 255u], 1u);
  }
  __syncthreads();
}

static __global__ void __launch_bounds__(kRadixWarps * kWarp)
    tr_hist_kernel(const uint32_t* __restrict__ key, int64_t n, int shift, int64_t nblk,
                   uint32_t* __restrict__ hist) {
  __shared__ uint32_t cnt[kRadixWarps][256];
  radix_count(key, n, shift, cnt);
  const int d = threadIdx.x;   // 256 threads, one digit each
  uint32_t t = 0;
#pragma unroll
  for (int w = 0; w < kRadixWarps; ++w) t += cnt[w][d];
  hist[(int64_t)d * nblk + blockIdx.x] = t;   // digit-major: the scan order of an LSD pass
}

// three-phase exclusive scan of v[0..n) in place (uint32)
static __global__ void __launch_bounds__(kTScan)
    tr_block_sum_kernel(const uint32_t* __restrict__ v, int64_t n, uint32_t* __restrict__ sums) {
  __shared__ uint32_t sh[kTScan / 32];
  const int64_t i = (int64_t)blockIdx.x * kTScan + threadIdx.x;
  uint32_t x = i < n ? v[i] : 0;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(kFull, x, off);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = x;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t t = 0;
    for (int w = 0; w < kTScan / 32; ++w) t += sh[w];
    sums[blockIdx.x] = t;
  }
}
static __global__ void __launch_bounds__(1024) tr_scan_sums_kernel(uint32_t* sums, int64_t nb) {
  __shared__ uint32_t part[1024];
  __shared__ uint32_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < nb; base += 1024) {
    const int64_t b = base + threadIdx.x;
    const uint32_t c = b < nb ? sums[b] : 0;
    part[threadIdx.x] = c;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const uint32_t v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
      __syncthreads();
      part[threadIdx.x] += v;
      __syncthreads();
    }
    if (b < nb) sums[b] = carry + part[threadIdx.x] - c;
    __syncthreads();
    if (threadIdx.x == 1023) carry += part[1023];
    __syncthreads();
  }
}
static __global__ void __launch_bounds__(kTScan)
    tr_scan_apply_kernel(uint32_t* __restrict__ v, int64_t n, const uint32_t* __restrict__ sums) {
  __shared__ uint32_t wsum[kTScan / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t i = (int64_t)blockIdx.x * kTScan + threadIdx.x;
  const uint32_t c = i < n ? v[i] : 0;
  uint32_t x = c;  // inclusive scan inside the warp
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t t = __shfl_up_sync(kFull, x, off);
    if (lane >= off) x += t;
  }
  if (lane == 31) wsum[warp] = x;
  __syncthreads();
  uint32_t before = sums[blockIdx.x];
  for (int w = 0; w < warp; ++w) before += wsum[w];
  if (i < n) v[i] = before + x - c;
}

// stable scatter of one pass: a key goes to (scanned start of its digit for this block) +
// (keys of that digit in lower warps of the block) + (its rank among the warp's earlier keys)
static __global__ void __launch_bounds__(kRadixWarps * kWarp)
    tr_scatter_kernel(const uint32_t* __restrict__ key, const uint32_t* __restrict__ val, int64_t n,
                      int shift, int64_t nblk, const uint32_t* __restrict__ hist,
                      uint32_t* __restrict__ key_out, uint32_t* __restrict__ val_out) {
  __shared__ uint32_t cnt[kRadixWarps][256];
  radix_count(key, n, shift, cnt);
  {
    const int d = threadIdx.x;
    uint32_t run = hist[(int64_t)d * nblk + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kRadixWarps; ++w) {
      const uint32_t c = cnt[w][d];
      cnt[w][d] = run;     // from now on: next free position of digit d for warp w
      run += c;
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned lt = (1u << lane) - 1u;
  const int64_t base = (int64_t)blockIdx.x * kRadixChunk + (int64_t)warp * (kRadixIters * kWarp);
  for (int it = 0; it < kRadixIters; ++it) {
    const int64_t i = base + it * kWarp + lane;
    const bool ok = i < n;
    const uint32_t k = ok ? key[i] : 0u;
    const uint32_t v = ok ? val[i] : 0u;
    const uint32_t d = ok ? ((k >> shift) & 255u) : 256u;   // lanes past the end match only each other
    const unsigned same = __match_any_sync(kFull, d);
    const int rank = __popc(same & lt);
    uint32_t pos = 0;
    if (ok) pos = cnt[warp][d] + rank;
    __syncwarp();
    if (ok && rank == 0) cnt[warp][d] += __popc(same);
    __syncwarp();
    if (ok) {
      key_out[pos] = k;
      val_out[pos] = v;
    }
  }
}


// scratch words (uint32) behind the four key/payload arrays: histogram + scan sums
inline int64_t radix_hist_words(int64_t n) {
  const int64_t nh = 256 * ceil_div(n > 0 ? n : 1, kRadixChunk);
  return nh + ceil_div(nh, kTScan) + 64;
}

// Sorts n pairs by the low `passes` digits of the key.  key[0]/val[0] hold the input; returns the
// index (0 or 1) of the buffers that hold the result.  hist: radix_hist_words(n) words.
inline int radix_sort_pairs(uint32_t* key[2], uint32_t* val[2], int64_t n, int passes, uint32_t* hist,
                            cudaStream_t st) {
  const int64_t nblk = ceil_div(n, kRadixChunk);
  const int64_t nh = 256 * nblk, nsum = ceil_div(nh, kTScan);
  uint32_t* sums = hist + nh;
  int cur = 0;
  for (int p = 0; p < passes; ++p) {
    const int shift = 8 * p;
    tr_hist_kernel<<<(unsigned)nblk, kRadixWarps * kWarp, 0, st>>>(key[cur], n, shift, nblk, hist);
    tr_block_sum_kernel<<<(unsigned)nsum, kTScan, 0, st>>>(hist, nh, sums);
    tr_scan_sums_kernel<<<1, 1024, 0, st>>>(sums, nsum);
    tr_scan_apply_kernel<<<(unsigned)nsum, kTScan, 0, st>>>(hist, nh, sums);
    tr_scatter_kernel<<<(unsigned)nblk, kRadixWarps * kWarp, 0, st>>>(key[cur], val[cur], n, shift, nblk,
                                                                     hist, key[cur ^ 1], val[cur ^ 1]);
    cur ^= 1;
  }
  return cur;
}

}  // namespace hc
