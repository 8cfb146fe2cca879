// Admission scores, quantile threshold, deterministic admission with history
// writeback, and eviction.
//
// Replaces record_history_kernel_used_mask (src/cpp/src/grad_check.cu:6-68)
// and the torch arithmetic of HistoryCache.update_history
// (hiscache/history_cache.py:180-254) and HistoryTable.record_history /
// evict_by_* (hiscache/history_table.py:128-254).  The reference takes ring
// slots with atomicInc in warp-scheduling order; here slots follow an
// exclusive scan of the admission mask, so the remaps are reproducible.
#include "common.cuh"

namespace hc {

// ---------------------------------------------------------------------------
// scores
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    score_rows_kernel(const float* __restrict__ x, int64_t n, int feat, int64_t stride, int kind,
                      float* __restrict__ score) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n) return;
  const float s = row_score(x + r * stride, feat, kind, lane);
  if (lane == 0) score[r] = s;
}

// ---------------------------------------------------------------------------
// quantile threshold: exact radix select of two order statistics + lerp
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t order_key(float x) {
  if (x != x) return 0xFFFFFFFFu;  // NaN sorts last
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(b);
}

// rank = q * (n - 1) in fp32 and the two order statistics around it (torch.quantile)
struct Ranks {
  int64_t n, k_lo, k_hi;
  float w;
};
__device__ __forceinline__ Ranks quantile_ranks(int64_t n_all, const int64_t* n_dev, float q) {
  // with n_dev the quantile is taken over the *n_dev smallest of the n_all scores: the caller
  // sets the scores of padding rows to +inf, which sorts them last
  Ranks r;
  r.n = n_all;
  if (n_dev) {
    r.n = n_dev[0];
    if (r.n > n_all) r.n = n_all;
  }
  if (r.n < 1) {
    r.k_lo = r.k_hi = 0;
    r.w = 0.f;
    return r;
  }
  const float pos = __fmul_rn(q, (float)(r.n - 1));
  r.k_lo = (int64_t)pos;  // truncation, pos >= 0
  if (r.k_lo > r.n - 1) r.k_lo = r.n - 1;
  if (r.k_lo < 0) r.k_lo = 0;
  r.k_hi = (int64_t)ceilf(pos);
  if (r.k_hi > r.n - 1) r.k_hi = r.n - 1;
  if (r.k_hi < 0) r.k_hi = 0;
  r.w = __fsub_rn(pos, (float)r.k_lo);
  return r;
}
__device__ __forceinline__ float quantile_lerp(uint32_t key_lo, uint32_t key_hi, float w) {
  const float lo = key_to_float(key_lo), hi = key_to_float(key_hi);
  const float diff = __fsub_rn(hi, lo);
  // torch's lerp with its fused multiply-add (CPU AVX2+ and CUDA builds)
  return fabsf(w) < 0.5f ? __fmaf_rn(w, diff, lo) : __fmaf_rn(-diff, __fsub_rn(1.f, w), hi);
}

// ---- up to kSelSmall scores: one block, keys staged once in shared memory ----------------
// One global read, then four 8-bit radix passes over shared memory find the k_lo-th key; the
// k_hi-th (k_lo or k_lo + 1) is the same key when enough copies exist, else the smallest larger
// key: one more pass.
constexpr int kSelSmall = 48 * 1024;
constexpr int kSelThreads = 1024;

__global__ void __launch_bounds__(kSelThreads)
    select_small_kernel(const float* __restrict__ score, int64_t n_all, const int64_t* n_dev, float q,
                        float* __restrict__ thres) {
  extern __shared__ uint32_t keys[];   // [n_all]
  __shared__ uint32_t hist[256];
  __shared__ uint32_t bcast[3];
  const Ranks rk = quantile_ranks(n_all, n_dev, q);
  if (rk.n < 1) {
    if (threadIdx.x == 0) thres[0] = __int_as_float(0x7fc00000);
    return;
  }
  const int n = (int)n_all;
  int has_nan = 0;
  for (int i = threadIdx.x; i < n; i += kSelThreads) {
    const float v = score[i];
    has_nan |= (v != v);
    keys[i] = order_key(v);
  }
  has_nan = __syncthreads_or(has_nan);
  uint32_t prefix = 0, mask = 0;
  uint32_t k = (uint32_t)rk.k_lo, below = 0;   // below: keys smaller than the current prefix range
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kSelThreads) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kSelThreads) {
      const uint32_t key = keys[i];
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x < 32) {   // one warp scans the 256 bins (8 per lane)
      uint32_t c[8], tot = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { c[j] = hist[threadIdx.x * 8 + j]; tot += c[j]; }
      uint32_t inc = tot;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t t = __shfl_up_sync(kFull, inc, off);
        if ((int)threadIdx.x >= off) inc += t;
      }
      uint32_t run = inc - tot;   // keys in bins of lower lanes
      if (k >= run && k < inc) {  // the wanted key is in one of this lane's bins
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (k < run + c[j]) {
            bcast[0] = threadIdx.x * 8 + j;
            bcast[1] = k - run;
            bcast[2] = run;
            break;
          }
          run += c[j];
        }
      }
    }
    __syncthreads();
    prefix |= bcast[0] << shift;
    mask |= 255u << shift;
    k = bcast[1];
    below += bcast[2];
    __syncthreads();
  }
  const uint32_t key_lo = prefix;
  // copies of key_lo occupy ranks [below, below + copies); key_hi is key_lo if k_hi falls inside
  uint32_t key_hi = key_lo;
  if (rk.k_hi != rk.k_lo) {
    uint32_t copies = 0, next = 0xFFFFFFFFu;
    for (int i = threadIdx.x; i < n; i += kSelThreads) {
      const uint32_t key = keys[i];
      copies += (key == key_lo);
      if (key > key_lo && key < next) next = key;
    }
    if (threadIdx.x == 0) { hist[0] = 0; hist[1] = 0xFFFFFFFFu; }
    __syncthreads();
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      copies += __shfl_xor_sync(kFull, copies, off);
      const uint32_t o = __shfl_xor_sync(kFull, next, off);
      next = o < next ? o : next;
    }
    if ((threadIdx.x & 31) == 0) {
      atomicAdd(&hist[0], copies);
      atomicMin(&hist[1], next);
    }
    __syncthreads();
    if ((uint32_t)rk.k_hi >= below + hist[0]) key_hi = hist[1];
  }
  if (threadIdx.x == 0)
    thres[0] = has_nan ? __int_as_float(0x7fc00000) : quantile_lerp(key_lo, key_hi, rk.w);
}

// ---- any size: histograms by many blocks, digit choice by one ----------------------------
// Both order statistics descend together (two prefixes); four passes of
//   sel_hist (grid over the scores) -> sel_pick (one block), state in caller scratch.
struct SelState {
  uint32_t prefix[2];
  uint32_t mask;
  int has_nan;
  long long k[2];
  uint32_t hist[2][256];
};

__global__ void __launch_bounds__(256) sel_init_kernel(SelState* st, int64_t n_all, const int64_t* n_dev, float q) {
  const Ranks rk = quantile_ranks(n_all, n_dev, q);
  if (threadIdx.x == 0) {
    st->prefix[0] = st->prefix[1] = 0;
    st->mask = 0;
    st->has_nan = rk.n < 1 ? 1 : 0;   // no valid score: NaN
    st->k[0] = rk.k_lo;
    st->k[1] = rk.k_hi;
  }
  for (int i = threadIdx.x; i < 512; i += blockDim.x) (&st->hist[0][0])[i] = 0;
}

__global__ void __launch_bounds__(256)
    sel_hist_kernel(const float* __restrict__ score, int64_t n, int shift, SelState* st) {
  __shared__ uint32_t h[2][256];
  for (int i = threadIdx.x; i < 512; i += blockDim.x) (&h[0][0])[i] = 0;
  __syncthreads();
  const uint32_t p0 = st->prefix[0], p1 = st->prefix[1], mask = st->mask;
  int nan = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = score[i];
    nan |= (v != v);
    const uint32_t key = order_key(v);
    const uint32_t d = (key >> shift) & 255u;
    if ((key & mask) == p0) atomicAdd(&h[0][d], 1u);
    if ((key & mask) == p1) atomicAdd(&h[1][d], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 512; i += blockDim.x) {
    const uint32_t c = (&h[0][0])[i];
    if (c) atomicAdd(&(&st->hist[0][0])[i], c);
  }
  if (shift == 24 && __syncthreads_or(nan) && threadIdx.x == 0) atomicOr(&st->has_nan, 1);
}

__global__ void __launch_bounds__(64) sel_pick_kernel(SelState* st, int shift, float q, int64_t n_all,
                                                      const int64_t* n_dev, float* __restrict__ thres) {
  const int s = threadIdx.x >> 5, lane = threadIdx.x & 31;   // warp s handles order statistic s
  uint32_t c[8];
  unsigned long long tot = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) { c[j] = st->hist[s][lane * 8 + j]; tot += c[j]; }
  unsigned long long inc = tot;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned long long t = __shfl_up_sync(kFull, inc, off);
    if (lane >= off) inc += t;
  }
  unsigned long long run = inc - tot;
  const unsigned long long k = (unsigned long long)st->k[s];
  uint32_t digit = 0xFFFFFFFFu;
  long long rem = 0;
  if (k >= run && k < inc) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (digit == 0xFFFFFFFFu && k < run + c[j]) { digit = lane * 8 + j; rem = (long long)(k - run); }
      run += c[j];
    }
  }
  // exactly one lane found it (or none when there is no valid score)
  const unsigned who = __ballot_sync(kFull, digit != 0xFFFFFFFFu);
  const int src = who ? __ffs(who) - 1 : 0;
  digit = __shfl_sync(kFull, digit, src);
  rem = __shfl_sync(kFull, rem, src);
  if (!who) { digit = 0; rem = 0; }
  __syncthreads();    // all reads of hist are done
  if (lane == 0) {
    st->prefix[s] |= digit << shift;
    st->k[s] = rem;
  }
  for (int i = lane; i < 256; i += 32) st->hist[s][i] = 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    st->mask |= 255u << shift;
    if (shift == 0) {
      const Ranks rk = quantile_ranks(n_all, n_dev, q);
      thres[0] = st->has_nan ? __int_as_float(0x7fc00000) : quantile_lerp(st->prefix[0], st->prefix[1], rk.w);
    }
  }
}

// ---------------------------------------------------------------------------
// admission
// ---------------------------------------------------------------------------
constexpr int kAdmitBlock = 1024;

struct AdmitArgs {
  int mode;  // 0 = per-layer table ring (grad_check.cu:6-46), 1 = unified cache buffer
  int64_t n;
  const float* rows; int64_t row_stride;   // candidate rows, fp32
  void* buffer; int buf_dtype; int width;  // destination rows
  int64_t capacity;
  const uint8_t* used;
  const int64_t* sub_to_full;
  const int64_t* sub_map;   // sub_to_history / sub2embed
  const float* score; const float* thres;
  int64_t* slot_to_full;    // history_to_full / embed2full
  int64_t* full_to_slot;    // full_to_history / full2embed
  int64_t* header;
  int64_t* checkin; int64_t glb_iter;
  // cache mode only
  int in_feat; int64_t total_num_node; const int64_t* feat2full; int64_t feat2full_len;
  int reset_header;
  int64_t* n_admitted;
  // scratch
  int64_t* block_counts;   // [nblocks]
  int64_t* block_offsets;  // [nblocks]
  int64_t* meta;           // [0] admitted (effective) [1] header before [2] raw admitted
  int64_t nblocks;
};

__device__ __forceinline__ bool admit_flag(const AdmitArgs& a, int64_t i, float thres) {
  if (i >= a.n) return false;
  if (a.sub_map[i] != -1) return false;
  if (a.used != nullptr && a.used[i] == 0) return false;
  if (a.mode == 0) return !(thres != 0.f && a.score[i] > thres);
  return a.score[i] < thres;
}

// exclusive rank of each thread's flag inside the block + block total
__device__ __forceinline__ int block_rank(bool flag, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned bal = __ballot_sync(kFull, flag);
  const int in_warp = __popc(bal & ((1u << lane) - 1u));
  if (lane == 0) warp_sums[warp] = __popc(bal);
  __syncthreads();
  int before = 0, sum = 0;
  const int nw = blockDim.x >> 5;
  for (int w = 0; w < nw; ++w) {
    const int c = warp_sums[w];
    if (w < warp) before += c;
    sum += c;
  }
  *total = sum;
  __syncthreads();
  return before + in_warp;
}

__global__ void __launch_bounds__(kAdmitBlock) admit_count_kernel(const AdmitArgs a) {
  const int64_t i = (int64_t)blockIdx.x * kAdmitBlock + threadIdx.x;
  const bool f = admit_flag(a, i, a.thres[0]);
  const int c = __syncthreads_count(f);
  if (threadIdx.x == 0) a.block_counts[blockIdx.x] = c;
}

__global__ void __launch_bounds__(1024) admit_scan_kernel(const AdmitArgs a) {
  __shared__ int64_t part[1024];
  __shared__ int64_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < a.nblocks; base += 1024) {
    const int64_t b = base + threadIdx.x;
    const int64_t c = b < a.nblocks ? a.block_counts[b] : 0;
    part[threadIdx.x] = c;
    __syncthreads();
    // Hillis-Steele inclusive scan over 1024 entries
    for (int off = 1; off < 1024; off <<= 1) {
      int64_t v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
      __syncthreads();
      part[threadIdx.x] += v;
      __syncthreads();
    }
    if (b < a.nblocks) a.block_offsets[b] = carry + part[threadIdx.x] - c;
    __syncthreads();
    if (threadIdx.x == 1023) carry += part[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const int64_t total = carry;
    int64_t h0 = a.header[0];
    int64_t eff = total;
    if (a.mode == 0) {
      if (a.capacity > 0) {
        h0 %= a.capacity;
        if (h0 < 0) h0 += a.capacity;
        a.header[0] = (h0 + total) % a.capacity;
      } else {
        eff = 0;
      }
    } else {
      if (a.reset_header) h0 = 0;
      if (h0 < 0) h0 = 0;
      const int64_t room = a.capacity > h0 ? a.capacity - h0 : 0;
      if (eff > room) eff = room;
      a.header[0] = h0 + eff;
    }
    a.meta[0] = eff;
    a.meta[1] = h0;
    a.meta[2] = total;
    if (a.n_admitted) a.n_admitted[0] = eff;
  }
}

// Phase 2: everything that must be unmapped is unmapped before anything is set.
__global__ void __launch_bounds__(kAdmitBlock) admit_invalidate_kernel(const AdmitArgs a) {
  __shared__ int warp_sums[kAdmitBlock / 32];
  const int64_t i = (int64_t)blockIdx.x * kAdmitBlock + threadIdx.x;
  const bool f = admit_flag(a, i, a.thres[0]);
  int total_blk;
  const int64_t rank = a.block_offsets[blockIdx.x] + block_rank(f, warp_sums, &total_blk);
  const int64_t eff = a.meta[0], h0 = a.meta[1];
  if (a.mode == 0) {
    if (f && a.capacity > 0) {
      const int64_t slot = (h0 + rank) % a.capacity;
      const int64_t old = a.slot_to_full[slot];
      if (old != -1 && a.full_to_slot[old] == slot) a.full_to_slot[old] = -1;
    }
  } else {
    if (f && rank < eff) {
      const int64_t slot = h0 + rank;
      const int64_t old = a.slot_to_full[slot];
      if (old != -1) {
        const int64_t cur = a.full_to_slot[old];
        if (cur >= h0 && cur < h0 + eff) a.full_to_slot[old] = -1;
      }
    }
    // raw-feature slots overlapped by embedding slots [h0, h0+eff)
    if (a.feat2full) {
      const int64_t fb = h0 * a.width / a.in_feat;
      int64_t fe = ((h0 + eff) * a.width + a.in_feat - 1) / a.in_feat;
      if (fe > a.feat2full_len) fe = a.feat2full_len;
      for (int64_t k = fb + i; k < fe; k += (int64_t)gridDim.x * kAdmitBlock)
        a.full_to_slot[a.feat2full[k]] = -1;
    }
  }
}

// Phase 3: copy rows, set both maps.
__global__ void __launch_bounds__(kAdmitBlock) admit_write_kernel(const AdmitArgs a, int vec_ok) {
  __shared__ int warp_sums[kAdmitBlock / 32];
  __shared__ int64_t list_row[kAdmitBlock];
  __shared__ int64_t list_slot[kAdmitBlock];
  const int64_t i = (int64_t)blockIdx.x * kAdmitBlock + threadIdx.x;
  const bool f = admit_flag(a, i, a.thres[0]);
  int total_blk;
  const int local = block_rank(f, warp_sums, &total_blk);
  const int64_t rank = a.block_offsets[blockIdx.x] + local;
  const int64_t eff = a.meta[0], h0 = a.meta[1], total = a.meta[2];
  if (f) {
    int64_t slot = -1;  // -1: admitted but displaced / out of room
    if (a.mode == 0) {
      if (a.capacity > 0 && rank >= total - a.capacity) slot = (h0 + rank) % a.capacity;
    } else if (rank < eff) {
      slot = h0 + rank;
    }
    list_row[local] = i;
    list_slot[local] = slot;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int k = warp; k < total_blk; k += kAdmitBlock / 32) {
    const int64_t row = list_row[k], slot = list_slot[k];
    const int64_t full = a.sub_to_full[row];
    if (slot < 0) {
      // ring mode, more admissions than slots: applied one by one, this row
      // was written and then displaced, which leaves it unmapped
      if (a.mode == 0 && lane == 0) a.full_to_slot[full] = -1;
      continue;
    }
    const float* __restrict__ src = a.rows + row * a.row_stride;
    if (a.buf_dtype == HC_F32) {
      float* dst = reinterpret_cast<float*>(a.buffer) + slot * a.width;
      if (vec_ok)
        for (int v = lane; v < (a.width >> 2); v += kWarp)
          reinterpret_cast<uint4*>(dst)[v] = ldg16(src + 4 * v);
      else
        for (int c = lane; c < a.width; c += kWarp) dst[c] = src[c];
    } else {
      __half* dst = reinterpret_cast<__half*>(a.buffer) + slot * a.width;
      if (vec_ok)
        for (int v = lane; v < (a.width >> 2); v += kWarp) {
          float f4[4];
          Vec16<float>::unpack(ldg16(src + 4 * v), f4);
          __half2 lo = __floats2half2_rn(f4[0], f4[1]), hi = __floats2half2_rn(f4[2], f4[3]);
          uint2 pk;
          pk.x = *reinterpret_cast<uint32_t*>(&lo);
          pk.y = *reinterpret_cast<uint32_t*>(&hi);
          reinterpret_cast<uint2*>(dst)[v] = pk;
        }
      else
        for (int c = lane; c < a.width; c += kWarp) dst[c] = __float2half_rn(src[c]);
    }
    if (lane == 0) {
      a.full_to_slot[full] = slot;
      a.slot_to_full[slot] = full;
      if (a.checkin) a.checkin[slot] = a.glb_iter;
    }
  }
}

static int run_admit(AdmitArgs& a, void* scratch, cudaStream_t st) {
  if (a.n == 0 && !(a.mode == 1 && a.reset_header)) {
    if (a.n_admitted) HC_CUDA(cudaMemsetAsync(a.n_admitted, 0, sizeof(int64_t), st));
    return 0;
  }
  HC_REQUIRE(scratch != nullptr, HC_ERR_NULL);
  HC_REQUIRE(aligned_to(scratch, 8), HC_ERR_ALIGN);
  a.nblocks = a.n > 0 ? ceil_div(a.n, kAdmitBlock) : 1;
  HC_REQUIRE(a.nblocks <= 0x7fffffffLL, HC_ERR_SIZE);
  int64_t* s = reinterpret_cast<int64_t*>(scratch);
  a.meta = s;
  a.block_counts = s + 8;
  a.block_offsets = s + 8 + a.nblocks;
  const unsigned grid = (unsigned)a.nblocks;
  admit_count_kernel<<<grid, kAdmitBlock, 0, st>>>(a);
  admit_scan_kernel<<<1, 1024, 0, st>>>(a);
  admit_invalidate_kernel<<<grid, kAdmitBlock, 0, st>>>(a);
  const int es = dtype_size(a.buf_dtype);
  const int vec_ok = a.width % 4 == 0 && aligned16(a.rows) && (a.row_stride % 4) == 0 &&
                     aligned_to(a.buffer, a.buf_dtype == HC_F32 ? 16 : 8) && es != 0;
  admit_write_kernel<<<grid, kAdmitBlock, 0, st>>>(a, vec_ok);
  HC_LAUNCH_OK();
  return 0;
}

// ---------------------------------------------------------------------------
// eviction
// ---------------------------------------------------------------------------
__global__ void evict_stale_kernel(int64_t* checkin, int64_t* h2f, int64_t* f2h, int64_t cap,
                                   int64_t stale_iter) {
  const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= cap) return;
  const int64_t c = checkin[s];
  if (c > -1 && c <= stale_iter) {
    const int64_t full = h2f[s];
    checkin[s] = -1;
    h2f[s] = -1;
    if (full != -1) f2h[full] = -1;
  }
}

// the same with the iteration number read from device memory (steps replayed from a CUDA graph
// cannot carry it as a launch argument)
__global__ void evict_stale_dev_kernel(int64_t* checkin, int64_t* h2f, int64_t* f2h, int64_t cap,
                                       const int64_t* __restrict__ iter_dev, int64_t limit) {
  const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= cap) return;
  const int64_t c = checkin[s];
  if (c > -1 && c <= iter_dev[0] - limit) {
    const int64_t full = h2f[s];
    checkin[s] = -1;
    h2f[s] = -1;
    if (full != -1) f2h[full] = -1;
  }
}
__global__ void stamp_checkin_kernel(int64_t* checkin, int64_t cap, int64_t marker,
                                     const int64_t* __restrict__ iter_dev) {
  const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (s < cap && checkin[s] == marker) checkin[s] = iter_dev[0];
}

__global__ void evict_by_score_kernel(const int64_t* __restrict__ sub_to_history,
                                      const float* __restrict__ score,
                                      const float* __restrict__ thres, int64_t n, int64_t* checkin,
                                      int64_t* h2f, int64_t* f2h) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int64_t slot = sub_to_history[r];
  if (slot == -1 || !(score[r] >= thres[0])) return;
  const int64_t full = h2f[slot];
  if (full != -1) f2h[full] = -1;
  h2f[slot] = -1;
  checkin[slot] = -1;
}

}  // namespace hc

using namespace hc;

extern "C" int hc_score_rows(const float* x, int64_t n, int32_t feat, int64_t stride, int32_t kind,
                             float* score, void* stream) {
  HC_REQUIRE(n >= 0 && feat > 0, HC_ERR_SIZE);
  HC_REQUIRE(kind == HC_SCORE_L2 || kind == HC_SCORE_L1, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(x && score, HC_ERR_NULL);
  if (stride == 0) stride = feat;
  HC_REQUIRE(stride >= feat, HC_ERR_SIZE);
  const int64_t blocks = ceil_div(n, 8);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  score_rows_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      x, n, feat, stride, kind, score);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int64_t hc_select_scratch_bytes(int64_t n) {
  return n > kSelSmall ? (int64_t)sizeof(SelState) + 64 : 0;
}

static int select_launch(const float* score, int64_t n, const int64_t* n_valid, float q, float* thres,
                         void* scratch, cudaStream_t st) {
  if (n <= kSelSmall) {
    const size_t smem = (size_t)n * sizeof(uint32_t);
    if (smem > 40 * 1024) {
      // raised once per device (not a stream operation, so keep it out of stream captures)
      static bool raised[64] = {};
      int devno = 0;
      HC_CUDA(cudaGetDevice(&devno));
      if (devno >= 0 && devno < 64 && !raised[devno]) {
        HC_CUDA(cudaFuncSetAttribute(select_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kSelSmall * (int)sizeof(uint32_t)));
        raised[devno] = true;
      }
    }
    select_small_kernel<<<1, kSelThreads, smem, st>>>(score, n, n_valid, q, thres);
    HC_LAUNCH_OK();
    return 0;
  }
  HC_REQUIRE(scratch != nullptr && aligned_to(scratch, 8), HC_ERR_NULL);
  HC_REQUIRE(n < 0xffffffffLL, HC_ERR_SIZE);
  SelState* state = reinterpret_cast<SelState*>(scratch);
  int64_t blocks = ceil_div(n, 256 * 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  sel_init_kernel<<<1, 256, 0, st>>>(state, n, n_valid, q);
  for (int shift = 24; shift >= 0; shift -= 8) {
    sel_hist_kernel<<<(unsigned)blocks, 256, 0, st>>>(score, n, shift, state);
    sel_pick_kernel<<<1, 64, 0, st>>>(state, shift, q, n, n_valid, thres);
  }
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_select_threshold(const float* score, int64_t n, float q, float* thres,
                                   void* scratch, void* stream) {
  HC_REQUIRE(n > 0, HC_ERR_SIZE);
  HC_REQUIRE(score && thres, HC_ERR_NULL);
  HC_REQUIRE(q >= 0.f && q <= 1.f, HC_ERR_SIZE);
  return select_launch(score, n, nullptr, q, thres, scratch, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int hc_select_threshold_counted(const float* score, int64_t n, const int64_t* n_valid,
                                           float q, float* thres, void* scratch, void* stream) {
  HC_REQUIRE(n > 0, HC_ERR_SIZE);
  HC_REQUIRE(score && thres && n_valid, HC_ERR_NULL);
  HC_REQUIRE(q >= 0.f && q <= 1.f, HC_ERR_SIZE);
  return select_launch(score, n, n_valid, q, thres, scratch, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int64_t hc_admit_scratch_bytes(int64_t n) {
  const int64_t nb = n > 0 ? ceil_div(n, kAdmitBlock) : 1;
  return (8 + 2 * nb) * (int64_t)sizeof(int64_t);
}

extern "C" int hc_record_history(const float* buffer_new, int64_t new_stride, int64_t n,
                                 void* buffer_all, int32_t table_dtype, int64_t capacity,
                                 int32_t history_size, const uint8_t* used_mask,
                                 const int64_t* sub_to_full, const int64_t* sub_to_history,
                                 int64_t* history_to_full, int64_t* full_to_history,
                                 int64_t* header, const float* score, const float* thres,
                                 int64_t* checkin_iter, int64_t glb_iter, int64_t* n_admitted,
                                 void* scratch, void* stream) {
  HC_REQUIRE(n >= 0 && capacity >= 0 && history_size > 0, HC_ERR_SIZE);
  HC_REQUIRE(dtype_size(table_dtype) != 0, HC_ERR_DTYPE);
  if (n > 0) {
    HC_REQUIRE(buffer_new && sub_to_full && sub_to_history && history_to_full && full_to_history &&
                   header && score && thres && checkin_iter,
               HC_ERR_NULL);
    HC_REQUIRE(capacity == 0 || buffer_all != nullptr, HC_ERR_NULL);
  }
  if (new_stride == 0) new_stride = history_size;
  HC_REQUIRE(new_stride >= history_size, HC_ERR_SIZE);
  AdmitArgs a{};
  a.mode = 0; a.n = n; a.rows = buffer_new; a.row_stride = new_stride;
  a.buffer = buffer_all; a.buf_dtype = table_dtype; a.width = history_size;
  a.capacity = capacity; a.used = used_mask; a.sub_to_full = sub_to_full;
  a.sub_map = sub_to_history; a.score = score; a.thres = thres;
  a.slot_to_full = history_to_full; a.full_to_slot = full_to_history; a.header = header;
  a.checkin = checkin_iter; a.glb_iter = glb_iter; a.n_admitted = n_admitted;
  if (capacity == 0) {
    // an empty table admits nothing (history_table.py:130-131 skips such layers)
    if (n_admitted)
      HC_CUDA(cudaMemsetAsync(n_admitted, 0, sizeof(int64_t), reinterpret_cast<cudaStream_t>(stream)));
    return 0;
  }
  return run_admit(a, scratch, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int hc_cache_admit(const float* produced, int64_t prod_stride, int64_t n, void* buffer,
                              int32_t buf_dtype, int32_t hidden, int32_t in_feat,
                              int64_t embed_capacity, const int64_t* sub_to_full,
                              const int64_t* sub2embed, const float* score, const float* thres,
                              int64_t* full2embed, int64_t total_num_node, int64_t* embed2full,
                              const int64_t* feat2full, int64_t feat2full_len, int64_t* header,
                              int32_t reset_header, const uint8_t* valid, int64_t* n_admitted,
                              void* scratch, void* stream) {
  HC_REQUIRE(n >= 0 && embed_capacity >= 0 && hidden > 0 && in_feat > 0 && total_num_node >= 0 &&
                 feat2full_len >= 0,
             HC_ERR_SIZE);
  HC_REQUIRE(dtype_size(buf_dtype) != 0, HC_ERR_DTYPE);
  HC_REQUIRE(header != nullptr, HC_ERR_NULL);
  if (n > 0)
    HC_REQUIRE(produced && buffer && sub_to_full && sub2embed && score && thres && full2embed &&
                   embed2full,
               HC_ERR_NULL);
  if (prod_stride == 0) prod_stride = hidden;
  HC_REQUIRE(prod_stride >= hidden, HC_ERR_SIZE);
  AdmitArgs a{};
  a.mode = 1; a.n = n; a.rows = produced; a.row_stride = prod_stride;
  a.buffer = buffer; a.buf_dtype = buf_dtype; a.width = hidden; a.capacity = embed_capacity;
  a.sub_to_full = sub_to_full; a.sub_map = sub2embed; a.score = score; a.thres = thres;
  a.slot_to_full = embed2full; a.full_to_slot = full2embed; a.header = header;
  a.in_feat = in_feat; a.total_num_node = total_num_node;
  a.feat2full = feat2full_len > 0 ? feat2full : nullptr; a.feat2full_len = feat2full_len;
  a.reset_header = reset_header; a.n_admitted = n_admitted; a.used = valid;
  if (n == 0 && reset_header) {
    // nothing to admit, but the ring still restarts
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    HC_CUDA(cudaMemsetAsync(header, 0, sizeof(int64_t), st));
    if (n_admitted) HC_CUDA(cudaMemsetAsync(n_admitted, 0, sizeof(int64_t), st));
    return 0;
  }
  return run_admit(a, scratch, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int hc_evict_stale(int64_t* checkin_iter, int64_t* history_to_full,
                              int64_t* full_to_history, int64_t capacity, int64_t glb_iter,
                              int64_t limit, void* stream) {
  HC_REQUIRE(capacity >= 0, HC_ERR_SIZE);
  if (capacity == 0) return 0;
  HC_REQUIRE(checkin_iter && history_to_full && full_to_history, HC_ERR_NULL);
  const int64_t blocks = ceil_div(capacity, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  evict_stale_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      checkin_iter, history_to_full, full_to_history, capacity, glb_iter - limit);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_evict_stale_dev(int64_t* checkin_iter, int64_t* history_to_full,
                                  int64_t* full_to_history, int64_t capacity,
                                  const int64_t* glb_iter_dev, int64_t limit, void* stream) {
  HC_REQUIRE(capacity >= 0, HC_ERR_SIZE);
  if (capacity == 0) return 0;
  HC_REQUIRE(checkin_iter && history_to_full && full_to_history && glb_iter_dev, HC_ERR_NULL);
  const int64_t blocks = ceil_div(capacity, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  evict_stale_dev_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      checkin_iter, history_to_full, full_to_history, capacity, glb_iter_dev, limit);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_stamp_checkin(int64_t* checkin_iter, int64_t capacity, int64_t marker,
                                const int64_t* glb_iter_dev, void* stream) {
  HC_REQUIRE(capacity >= 0, HC_ERR_SIZE);
  if (capacity == 0) return 0;
  HC_REQUIRE(checkin_iter && glb_iter_dev, HC_ERR_NULL);
  const int64_t blocks = ceil_div(capacity, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  stamp_checkin_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      checkin_iter, capacity, marker, glb_iter_dev);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_evict_by_score(const int64_t* sub_to_history, const float* score,
                                 const float* thres, int64_t n, int64_t* checkin_iter,
                                 int64_t* history_to_full, int64_t* full_to_history, void* stream) {
  HC_REQUIRE(n >= 0, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(sub_to_history && score && thres && checkin_iter && history_to_full && full_to_history,
             HC_ERR_NULL);
  const int64_t blocks = ceil_div(n, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  evict_by_score_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      sub_to_history, score, thres, n, checkin_iter, history_to_full, full_to_history);
  HC_LAUNCH_OK();
  return 0;
}


// ---------------------------------------------------------------------------
// Ring admission with built-in scratch (no allocation by anybody)
// ---------------------------------------------------------------------------
// hc_record_history needs a few KB of device scratch that the caller allocates.  Some
// callers have nothing to allocate with: a plain-C, cgo or JNI host that was only handed the
// input and output buffers and holds no handle to the framework's device allocator, or a
// training loop whose memory is entirely owned by a caching allocator and in which a raw
// cudaMalloc / cudaFree would stall the device.  For them the scratch lives in this
// file-scope array, which every GPU that loads the library carries until the process exits.
namespace hc {

constexpr int64_t kNoAllocMaxRows = 1 << 20;  // HC_NOALLOC_MAX_ROWS
constexpr int64_t kNoAllocBytes = (8 + 2 * (kNoAllocMaxRows / kAdmitBlock)) * (int64_t)sizeof(int64_t);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kNoAllocMaxDevices = 64;
// Device address of g_noalloc_scratch per device ordinal.  In host code the array's name is
// only a handle for the runtime, never an address a kernel may be given; the address comes
// from cudaGetSymbolAddress, asked once per device with that device current.
static void* g_noalloc_addr[kNoAllocMaxDevices];

static int noalloc_scratch(void** out) {
  int dev = -1;
  HC_CUDA(cudaGetDevice(&dev));
  HC_REQUIRE(dev >= 0 && dev < kNoAllocMaxDevices, HC_ERR_SIZE);
  void* p = __atomic_load_n(&g_noalloc_addr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    HC_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    HC_REQUIRE(p != nullptr, HC_ERR_NULL);
    __atomic_store_n(&g_noalloc_addr[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return 0;
}

}  // namespace hc

extern "C" int64_t hc_noalloc_max_rows(void) { return hc::kNoAllocMaxRows; }

extern "C" int hc_record_history_noalloc(const float* buffer_new, int64_t new_stride, int64_t n,
                                         void* buffer_all, int32_t table_dtype, int64_t capacity,
                                         int32_t history_size, const uint8_t* used_mask,
                                         const int64_t* sub_to_full,
                                         const int64_t* sub_to_history, int64_t* history_to_full,
                                         int64_t* full_to_history, int64_t* header,
                                         const float* score, const float* thres,
                                         int64_t* checkin_iter, int64_t glb_iter,
                                         int64_t* n_admitted, void* stream) {
  if (n > hc::kNoAllocMaxRows) return -HC_ERR_LIMIT;
  void* scratch = nullptr;
  const int rc = hc::noalloc_scratch(&scratch);
  if (rc != 0) return rc;
  // every scratch word that is read was written earlier in the same call, so the contents
  // left by the previous call need no clearing
  return hc_record_history(buffer_new, new_stride, n, buffer_all, table_dtype, capacity,
                           history_size, used_mask, sub_to_full, sub_to_history, history_to_full,
                           full_to_history, header, score, thres, checkin_iter, glb_iter,
                           n_admitted, scratch, stream);
}
