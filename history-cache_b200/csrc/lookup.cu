// Cache lookup, row gathers and the one-pass assembly of batch.x.
//
// Replaces the torch index arithmetic of HistoryCache.lookup_and_load
// (hiscache/history_cache.py:275-356) and HistoryTable.lookup
// (hiscache/history_table.py:94-125).  The reference builds batch.x with a
// masked host read followed by two more full-width passes; here one kernel
// decides per row between the host-resident table, the raw-feature cache in
// HBM and zeros, and writes the row once.

#include "common.cuh"

namespace hc {

// Moves `units` groups of 8 elements (unit8) or 4 fp32 elements (unit4) of one
// row with 16-byte accesses; `gl`/`G` = lane and width of the lane group.
__device__ __forceinline__ void load_unit8(const void* src, int sdt, int64_t off, float* f) {
  if (sdt == HC_F16) {
    Vec16<__half>::unpack(ldg16(reinterpret_cast<const __half*>(src) + off), f);
  } else {
    Vec16<float>::unpack(ldg16(reinterpret_cast<const float*>(src) + off), f);
    Vec16<float>::unpack(ldg16(reinterpret_cast<const float*>(src) + off + 4), f + 4);
  }
}
__device__ __forceinline__ void store_unit8(void* dst, int ddt, int64_t off, const float* f) {
  if (ddt == HC_F16) {
    __half2 h0 = __floats2half2_rn(f[0], f[1]), h1 = __floats2half2_rn(f[2], f[3]);
    __half2 h2 = __floats2half2_rn(f[4], f[5]), h3 = __floats2half2_rn(f[6], f[7]);
    uint4 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&h0);
    pk.y = *reinterpret_cast<uint32_t*>(&h1);
    pk.z = *reinterpret_cast<uint32_t*>(&h2);
    pk.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(dst) + off) = pk;
  } else {
    float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + off);
    d[0] = make_float4(f[0], f[1], f[2], f[3]);
    d[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

// Copies / converts one row. src == nullptr writes zeros.
//   mode 2: same dtype, 16-byte copies; mode 1: groups of 8 elements with
//   conversion; mode 0: scalar.
__device__ __forceinline__ void move_row(const void* src, int sdt, int64_t soff, void* dst,
                                         int ddt, int64_t doff, int feat, int gl, int G,
                                         int mode) {
  if (mode == 2) {
    const int es = ddt == HC_F16 ? 2 : 4;
    const int nvec = feat * es / 16;
    const char* s = src ? reinterpret_cast<const char*>(src) + soff * es : nullptr;
    char* d = reinterpret_cast<char*>(dst) + doff * es;
    for (int v = gl; v < nvec; v += G)
      reinterpret_cast<uint4*>(d)[v] = s ? ldg16(s + 16 * v) : make_uint4(0u, 0u, 0u, 0u);
  } else if (mode == 1) {
    for (int u = gl; u < (feat >> 3); u += G) {
      float f[8];
      if (src) {
        load_unit8(src, sdt, soff + 8 * u, f);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = 0.f;
      }
      store_unit8(dst, ddt, doff + 8 * u, f);
    }
  } else {
    for (int c = gl; c < feat; c += G)
      store_from_f32(dst, ddt, doff + c, src ? load_as_f32(src, sdt, soff + c) : 0.f);
  }
}

__global__ void map_lookup_kernel(const int64_t* __restrict__ map, int64_t map_len,
                                  const int64_t* __restrict__ ids, int64_t n, int64_t offset,
                                  int64_t force_miss_below, int64_t* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int64_t v = -1;
  if (i >= force_miss_below) {
    int64_t p = ids[i] + offset;
    if (p < 0) p += map_len;  // torch negative indexing
    if (p >= 0 && p < map_len) v = map[p];
  }
  out[i] = v;
}

template <int G>
__global__ void __launch_bounds__(256)
    gather_rows_kernel(const void* __restrict__ table, int tdt, int64_t table_rows,
                       int64_t table_stride, int feat, const int64_t* __restrict__ rows, int64_t n,
                       int zero_missing, void* __restrict__ out, int odt, int64_t out_stride,
                       int mode) {
  const int gl = threadIdx.x % G;
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (i >= n) return;
  int64_t r = rows[i];
  const void* src = table;
  if (r < 0) {
    if (zero_missing) src = nullptr;
    r += table_rows;  // -1 reads the last row
  }
  if (r < 0 || r >= table_rows) src = nullptr;
  move_row(src, tdt, r * table_stride, out, odt, i * out_stride, feat, gl, G, mode);
}

struct LoadArgs {
  const void* host_table; int host_dtype; int64_t host_rows; int64_t host_stride;
  const void* feat_cache; int cache_dtype; int64_t cache_rows; int64_t cache_stride;
  int feat;
  const int64_t* sub_to_full; const int64_t* sub2feat; const uint8_t* used;
  int64_t n;
  void* x; int x_dtype; int64_t x_stride;
  uint8_t* load_mask_out; unsigned long long* stats;
  int host_mode, cache_mode, zero_mode;
  // rows fetched ahead of the step: staged_rows[i] is host_table[sub_to_full[i]] where staged_mask[i]
  const void* staged_rows; const uint8_t* staged_mask; int staged_mode;
  int sparse_out;   // != 0: the staging call (rows that are not loaded need not be written); its grid cap
};

template <int G>
__global__ void __launch_bounds__(256) load_rows_kernel(const LoadArgs a) {
  const int gl = threadIdx.x % G;
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  const bool live = i < a.n;
  int from_host = 0, from_cache = 0, from_staged = 0;
  if (live) {
    const int64_t sf = a.sub2feat ? a.sub2feat[i] : -1;
    const bool used = a.used == nullptr || a.used[i] != 0;
    bool load = used && sf == -1;
    if (load && a.sparse_out) {
      const int64_t g = a.sub_to_full[i];
      load = g >= 0 && g < a.host_rows;
    }
    if (load && a.staged_mask && a.staged_mask[i]) {
      move_row(a.staged_rows, a.x_dtype, i * (int64_t)a.feat, a.x, a.x_dtype, i * a.x_stride, a.feat, gl, G,
               a.staged_mode);
      from_staged = gl == 0;
    } else if (load) {
      const int64_t g = a.sub_to_full[i];
      const bool ok = g >= 0 && g < a.host_rows;
      move_row(ok ? a.host_table : nullptr, a.host_dtype, g * a.host_stride, a.x, a.x_dtype,
               i * a.x_stride, a.feat, gl, G, ok ? a.host_mode : a.zero_mode);
      from_host = gl == 0;
    } else if (sf != -1 && !(a.sparse_out && a.feat_cache == nullptr)) {
      int64_t r = sf < 0 ? sf + a.cache_rows : sf;
      const bool ok = r >= 0 && r < a.cache_rows;
      move_row(ok ? a.feat_cache : nullptr, a.cache_dtype, r * a.cache_stride, a.x, a.x_dtype,
               i * a.x_stride, a.feat, gl, G, ok ? a.cache_mode : a.zero_mode);
      from_cache = gl == 0;
    } else if (!a.sparse_out) {
      move_row(nullptr, a.x_dtype, 0, a.x, a.x_dtype, i * a.x_stride, a.feat, gl, G, a.zero_mode);
    }
    if (a.load_mask_out && gl == 0) a.load_mask_out[i] = load ? 1 : 0;
  }
  if (a.stats) {
    const int h = __syncthreads_count(from_host), c = __syncthreads_count(from_cache);
    const int p = __syncthreads_count(from_staged);
    if (threadIdx.x == 0) {
      if (h) atomicAdd(a.stats, (unsigned long long)h);
      if (c) atomicAdd(a.stats + 1, (unsigned long long)c);
      if (p) atomicAdd(a.stats + 2, (unsigned long long)p);     // only callers that stage rows get here
    }
  }
}

// ---------------------------------------------------------------------------
// batch.x assembly with the rows staged through shared memory by the bulk-copy
// engine (TMA, untiled cp.async.bulk): one copy instruction per row instead of
// one 16-byte load per lane, one bulk store per tile of 32 rows.  Used when no
// conversion is needed (table, cache and batch share a dtype, rows are multiples
// of 16 bytes and the batch rows are contiguous).  Every wait is bounded; a warp
// whose wait runs out stops using the engine and finishes with plain loads.
// ---------------------------------------------------------------------------
constexpr int kBulkWarps = 4;      // warps per block
constexpr int kBulkTile = 32;      // rows per tile = one row per lane
constexpr int kBulkSpin = 1 << 22; // bound of every wait loop
constexpr int kStageBlocks = 16;   // grid of a staging call (hc_stage_host_rows), see stage_rows_kernel

__global__ void __launch_bounds__(kBulkWarps * 32)
    load_rows_bulk_kernel(const LoadArgs a, const int row_bytes, const int64_t tiles) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[kBulkWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char* buf[2];
  buf[0] = smem + (size_t)(warp * 2) * kBulkTile * row_bytes;
  buf[1] = buf[0] + (size_t)kBulkTile * row_bytes;
  const uint32_t bar = smem_u32(&bars[warp]);
  if (lane == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const int es = a.x_dtype == HC_F16 ? 2 : 4;
  bool engine_ok = true;
  uint32_t phase = 0;
  unsigned long long n_host = 0, n_cache = 0, n_staged = 0;
  int which = 0;
  const int64_t warps_total = (int64_t)gridDim.x * kBulkWarps;
  for (int64_t t = (int64_t)blockIdx.x * kBulkWarps + warp; t < tiles; t += warps_total) {
    const int64_t i = t * kBulkTile + lane;
    const bool live = i < a.n;
    const void* src = nullptr;
    bool load = false, from_cache = false, from_staged = false;
    if (live) {
      const int64_t sf = a.sub2feat ? a.sub2feat[i] : -1;
      const bool used = a.used == nullptr || a.used[i] != 0;
      load = used && sf == -1;
      if (load && a.staged_mask && a.staged_mask[i]) {
        src = reinterpret_cast<const char*>(a.staged_rows) + i * (int64_t)row_bytes;
        from_staged = true;
        load = false;
      } else if (load) {
        const int64_t g = a.sub_to_full[i];
        if (g >= 0 && g < a.host_rows)
          src = reinterpret_cast<const char*>(a.host_table) + g * a.host_stride * es;
        else if (a.sparse_out)
          load = false;     // an id outside the table is not staged; the step gives it a zero row
      } else if (sf != -1) {
        const int64_t r = sf < 0 ? sf + a.cache_rows : sf;
        if (r >= 0 && r < a.cache_rows) src = reinterpret_cast<const char*>(a.feat_cache) + r * a.cache_stride * es;
        from_cache = true;
      }
      if (a.load_mask_out) a.load_mask_out[i] = (load || from_staged) ? 1 : 0;
    }
    n_host += __popc(__ballot_sync(kFull, load));
    n_cache += __popc(__ballot_sync(kFull, from_cache));
    n_staged += __popc(__ballot_sync(kFull, from_staged));
    if (a.sparse_out && !__any_sync(kFull, src != nullptr)) continue;   // nothing to move in this tile
    const int64_t left = a.n - t * kBulkTile;
    const int rows_here = (int)(left < kBulkTile ? left : kBulkTile);
    char* xrow = reinterpret_cast<char*>(a.x) + i * (int64_t)row_bytes;
    if (engine_ok) {
      unsigned char* stage = buf[which];
      // the store that last read this buffer must be done with it
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      const unsigned has = __ballot_sync(kFull, src != nullptr);
      if (lane == 0 && has) mbar_expect_tx(bar, (uint32_t)__popc(has) * (uint32_t)row_bytes);
      __syncwarp();
      if (src) {
        bulk_load(smem_u32(stage + (size_t)lane * row_bytes), src, (uint32_t)row_bytes, bar);
      } else if (live) {
        uint4* z = reinterpret_cast<uint4*>(stage + (size_t)lane * row_bytes);
        for (int v = 0; v < row_bytes / 16; ++v) z[v] = make_uint4(0u, 0u, 0u, 0u);
      }
      if (has) {
        int spins = 0;
        while (!mbar_try_wait(bar, phase)) {
          if (++spins > kBulkSpin) { engine_ok = false; break; }
        }
        phase ^= 1u;
      }
      engine_ok = __all_sync(kFull, engine_ok);
      if (engine_ok) {
        // zeros written by lanes must be visible to the bulk store
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0)
          bulk_store(reinterpret_cast<char*>(a.x) + t * kBulkTile * (int64_t)row_bytes,
                     smem_u32(stage), (uint32_t)rows_here * (uint32_t)row_bytes);
        which ^= 1;
        continue;
      }
      // the wait ran out: finish this tile and all later ones with plain loads
    }
    if (live) {
      for (int v = 0; v < row_bytes / 16; ++v)
        reinterpret_cast<uint4*>(xrow)[v] = src ? ldg16(reinterpret_cast<const char*>(src) + 16 * v)
                                                : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  // shared memory must outlive the stores that read it
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  if (!engine_ok) {
    // copies issued before the wait ran out may still be landing: give them one more
    // bounded wait before the block's shared memory is released
    int spins = 0;
    while (!mbar_try_wait(bar, phase ^ 1u) && ++spins < kBulkSpin) {
    }
  }
  if (a.stats && lane == 0) {
    if (n_host) atomicAdd(a.stats, n_host);
    if (n_cache) atomicAdd(a.stats + 1, n_cache);
    if (n_staged) atomicAdd(a.stats + 2, n_staged);
  }
}

__global__ void __launch_bounds__(256)
    owner_lookup_flags_kernel(const int64_t* __restrict__ map, int64_t map_len,
                              const int64_t* __restrict__ ids, int64_t n, int64_t* slots,
                              uint8_t* flags) {
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int64_t id = ids[k];
  const int64_t s = (id >= 0 && id < map_len) ? map[id] : -1;
  if (slots) slots[k] = s;
  flags[k] = s != -1;
}

template <int G>
__global__ void __launch_bounds__(256)
    owner_lookup_rows_kernel(const int64_t* __restrict__ map, int64_t map_len,
                             const int64_t* __restrict__ ids, int64_t n,
                             const void* __restrict__ table, int dt, int64_t table_rows,
                             int64_t table_stride, int feat, void* __restrict__ rows_out,
                             int64_t out_stride, uint8_t* __restrict__ flags, int mode) {
  const int gl = threadIdx.x % G;
  const int64_t k = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (k >= n) return;
  const int64_t id = ids[k];
  const int64_t s = (id >= 0 && id < map_len) ? map[id] : -1;
  const bool hit = s >= 0 && s < table_rows;
  if (gl == 0) flags[k] = hit ? 1 : 0;
  if (hit) move_row(table, dt, s * table_stride, rows_out, dt, k * out_stride, feat, gl, G, mode);
}

template <int G>
__global__ void __launch_bounds__(256)
    unpermute_rows_kernel(const void* __restrict__ src, int dt, int64_t src_stride, int feat,
                          const int64_t* __restrict__ perm, const uint8_t* __restrict__ flags,
                          int64_t n, void* __restrict__ dst, int64_t dst_stride,
                          int64_t* __restrict__ hit_out, int mode) {
  const int gl = threadIdx.x % G;
  const int64_t k = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (k >= n) return;
  const int64_t p = perm[k];
  const bool on = flags == nullptr || flags[k] != 0;
  if (hit_out && gl == 0) hit_out[p] = on ? k : -1;
  if (on && dst) move_row(src, dt, k * src_stride, dst, dt, p * dst_stride, feat, gl, G, mode);
}

// how a row of `feat` elements can be moved between the two layouts
static int move_mode(const void* src, int sdt, int64_t sstride, const void* dst, int ddt,
                     int64_t dstride, int feat) {
  const int ss = dtype_size(sdt), ds = dtype_size(ddt);
  const bool s_ok = src == nullptr || (aligned16(src) && (sstride * ss) % 16 == 0);
  const bool d_ok = aligned16(dst) && (dstride * ds) % 16 == 0;
  if (!s_ok || !d_ok) return 0;
  if (sdt == ddt && ((int64_t)feat * ds) % 16 == 0) return 2;
  if (feat % 8 == 0) return 1;
  return 0;
}

static int group_width(int feat, int mode, int dt) {
  int units = mode == 2 ? feat * dtype_size(dt) / 16 : (mode == 1 ? feat / 8 : feat);
  int g = 4;
  while (g < 32 && g < units) g <<= 1;
  return g;
}

}  // namespace hc

using namespace hc;

#define HC_DISPATCH_G(G, ...)                \
  switch (G) {                               \
    case 4: { constexpr int kG = 4; __VA_ARGS__; } break;   \
    case 8: { constexpr int kG = 8; __VA_ARGS__; } break;   \
    case 16: { constexpr int kG = 16; __VA_ARGS__; } break; \
    default: { constexpr int kG = 32; __VA_ARGS__; } break; \
  }

// ---------------------------------------------------------------------------
// Staging of host rows beside a training step (hc_stage_host_rows).  The call shares the GPU with
// the step's own kernels, so it is written to need almost nothing of an SM: a few small blocks, no
// shared memory, no polling.  A batch is seen as a list of 16-byte units (unit u belongs to row
// u / units_per_row); consecutive lanes take consecutive units, every thread issues kStageUnroll
// independent 16-byte loads before it stores the first, and a warp that waits for the host link
// is simply stalled on its loads.  The grid is deliberately small: measured inside a training
// step of 0.8 ms, 16 blocks (about 0.6 ms alone for 20 K rows of 256 B, 9 GB/s) leave the step's
// own kernels undisturbed, while 64 or 148 blocks (0.43 ms alone) slow them down by as much as
// the call takes; the more read requests to host memory are outstanding, the more the step's
// own memory traffic waits behind them.
// ---------------------------------------------------------------------------
namespace hc {

constexpr int kStageThreads = 128;
constexpr int kStageUnroll = 8;

__global__ void __launch_bounds__(kStageThreads)
    stage_rows_kernel(const LoadArgs a, const int units_per_row, const int64_t units) {
  const int es = a.x_dtype == HC_F16 ? 2 : 4;
  const int64_t tile = (int64_t)kStageThreads * kStageUnroll;
  unsigned long long n_rows = 0, n_skipped = 0;
  for (int64_t base = (int64_t)blockIdx.x * tile; base < units; base += (int64_t)gridDim.x * tile) {
    uint4 v[kStageUnroll];
    bool take[kStageUnroll];
#pragma unroll
    for (int j = 0; j < kStageUnroll; ++j) {
      const int64_t u = base + (int64_t)j * kStageThreads + threadIdx.x;
      take[j] = false;
      if (u < units) {
        const int64_t i = u / units_per_row;
        const int off = (int)(u - i * units_per_row);
        const bool cached = a.sub2feat != nullptr && a.sub2feat[i] != -1;
        const bool wanted = a.used == nullptr || a.used[i] != 0;
        const int64_t g = a.sub_to_full[i];
        take[j] = wanted && !cached && g >= 0 && g < a.host_rows;
        if (take[j])
          v[j] = ldg16(reinterpret_cast<const char*>(a.host_table) + g * a.host_stride * es + 16 * off);
        if (off == 0) {
          a.load_mask_out[i] = take[j] ? 1 : 0;
          n_rows += take[j];
          n_skipped += wanted && cached;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kStageUnroll; ++j) {
      if (take[j]) {
        const int64_t u = base + (int64_t)j * kStageThreads + threadIdx.x;
        reinterpret_cast<uint4*>(a.x)[u] = v[j];
      }
    }
  }
  if (a.stats) {
    n_rows = __reduce_add_sync(kFull, (unsigned)n_rows);
    n_skipped = __reduce_add_sync(kFull, (unsigned)n_skipped);
    if ((threadIdx.x & 31) == 0) {
      if (n_rows) atomicAdd(a.stats, n_rows);
      if (n_skipped) atomicAdd(a.stats + 1, n_skipped);
    }
  }
}

}  // namespace hc

extern "C" int hc_map_lookup(const int64_t* map, int64_t map_len, const int64_t* ids, int64_t n,
                             int64_t offset, int64_t force_miss_below, int64_t* out, void* stream) {
  HC_REQUIRE(n >= 0 && map_len >= 0, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(map && ids && out, HC_ERR_NULL);
  const int64_t blocks = ceil_div(n, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  map_lookup_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      map, map_len, ids, n, offset, force_miss_below, out);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_gather_rows(const void* table, int32_t table_dtype, int64_t table_rows,
                              int64_t table_stride, int32_t feat, const int64_t* rows, int64_t n,
                              int32_t zero_missing, void* out, int32_t out_dtype,
                              int64_t out_stride, void* stream) {
  HC_REQUIRE(n >= 0 && feat > 0 && table_rows >= 0, HC_ERR_SIZE);
  HC_REQUIRE(dtype_size(table_dtype) && dtype_size(out_dtype), HC_ERR_DTYPE);
  if (n == 0) return 0;
  HC_REQUIRE(rows && out && (table || table_rows == 0), HC_ERR_NULL);
  if (table_stride == 0) table_stride = feat;
  if (out_stride == 0) out_stride = feat;
  HC_REQUIRE(table_stride >= feat && out_stride >= feat, HC_ERR_SIZE);
  const int mode = move_mode(table, table_dtype, table_stride, out, out_dtype, out_stride, feat);
  const int G = group_width(feat, mode, out_dtype);
  const int64_t blocks = ceil_div(n * G, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  HC_DISPATCH_G(G, gather_rows_kernel<kG><<<(unsigned)blocks, 256, 0, st>>>(
                       table, table_dtype, table_rows, table_stride, feat, rows, n, zero_missing,
                       out, out_dtype, out_stride, mode));
  HC_LAUNCH_OK();
  return 0;
}

static int load_rows_impl(const void* host_table, int32_t host_dtype, int64_t host_rows,
                          int64_t host_stride, const void* feat_cache, int32_t cache_dtype,
                          int64_t cache_rows, int64_t cache_stride, int32_t feat,
                          const int64_t* sub_to_full, const int64_t* sub2feat,
                          const uint8_t* used, int64_t n, void* x, int32_t x_dtype,
                          int64_t x_stride, uint8_t* load_mask_out, int64_t* stats,
                          const void* staged_rows, const uint8_t* staged_mask, int sparse_out,
                          void* stream) {
  HC_REQUIRE(n >= 0 && feat > 0 && host_rows >= 0 && cache_rows >= 0, HC_ERR_SIZE);
  HC_REQUIRE(dtype_size(x_dtype) != 0, HC_ERR_DTYPE);
  if (n == 0) return 0;
  HC_REQUIRE(sub_to_full && x, HC_ERR_NULL);
  HC_REQUIRE(host_table != nullptr || host_rows == 0, HC_ERR_NULL);
  if (host_table) HC_REQUIRE(dtype_size(host_dtype) != 0, HC_ERR_DTYPE);
  if (sub2feat) {
    HC_REQUIRE(feat_cache != nullptr || cache_rows == 0, HC_ERR_NULL);
    if (feat_cache) HC_REQUIRE(dtype_size(cache_dtype) != 0, HC_ERR_DTYPE);
  }
  if (host_stride == 0) host_stride = feat;
  if (cache_stride == 0) cache_stride = feat;
  if (x_stride == 0) x_stride = feat;
  HC_REQUIRE(host_stride >= feat && cache_stride >= feat && x_stride >= feat, HC_ERR_SIZE);
  LoadArgs a{};
  a.host_table = host_table; a.host_dtype = host_table ? host_dtype : x_dtype;
  a.host_rows = host_table ? host_rows : 0; a.host_stride = host_stride;
  a.feat_cache = feat_cache; a.cache_dtype = feat_cache ? cache_dtype : x_dtype;
  a.cache_rows = feat_cache ? cache_rows : 0; a.cache_stride = cache_stride;
  a.feat = feat; a.sub_to_full = sub_to_full; a.sub2feat = sub2feat; a.used = used; a.n = n;
  a.x = x; a.x_dtype = x_dtype; a.x_stride = x_stride; a.load_mask_out = load_mask_out;
  a.stats = reinterpret_cast<unsigned long long*>(stats);
  a.zero_mode = move_mode(nullptr, x_dtype, 0, x, x_dtype, x_stride, feat);
  a.host_mode = host_table ? move_mode(host_table, a.host_dtype, host_stride, x, x_dtype, x_stride, feat) : a.zero_mode;
  a.cache_mode = feat_cache ? move_mode(feat_cache, a.cache_dtype, cache_stride, x, x_dtype, x_stride, feat) : a.zero_mode;
  a.staged_rows = staged_mask ? staged_rows : nullptr;
  a.staged_mask = staged_mask;
  a.sparse_out = sparse_out;
  a.staged_mode = staged_mask ? move_mode(staged_rows, x_dtype, feat, x, x_dtype, x_stride, feat) : a.zero_mode;
  int worst = a.zero_mode < a.host_mode ? a.zero_mode : a.host_mode;
  if (a.cache_mode < worst) worst = a.cache_mode;
  if (a.staged_mode < worst) worst = a.staged_mode;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int row_bytes = feat * dtype_size(x_dtype);
  if (sparse_out && a.host_mode == 2 && x_stride == feat && load_mask_out != nullptr) {
    const int upr = row_bytes / 16;
    const int64_t units = n * upr;
    int64_t blocks = ceil_div(units, (int64_t)kStageThreads * kStageUnroll);
    if (blocks > sparse_out) blocks = sparse_out;
    stage_rows_kernel<<<(unsigned)blocks, kStageThreads, 0, st>>>(a, upr, units);
    HC_LAUNCH_OK();
    return 0;
  }
  // With rows staged ahead nearly every source is device memory.  The bulk-copy pipeline is built to
  // keep many long host reads in flight and took 76 us for a batch's 47 K rows even when all of them
  // were in HBM; plain 16-byte loads by a lane group per row are the better form there (measured in
  // the training step: 1 247 -> 1 276 iterations/s).
  if (worst == 2 && x_stride == feat && row_bytes <= 512 && n >= kBulkTile && staged_mask == nullptr) {
    const int64_t tiles = ceil_div(n, kBulkTile);
    const size_t smem = (size_t)kBulkWarps * 2 * kBulkTile * row_bytes;
    int64_t blocks = ceil_div(tiles, kBulkWarps);
    const int64_t cap = 148 * 8;
    if (blocks > cap) blocks = cap;
    // raised once per device (not a stream operation, so keep it out of stream captures)
    static bool smem_raised[64] = {};
    int devno = 0;
    HC_CUDA(cudaGetDevice(&devno));
    if (smem > 48 * 1024 && devno >= 0 && devno < 64 && !smem_raised[devno]) {
      HC_CUDA(cudaFuncSetAttribute(load_rows_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)((size_t)kBulkWarps * 2 * kBulkTile * 512)));
      smem_raised[devno] = true;
    }
    load_rows_bulk_kernel<<<(unsigned)blocks, kBulkWarps * 32, smem, st>>>(a, row_bytes, tiles);
    HC_LAUNCH_OK();
    return 0;
  }
  const int G = group_width(feat, worst, x_dtype);
  const int64_t blocks = ceil_div(n * G, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  HC_DISPATCH_G(G, load_rows_kernel<kG><<<(unsigned)blocks, 256, 0, st>>>(a));
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_load_rows(const void* host_table, int32_t host_dtype, int64_t host_rows,
                            int64_t host_stride, const void* feat_cache, int32_t cache_dtype,
                            int64_t cache_rows, int64_t cache_stride, int32_t feat,
                            const int64_t* sub_to_full, const int64_t* sub2feat,
                            const uint8_t* used, int64_t n, void* x, int32_t x_dtype,
                            int64_t x_stride, uint8_t* load_mask_out, int64_t* stats,
                            void* stream) {
  return load_rows_impl(host_table, host_dtype, host_rows, host_stride, feat_cache, cache_dtype, cache_rows,
                        cache_stride, feat, sub_to_full, sub2feat, used, n, x, x_dtype, x_stride,
                        load_mask_out, stats, nullptr, nullptr, 0, stream);
}

extern "C" int hc_load_rows_staged(const void* host_table, int32_t host_dtype, int64_t host_rows,
                                   int64_t host_stride, const void* feat_cache, int32_t cache_dtype,
                                   int64_t cache_rows, int64_t cache_stride, int32_t feat,
                                   const int64_t* sub_to_full, const int64_t* sub2feat,
                                   const uint8_t* used, int64_t n, void* x, int32_t x_dtype,
                                   int64_t x_stride, uint8_t* load_mask_out, int64_t* stats,
                                   const void* staged_rows, const uint8_t* staged_mask,
                                   void* stream) {
  HC_REQUIRE(staged_rows && staged_mask, HC_ERR_NULL);
  return load_rows_impl(host_table, host_dtype, host_rows, host_stride, feat_cache, cache_dtype, cache_rows,
                        cache_stride, feat, sub_to_full, sub2feat, used, n, x, x_dtype, x_stride,
                        load_mask_out, stats, staged_rows, staged_mask, 0, stream);
}

extern "C" int hc_stage_host_rows(const void* host_table, int32_t host_dtype, int64_t host_rows,
                                  int64_t host_stride, int32_t feat, const int64_t* ids,
                                  const int64_t* sub2feat, const uint8_t* consider, int64_t n,
                                  void* staged_rows, uint8_t* staged_mask, int64_t* stats,
                                  int32_t max_blocks, void* stream) {
  HC_REQUIRE(n == 0 || (staged_rows && staged_mask), HC_ERR_NULL);
  HC_REQUIRE(max_blocks >= 0 && max_blocks <= 65535, HC_ERR_SIZE);
  return load_rows_impl(host_table, host_dtype, host_rows, host_stride, nullptr, host_dtype, 0, 0, feat, ids,
                        sub2feat, consider, n, staged_rows, host_dtype, feat, staged_mask, stats, nullptr,
                        nullptr, max_blocks > 0 ? max_blocks : kStageBlocks, stream);
}

extern "C" int hc_owner_lookup(const int64_t* map, int64_t map_len, const int64_t* ids, int64_t n,
                               const void* table, int32_t dtype, int64_t table_rows,
                               int64_t table_stride, int32_t feat, void* rows_out,
                               int64_t out_stride, uint8_t* flags, void* stream) {
  HC_REQUIRE(n >= 0 && map_len >= 0 && table_rows >= 0, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(map && ids && flags, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows_out == nullptr) {
    const int64_t blocks = ceil_div(n, 256);
    HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
    owner_lookup_flags_kernel<<<(unsigned)blocks, 256, 0, st>>>(map, map_len, ids, n, nullptr, flags);
    HC_LAUNCH_OK();
    return 0;
  }
  HC_REQUIRE(feat > 0, HC_ERR_SIZE);
  HC_REQUIRE(dtype_size(dtype) != 0, HC_ERR_DTYPE);
  HC_REQUIRE(table != nullptr || table_rows == 0, HC_ERR_NULL);
  if (table_stride == 0) table_stride = feat;
  if (out_stride == 0) out_stride = feat;
  HC_REQUIRE(table_stride >= feat && out_stride >= feat, HC_ERR_SIZE);
  const int mode = move_mode(table, dtype, table_stride, rows_out, dtype, out_stride, feat);
  const int G = group_width(feat, mode, dtype);
  const int64_t blocks = ceil_div(n * G, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  HC_DISPATCH_G(G, owner_lookup_rows_kernel<kG><<<(unsigned)blocks, 256, 0, st>>>(
                       map, map_len, ids, n, table, dtype, table_rows, table_stride, feat,
                       rows_out, out_stride, flags, mode));
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_unpermute_rows(const void* src, int32_t dtype, int64_t src_stride, int32_t feat,
                                 const int64_t* perm, const uint8_t* flags, int64_t n, void* dst,
                                 int64_t dst_stride, int64_t* hit_out, void* stream) {
  HC_REQUIRE(n >= 0, HC_ERR_SIZE);
  if (n == 0) return 0;
  HC_REQUIRE(perm != nullptr, HC_ERR_NULL);
  HC_REQUIRE(dst != nullptr || hit_out != nullptr, HC_ERR_NULL);
  int mode = 0, G = 4;
  if (dst) {
    HC_REQUIRE(src != nullptr, HC_ERR_NULL);
    HC_REQUIRE(feat > 0, HC_ERR_SIZE);
    HC_REQUIRE(dtype_size(dtype) != 0, HC_ERR_DTYPE);
    if (src_stride == 0) src_stride = feat;
    if (dst_stride == 0) dst_stride = feat;
    HC_REQUIRE(src_stride >= feat && dst_stride >= feat, HC_ERR_SIZE);
    mode = move_mode(src, dtype, src_stride, dst, dtype, dst_stride, feat);
    G = group_width(feat, mode, dtype);
  }
  const int64_t blocks = ceil_div(n * G, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  HC_DISPATCH_G(G, unpermute_rows_kernel<kG><<<(unsigned)blocks, 256, 0, st>>>(
                       src, dtype, src_stride, feat, perm, flags, n, dst, dst_stride, hit_out,
                       mode));
  HC_LAUNCH_OK();
  return 0;
}
