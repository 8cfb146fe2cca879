// History exchange over peer memory (NVLink / NVSwitch loads), one process per GPU.
//
// Every rank keeps its shard of the node-partitioned embedding history (id -> slot map and
// the rows) and a small "published candidates" area in one device allocation that the other
// ranks of the box map into their address space (CUDA IPC).  With that,
//   * a lookup is ONE kernel on the asking rank: it hashes each id to its owner, reads the
//     owner's map entry and, on a hit, copies the owner's row straight into local memory;
//   * an admission is a local publish (ids + rows of the candidates), and after a fence the
//     owner PULLS the candidates it owns from every rank's published area, in (rank, row)
//     order, into a local candidate list that the ordinary admission kernels consume.
// No kernel here waits for another GPU: ordering between ranks comes from the collectives
// the training step already contains (the caller's fences).  All peer accesses are plain
// loads; nothing is written into another GPU's memory.
//
// The reference's counterpart is the p2psend / all2all machinery of src/cpp/src/comm.cu:5-29
// and hiscache/comm.py:8-151, which its only caller never completes
// (hiscache/multi_gpu_history_trainer.py:74-79).
#include <string.h>

#include "common.cuh"

namespace hc {

constexpr int kMaxPeers = HC_MAX_PEERS;
constexpr int kPullBlock = 256;

struct PeerPtrs {
  const void* p[kMaxPeers];
};

__device__ __forceinline__ const void* pick(const PeerPtrs& s, int r) {
  // a select chain keeps the pointer table in registers / constant bank (no local-memory copy)
  const void* out = s.p[0];
#pragma unroll
  for (int k = 1; k < kMaxPeers; ++k) out = (r == k) ? s.p[k] : out;
  return out;
}

template <int G>
__global__ void __launch_bounds__(256)
    peer_lookup_kernel(const PeerPtrs maps, const PeerPtrs bufs, const int world,
                       const int64_t map_len, const int64_t table_rows,
                       const int64_t table_stride_bytes, const int row_bytes,
                       const int64_t* __restrict__ ids, const int64_t n, char* __restrict__ rows_out,
                       const int64_t out_stride_bytes, int64_t* __restrict__ hit_map) {
  const int gl = threadIdx.x % G;
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (i >= n) return;
  const int64_t id = ids[i];
  int64_t slot = -1;
  int owner = 0;
  if (id >= 0 && id < map_len) {
    owner = (int)(mix64((uint64_t)id) % (uint64_t)world);
    slot = __ldg(reinterpret_cast<const int64_t*>(pick(maps, owner)) + id);
  }
  const bool hit = slot >= 0 && slot < table_rows;
  if (hit) {
    const char* src = reinterpret_cast<const char*>(pick(bufs, owner)) + slot * table_stride_bytes;
    char* dst = rows_out + i * out_stride_bytes;
    const int nvec = row_bytes >> 4;
    for (int v = gl; v < nvec; v += G) reinterpret_cast<uint4*>(dst)[v] = ldg16(src + 16 * v);
  }
  if (gl == 0) hit_map[i] = hit ? i : -1;
}

template <int G>
__global__ void __launch_bounds__(256)
    peer_publish_kernel(const int64_t* __restrict__ ids, const uint8_t* __restrict__ mask,
                        const float* __restrict__ score, const float* __restrict__ thres,
                        const int64_t* __restrict__ present, const int64_t n,
                        const float* __restrict__ rows, const int64_t row_stride, const int feat,
                        const int vec_ok, int64_t* __restrict__ pub_ids, float* __restrict__ pub_rows,
                        int64_t* __restrict__ pub_n) {
  if (blockIdx.x == 0 && threadIdx.x == 0) pub_n[0] = n;
  const int gl = threadIdx.x % G;
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (i >= n) return;
  bool take = mask == nullptr || mask[i] != 0;
  if (take && score != nullptr) take = score[i] < thres[0];   // the admission test
  if (take && present != nullptr) take = present[i] == -1;    // rows served from history are not re-admitted
  const int64_t id = take ? ids[i] : -1;
  if (gl == 0) pub_ids[i] = id;
  if (id < 0) return;
  const float* src = rows + i * row_stride;
  float* dst = pub_rows + i * (int64_t)feat;
  if (vec_ok) {
    for (int v = gl; v < (feat >> 2); v += G)
      reinterpret_cast<uint4*>(dst)[v] = ldg16(reinterpret_cast<const char*>(src) + 16 * v);
  } else {
    for (int e = gl; e < feat; e += G) dst[e] = src[e];
  }
}

__device__ __forceinline__ bool pull_flag(const PeerPtrs& pub_ids, const PeerPtrs& pub_n, int p,
                                          int64_t r, int world, int me, int64_t max_ids,
                                          int64_t* id_out) {
  int64_t n_p = __ldg(reinterpret_cast<const int64_t*>(pick(pub_n, p)));
  n_p = n_p < 0 ? 0 : (n_p > max_ids ? max_ids : n_p);
  if (r >= n_p) return false;
  const int64_t id = __ldg(reinterpret_cast<const int64_t*>(pick(pub_ids, p)) + r);
  *id_out = id;
  return id >= 0 && (int)(mix64((uint64_t)id) % (uint64_t)world) == me;
}

// counts[p * chunks + c] = candidates of rank p's chunk c that this rank owns
__global__ void __launch_bounds__(kPullBlock)
    pull_count_kernel(const PeerPtrs pub_ids, const PeerPtrs pub_n, const int world, const int me,
                      const int64_t max_ids, int64_t* __restrict__ counts) {
  const int p = blockIdx.y;
  const int64_t r = (int64_t)blockIdx.x * kPullBlock + threadIdx.x;
  int64_t id;
  const bool f = pull_flag(pub_ids, pub_n, p, r, world, me, max_ids, &id);
  const int c = __syncthreads_count(f);
  if (threadIdx.x == 0) counts[(int64_t)p * gridDim.x + blockIdx.x] = c;
}

// exclusive scan of counts[0..m) in place, total in counts[m]; pads got_ids with -1 from the
// total up to cap and adds the ids that did not fit to *overflow
__global__ void __launch_bounds__(1024)
    pull_scan_kernel(int64_t* __restrict__ counts, const int64_t m, int64_t* __restrict__ got_ids,
                     const int64_t cap, int64_t* __restrict__ overflow) {
  __shared__ int64_t warp_sum[32];
  __shared__ int64_t total_s;
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  const int64_t per = ceil_div(m, 1024);
  const int64_t b = (int64_t)t * per, e = b + per < m ? b + per : m;
  int64_t s = 0;
  for (int64_t k = b; k < e; ++k) s += counts[k];
  int64_t inc = s;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int64_t o = __shfl_up_sync(kFull, (long long)inc, off);
    if (lane >= off) inc += o;
  }
  if (lane == 31) warp_sum[w] = inc;
  __syncthreads();
  if (w == 0) {
    int64_t v = warp_sum[lane], iv = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int64_t o = __shfl_up_sync(kFull, (long long)iv, off);
      if (lane >= off) iv += o;
    }
    warp_sum[lane] = iv - v;
    if (lane == 31) total_s = iv;
  }
  __syncthreads();
  int64_t run = warp_sum[w] + inc - s;
  for (int64_t k = b; k < e; ++k) {
    const int64_t c = counts[k];
    counts[k] = run;
    run += c;
  }
  const int64_t total = total_s;
  if (t == 0) {
    counts[m] = total;
    if (total > cap && overflow) atomicAdd(reinterpret_cast<unsigned long long*>(overflow),
                                           (unsigned long long)(total - cap));
  }
  for (int64_t k = (total < cap ? total : cap) + t; k < cap; k += 1024) got_ids[k] = -1;
}

__global__ void __launch_bounds__(kPullBlock)
    pull_place_kernel(const PeerPtrs pub_ids, const PeerPtrs pub_rows, const PeerPtrs pub_n,
                      const int world, const int me, const int64_t max_ids, const int feat,
                      const int vec_ok, const int64_t* __restrict__ offsets,
                      int64_t* __restrict__ got_ids, float* __restrict__ got_rows,
                      const int64_t cap) {
  __shared__ int warp_cnt[kPullBlock / 32];
  __shared__ int64_t s_k[kPullBlock];
  __shared__ int64_t s_r[kPullBlock];
  const int p = blockIdx.y, t = threadIdx.x, lane = t & 31, w = t >> 5;
  const int64_t r = (int64_t)blockIdx.x * kPullBlock + t;
  int64_t id = -1;
  const bool f = pull_flag(pub_ids, pub_n, p, r, world, me, max_ids, &id);
  const unsigned bal = __ballot_sync(kFull, f);
  if (lane == 0) warp_cnt[w] = __popc(bal);
  __syncthreads();
  int before = 0, cnt = 0;
#pragma unroll
  for (int k = 0; k < kPullBlock / 32; ++k) {
    before += k < w ? warp_cnt[k] : 0;
    cnt += warp_cnt[k];
  }
  if (f) {
    const int local = before + __popc(bal & ((1u << lane) - 1u));
    const int64_t k = offsets[(int64_t)p * gridDim.x + blockIdx.x] + local;
    s_k[local] = k;
    s_r[local] = r;
    if (k < cap) got_ids[k] = id;
  }
  __syncthreads();
  const float* src_rows = reinterpret_cast<const float*>(pick(pub_rows, p));
  if (vec_ok) {
    const int nvec = feat >> 2;
    for (int x = t; x < cnt * nvec; x += kPullBlock) {
      const int j = x / nvec, v = x - j * nvec;
      const int64_t k = s_k[j];
      if (k < cap)
        reinterpret_cast<uint4*>(got_rows + k * (int64_t)feat)[v] =
            ldg16(reinterpret_cast<const char*>(src_rows + s_r[j] * (int64_t)feat) + 16 * v);
    }
  } else {
    for (int x = t; x < cnt * feat; x += kPullBlock) {
      const int j = x / feat, e = x - j * feat;
      const int64_t k = s_k[j];
      if (k < cap) got_rows[k * (int64_t)feat + e] = __ldg(src_rows + s_r[j] * (int64_t)feat + e);
    }
  }
}

static int fill_ptrs(PeerPtrs* out, const void* const* in, int world) {
  for (int k = 0; k < kMaxPeers; ++k) out->p[k] = nullptr;
  for (int k = 0; k < world; ++k) {
    if (in[k] == nullptr) return -HC_ERR_NULL;
    out->p[k] = in[k];
  }
  return 0;
}

static int lane_group(int nvec) { return nvec >= 32 ? 32 : (nvec >= 16 ? 16 : (nvec >= 8 ? 8 : 4)); }

}  // namespace hc

using namespace hc;

#define HC_PEER_DISPATCH_G(G, ...)                           \
  switch (G) {                                               \
    case 4: { constexpr int kG = 4; __VA_ARGS__; } break;    \
    case 8: { constexpr int kG = 8; __VA_ARGS__; } break;    \
    case 16: { constexpr int kG = 16; __VA_ARGS__; } break;  \
    default: { constexpr int kG = 32; __VA_ARGS__; } break;  \
  }

static_assert(sizeof(cudaIpcMemHandle_t) == HC_PEER_HANDLE_BYTES, "handle size");

extern "C" int hc_peer_alloc(int64_t bytes, void** ptr) {
  HC_REQUIRE(ptr != nullptr, HC_ERR_NULL);
  HC_REQUIRE(bytes > 0, HC_ERR_SIZE);
  void* p = nullptr;
  HC_CUDA(cudaMalloc(&p, (size_t)bytes));
  cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
  // the fill runs on the legacy default stream; wait for it here, once, so that a caller
  // working on a non-blocking stream never sees a region that is still being cleared
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(p);
    return (int)e;
  }
  *ptr = p;
  return 0;
}

extern "C" int hc_peer_free(void* ptr) {
  if (ptr) HC_CUDA(cudaFree(ptr));
  return 0;
}

extern "C" int hc_peer_export(const void* ptr, void* handle) {
  HC_REQUIRE(ptr && handle, HC_ERR_NULL);
  cudaIpcMemHandle_t h;
  HC_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  memcpy(handle, &h, sizeof(h));
  return 0;
}

extern "C" int hc_peer_open(const void* handle, void** ptr) {
  HC_REQUIRE(ptr && handle, HC_ERR_NULL);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  HC_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return 0;
}

extern "C" int hc_peer_close(void* ptr) {
  if (ptr) HC_CUDA(cudaIpcCloseMemHandle(ptr));
  return 0;
}

extern "C" int hc_peer_lookup(const void* const* peer_maps, const void* const* peer_tables,
                              int32_t world, int64_t map_len, int32_t dtype, int64_t table_rows,
                              int64_t table_stride, int32_t feat, const int64_t* ids, int64_t n,
                              void* rows_out, int64_t out_stride, int64_t* hit_map, void* stream) {
  HC_REQUIRE(world >= 1 && world <= kMaxPeers && n >= 0 && map_len >= 0 && table_rows >= 0 && feat > 0,
             HC_ERR_SIZE);
  const int es = dtype_size(dtype);
  HC_REQUIRE(es != 0, HC_ERR_DTYPE);
  if (n == 0) return 0;
  HC_REQUIRE(peer_maps && peer_tables && ids && rows_out && hit_map, HC_ERR_NULL);
  if (table_stride == 0) table_stride = feat;
  if (out_stride == 0) out_stride = feat;
  HC_REQUIRE(table_stride >= feat && out_stride >= feat, HC_ERR_SIZE);
  const int row_bytes = feat * es;
  // rows move as 16-byte vectors
  HC_REQUIRE(row_bytes % 16 == 0 && (table_stride * es) % 16 == 0 && (out_stride * es) % 16 == 0,
             HC_ERR_UNSUPPORTED);
  HC_REQUIRE(aligned16(rows_out), HC_ERR_ALIGN);
  PeerPtrs maps, bufs;
  int rc = fill_ptrs(&maps, peer_maps, world);
  if (rc) return rc;
  rc = fill_ptrs(&bufs, peer_tables, world);
  if (rc) return rc;
  for (int k = 0; k < world; ++k) HC_REQUIRE(aligned16(bufs.p[k]) && aligned_to(maps.p[k], 8), HC_ERR_ALIGN);
  const int G = lane_group(row_bytes / 16);
  const int64_t blocks = ceil_div(n * G, 256);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  HC_PEER_DISPATCH_G(G, peer_lookup_kernel<kG><<<(unsigned)blocks, 256, 0, st>>>(
                            maps, bufs, world, map_len, table_rows, table_stride * es, row_bytes, ids, n,
                            reinterpret_cast<char*>(rows_out), out_stride * es, hit_map));
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_peer_publish(const int64_t* ids, const uint8_t* mask, const float* score,
                               const float* thres, const int64_t* present, int64_t n,
                               const float* rows, int64_t row_stride, int32_t feat, int64_t* pub_ids,
                               float* pub_rows, int64_t* pub_n, int64_t max_ids, void* stream) {
  HC_REQUIRE(n >= 0 && feat > 0 && max_ids >= 0, HC_ERR_SIZE);
  HC_REQUIRE(n <= max_ids, HC_ERR_LIMIT);
  HC_REQUIRE(pub_ids && pub_rows && pub_n, HC_ERR_NULL);
  HC_REQUIRE(n == 0 || (ids && rows), HC_ERR_NULL);
  HC_REQUIRE(score == nullptr || thres != nullptr, HC_ERR_NULL);
  if (row_stride == 0) row_stride = feat;
  HC_REQUIRE(row_stride >= feat, HC_ERR_SIZE);
  const int vec_ok = (feat % 4 == 0) && (row_stride % 4 == 0) && aligned16(rows) && aligned16(pub_rows);
  const int G = lane_group(vec_ok ? feat / 4 : feat);
  const int64_t blocks = n > 0 ? ceil_div(n * G, 256) : 1;
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  HC_PEER_DISPATCH_G(G, peer_publish_kernel<kG><<<(unsigned)blocks, 256, 0, st>>>(
                            ids, mask, score, thres, present, n, rows, row_stride, feat, vec_ok, pub_ids,
                            pub_rows, pub_n));
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int64_t hc_peer_pull_scratch_bytes(int32_t world, int64_t max_ids) {
  const int64_t chunks = max_ids > 0 ? ceil_div(max_ids, kPullBlock) : 1;
  return ((world > 0 ? world : 1) * chunks + 1) * (int64_t)sizeof(int64_t);
}

extern "C" int hc_peer_pull(const void* const* peer_pub_ids, const void* const* peer_pub_rows,
                            const void* const* peer_pub_n, int32_t world, int32_t me,
                            int64_t max_ids, int32_t feat, int64_t* got_ids, float* got_rows,
                            int64_t cap, int64_t* overflow, void* scratch, void* stream) {
  HC_REQUIRE(world >= 1 && world <= kMaxPeers && me >= 0 && me < world && max_ids > 0 && feat > 0 &&
                 cap > 0,
             HC_ERR_SIZE);
  HC_REQUIRE(peer_pub_ids && peer_pub_rows && peer_pub_n && got_ids && got_rows && scratch, HC_ERR_NULL);
  PeerPtrs pid, prow, pn;
  int rc = fill_ptrs(&pid, peer_pub_ids, world);
  if (rc) return rc;
  rc = fill_ptrs(&prow, peer_pub_rows, world);
  if (rc) return rc;
  rc = fill_ptrs(&pn, peer_pub_n, world);
  if (rc) return rc;
  int vec_ok = (feat % 4 == 0) && aligned16(got_rows);
  for (int k = 0; k < world; ++k) {
    HC_REQUIRE(aligned_to(pid.p[k], 8) && aligned_to(pn.p[k], 8) && aligned_to(prow.p[k], 4), HC_ERR_ALIGN);
    vec_ok = vec_ok && aligned16(prow.p[k]);
  }
  const int64_t chunks = ceil_div(max_ids, kPullBlock);
  HC_REQUIRE(chunks <= 0x7fffffffLL, HC_ERR_SIZE);
  int64_t* counts = reinterpret_cast<int64_t*>(scratch);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)chunks, (unsigned)world);
  pull_count_kernel<<<grid, kPullBlock, 0, st>>>(pid, pn, world, me, max_ids, counts);
  HC_LAUNCH_OK();
  pull_scan_kernel<<<1, 1024, 0, st>>>(counts, (int64_t)world * chunks, got_ids, cap, overflow);
  HC_LAUNCH_OK();
  pull_place_kernel<<<grid, kPullBlock, 0, st>>>(pid, prow, pn, world, me, max_ids, feat, vec_ok, counts,
                                                got_ids, got_rows, cap);
  HC_LAUNCH_OK();
  return 0;
}

// ---------------------------------------------------------------------------
// The whole owner-side admission of a step as one call: eviction of stale entries, pull of
// the published candidates, last-copy-wins, skip of ids already held, ring admission, check-in
// stamp and (optionally) the advance of the device-side iteration counter.  The same entry
// points a host would call one by one, launched back to back on one stream.
// ---------------------------------------------------------------------------
namespace hc {
static __device__ float g_zero_thres = 0.f;   // threshold 0 = "admit every candidate" for the ring admission
static void* g_zero_thres_addr[64];

static int zero_thres_ptr(const float** out) {
  int dev = -1;
  HC_CUDA(cudaGetDevice(&dev));
  HC_REQUIRE(dev >= 0 && dev < 64, HC_ERR_SIZE);
  void* p = __atomic_load_n(&g_zero_thres_addr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    HC_CUDA(cudaGetSymbolAddress(&p, g_zero_thres));
    HC_REQUIRE(p != nullptr, HC_ERR_NULL);
    __atomic_store_n(&g_zero_thres_addr[dev], p, __ATOMIC_RELEASE);
  }
  *out = reinterpret_cast<const float*>(p);
  return 0;
}

__global__ void advance_iter_kernel(int64_t* iter_dev) { iter_dev[0] += 1; }

constexpr int64_t kCheckinMarker = 1ll << 60;  // a check-in time no iteration takes
inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }
}  // namespace hc

extern "C" int64_t hc_peer_admit_scratch_bytes(int32_t world, int64_t max_ids, int64_t cap) {
  if (cap < 0) cap = 0;
  return align256(hc_peer_pull_scratch_bytes(world, max_ids)) + align256(hc_admit_scratch_bytes(cap)) +
         align256(cap) + align256(cap * 8);
}

extern "C" int hc_peer_admit(const hc_shard* sh, const void* const* peer_pub_ids,
                             const void* const* peer_pub_rows, const void* const* peer_pub_n,
                             int32_t world, int32_t me, int64_t max_ids, int64_t* got_ids,
                             float* got_rows, int64_t cap, int64_t* overflow, int32_t evict,
                             int32_t advance_iter, void* scratch, void* stream) {
  HC_REQUIRE(sh != nullptr && scratch != nullptr, HC_ERR_NULL);
  HC_REQUIRE(sh->struct_size == sizeof(hc_shard), HC_ERR_STRUCT);
  HC_REQUIRE(sh->full_to_slot && sh->slot_to_full && sh->checkin && sh->table && sh->header &&
                 sh->iter_dev && sh->claim,
             HC_ERR_NULL);
  HC_REQUIRE(cap > 0 && sh->capacity > 0 && sh->feat > 0, HC_ERR_SIZE);
  const float* zero = nullptr;
  int rc = zero_thres_ptr(&zero);
  if (rc) return rc;
  char* sc = reinterpret_cast<char*>(scratch);
  void* pull_sc = sc;
  sc += align256(hc_peer_pull_scratch_bytes(world, max_ids));
  void* admit_sc = sc;
  sc += align256(hc_admit_scratch_bytes(cap));
  uint8_t* winners = reinterpret_cast<uint8_t*>(sc);
  sc += align256(cap);
  int64_t* present = reinterpret_cast<int64_t*>(sc);
  if (evict && sh->staleness > 0) {
    rc = hc_evict_stale_dev(sh->checkin, sh->slot_to_full, sh->full_to_slot, sh->capacity, sh->iter_dev,
                            sh->staleness, stream);
    if (rc) return rc;
  }
  rc = hc_peer_pull(peer_pub_ids, peer_pub_rows, peer_pub_n, world, me, max_ids, sh->feat, got_ids,
                    got_rows, cap, overflow, pull_sc, stream);
  if (rc) return rc;
  rc = hc_last_occurrence(got_ids, cap, sh->claim, sh->map_len, winners, stream);
  if (rc) return rc;
  rc = hc_map_lookup(sh->full_to_slot, sh->map_len, got_ids, cap, 0, 0, present, stream);
  if (rc) return rc;
  // score is never read when the threshold is 0 (every candidate that won is admitted)
  rc = hc_record_history(got_rows, sh->feat, cap, sh->table, sh->dtype, sh->capacity, sh->feat, winners,
                         got_ids, present, sh->slot_to_full, sh->full_to_slot, sh->header, got_rows, zero,
                         sh->checkin, kCheckinMarker, sh->n_admitted, admit_sc, stream);
  if (rc) return rc;
  rc = hc_stamp_checkin(sh->checkin, sh->capacity, kCheckinMarker, sh->iter_dev, stream);
  if (rc) return rc;
  if (advance_iter) {
    advance_iter_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sh->iter_dev);
    HC_LAUNCH_OK();
  }
  return 0;
}
