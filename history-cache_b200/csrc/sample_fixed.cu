// A whole sampled batch in a FIXED shape, built without one device->host read.
//
// hc_sample_counts / hc_sample_picks / hc_relabel (sampler.cu) build a batch hop by hop, and the
// host reads two sizes back per hop to allocate the next arrays.  With the layer sizes fixed
// in advance (caps) nothing depends on those sizes on the host any more: every array has its
// capacity, the real counts stay on the device, rows behind them are padding (no neighbours,
// node 0, mask 0).  The whole batch is then a fixed sequence of launches, so it can run on a
// second stream behind the training step or be captured in the step's CUDA graph.
//
// Layout (the one NeighborSampler.sample_padded produces): layer k owns rows [0, caps[k]); the new
// nodes of hop h start at row caps[h-1]; ptr has caps[L-1] + 1 entries, idx edge_cap entries.
// Draws are the ones of hc_sample_picks: a function of (batch seed, frontier position, draw), the
// position counted over the REAL frontier nodes, so a batch that fits its caps is bit-identical to
// the host-driven one.  What does not fit is cut in a memory-safe way and counted: a new node beyond
// its layer's capacity is not added and the edges to it become self loops of their destination row;
// edges beyond edge_cap are dropped.
#include "common.cuh"

namespace hc {

constexpr int kAbsentF = (int)0x80000000;
constexpr int kMaxHops = 8;

struct FixedPlan {
  int num_hops;
  int fanout[kMaxHops];
  int64_t caps[kMaxHops + 1];
  int64_t edge_cap;
  int64_t* ptr;
  int64_t* idx;
  int64_t* sub_to_full;
  uint8_t* mask;
  int64_t* counters;     // [0] real nodes [1] real edges [2] new nodes cut [3] edges cut
  // scratch
  int64_t* state;        // [0] batch seed [1] edge offset [2] frontier base [3] hop edges [4] hop new nodes
  int64_t* cnt;          // [max frontier + 1] counts, then their exclusive scan
  int64_t* nbr;          // [max frontier * fanout]
  int64_t* new_nodes;    // [max frontier * fanout]
  int64_t* block_counts; // [blocks]
};

__global__ void fixed_begin_kernel(const FixedPlan p, const int64_t* __restrict__ seeds, int64_t n_seeds,
                                   int* local_map, uint64_t seed, int64_t* batch_no) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = p.caps[p.num_hops];
  if (i < total) {
    const bool s = i < n_seeds;
    p.sub_to_full[i] = s ? seeds[i] : 0;
    p.mask[i] = s ? 1 : 0;
    if (s) local_map[seeds[i]] = (int)i;
  }
  if (i == 0) {
    // the same arithmetic as the host-driven sampler: mix64(seed * 1000003 + batch number)
    p.state[0] = (int64_t)mix64(seed * 1000003ull + (uint64_t)batch_no[0]);
    batch_no[0] += 1;
    p.state[1] = 0;
    p.state[2] = 0;
    p.counters[0] = n_seeds;
    p.counters[1] = 0;
    p.counters[2] = 0;
    p.counters[3] = 0;
  }
}

__global__ void fixed_counts_kernel(const FixedPlan p, const int64_t* __restrict__ gptr, int64_t fs, int64_t nf,
                                    int fanout) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nf) return;
  int64_t c = 0;
  if (p.mask[fs + i]) {
    const int64_t v = p.sub_to_full[fs + i];
    const int64_t deg = gptr[v + 1] - gptr[v];
    c = deg < fanout ? deg : fanout;
  }
  p.cnt[i] = c;
}

// exclusive scan of cnt[0..n) in place by one block; cnt[n] = total, also kept in state[3]
__global__ void __launch_bounds__(1024) fixed_scan_kernel(const FixedPlan p, int64_t n) {
  __shared__ int64_t part[1024];
  __shared__ int64_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < n; base += 1024) {
    const int64_t b = base + threadIdx.x;
    const int64_t c = b < n ? p.cnt[b] : 0;
    part[threadIdx.x] = c;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int64_t v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
      __syncthreads();
      part[threadIdx.x] += v;
      __syncthreads();
    }
    if (b < n) p.cnt[b] = carry + part[threadIdx.x] - c;
    __syncthreads();
    if (threadIdx.x == 1023) carry += part[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    p.cnt[n] = carry;
    p.state[3] = carry;
  }
}

__global__ void fixed_picks_kernel(const FixedPlan p, const int64_t* __restrict__ gptr,
                                   const int64_t* __restrict__ gidx, int64_t fs, int64_t nf, int fanout) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t i = t / fanout;
  const int j = (int)(t % fanout);
  if (i >= nf) return;
  const int64_t o = p.cnt[i];
  if (j >= p.cnt[i + 1] - o) return;
  const int64_t v = p.sub_to_full[fs + i];
  const int64_t b = gptr[v];
  const uint64_t deg = (uint64_t)(gptr[v + 1] - b);
  const uint64_t seed = (uint64_t)p.state[0];
  const uint64_t u = mix64(seed ^ mix64((uint64_t)(p.state[2] + i) * (uint64_t)fanout + (uint64_t)j));
  p.nbr[o + j] = gidx[b + (int64_t)(u % deg)];
}

// position q claims node nbr[q] unless the node already has a local id; the lowest q wins
__global__ void fixed_claim_kernel(const FixedPlan p, int* local_map) {
  const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (q < p.state[3]) atomicMax(local_map + p.nbr[q], -(int)(q + 2));
}

__device__ __forceinline__ bool fixed_is_first(const FixedPlan& p, const int* local_map, int64_t q) {
  return q < p.state[3] && local_map[p.nbr[q]] == -(int)(q + 2);
}

__global__ void __launch_bounds__(1024)
    fixed_first_count_kernel(const FixedPlan p, const int* __restrict__ local_map) {
  const int64_t q = (int64_t)blockIdx.x * 1024 + threadIdx.x;
  const int c = __syncthreads_count(fixed_is_first(p, local_map, q));
  if (threadIdx.x == 0) p.block_counts[blockIdx.x] = c;
}

__global__ void __launch_bounds__(1024) fixed_first_scan_kernel(const FixedPlan p, int64_t nblocks) {
  __shared__ int64_t part[1024];
  __shared__ int64_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < nblocks; base += 1024) {
    const int64_t b = base + threadIdx.x;
    const int64_t c = b < nblocks ? p.block_counts[b] : 0;
    part[threadIdx.x] = c;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int64_t v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
      __syncthreads();
      part[threadIdx.x] += v;
      __syncthreads();
    }
    if (b < nblocks) p.block_counts[b] = carry + part[threadIdx.x] - c;
    __syncthreads();
    if (threadIdx.x == 1023) carry += part[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) p.state[4] = carry;
}

// new nodes in order of first occurrence; those beyond the layer's capacity are cut
__global__ void __launch_bounds__(1024)
    fixed_place_kernel(const FixedPlan p, int* local_map, int64_t row0, int64_t cap_new) {
  __shared__ int warp_sums[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t q = (int64_t)blockIdx.x * 1024 + threadIdx.x;
  const bool f = fixed_is_first(p, local_map, q);
  const unsigned bal = __ballot_sync(kFull, f);
  if (lane == 0) warp_sums[warp] = __popc(bal);
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += warp_sums[w];
  if (f) {
    const int64_t rank = p.block_counts[blockIdx.x] + before + __popc(bal & ((1u << lane) - 1u));
    const int64_t v = p.nbr[q];
    if (rank < cap_new) {
      p.sub_to_full[row0 + rank] = v;
      p.mask[row0 + rank] = 1;
      p.new_nodes[rank] = v;
    } else {
      p.new_nodes[rank] = -1 - v;     // cut: remembered so that its claim can be withdrawn
    }
  }
}

// local ids of the nodes that got a row; the claims of cut nodes are withdrawn
__global__ void fixed_assign_kernel(const FixedPlan p, int* local_map, int64_t row0, int64_t cap_new) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= p.state[4]) return;
  const int64_t v = p.new_nodes[r];
  if (v >= 0) local_map[v] = (int)(row0 + r);
}

// edges of this hop into idx (behind the edges of the earlier hops) and the rows' ptr entries
__global__ void fixed_translate_kernel(const FixedPlan p, const int* __restrict__ local_map, int64_t fs, int64_t nf,
                                       int fanout) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t i = t / fanout;
  const int j = (int)(t % fanout);
  if (i >= nf) return;
  const int64_t e_off = p.state[1];
  const int64_t o = p.cnt[i];
  if (j == 0) {
    const int64_t at = e_off + o;
    p.ptr[fs + i] = at < p.edge_cap ? at : p.edge_cap;
  }
  if (j >= p.cnt[i + 1] - o) return;
  const int64_t e = e_off + o + j;
  if (e >= p.edge_cap) {
    atomicAdd(reinterpret_cast<unsigned long long*>(p.counters + 3), 1ull);
    return;
  }
  const int loc = local_map[p.nbr[o + j]];
  // a node that was cut has no row: the edge becomes a self loop of its destination row
  p.idx[e] = loc >= 0 ? (int64_t)loc : fs + i;
}

__global__ void fixed_unclaim_kernel(const FixedPlan p, int* local_map) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= p.state[4]) return;
  const int64_t v = p.new_nodes[r];
  if (v < 0) {
    local_map[-1 - v] = kAbsentF;
    atomicAdd(reinterpret_cast<unsigned long long*>(p.counters + 2), 1ull);
  }
}

__global__ void fixed_hop_end_kernel(const FixedPlan p, int64_t cap_new, int last, int64_t ptr_end_row) {
  // advance the device-side offsets for the next hop
  const int64_t edges = p.state[3];
  int64_t kept = p.state[4] < cap_new ? p.state[4] : cap_new;
  int64_t e_off = p.state[1] + edges;
  p.state[2] += p.state[5];          // frontier base: real nodes of the frontier just expanded
  p.state[5] = kept;                 // size of the next frontier
  p.state[1] = e_off;
  p.counters[0] += kept;
  p.counters[1] = e_off < p.edge_cap ? e_off : p.edge_cap;
  if (last) p.ptr[ptr_end_row] = e_off < p.edge_cap ? e_off : p.edge_cap;
}

__global__ void fixed_finish_kernel(const FixedPlan p, int* local_map) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < p.caps[p.num_hops] && p.mask[i]) local_map[p.sub_to_full[i]] = kAbsentF;
}

}  // namespace hc

using namespace hc;

static int64_t max_frontier(const hc_fixed_batch* b) {
  int64_t m = b->caps[0];
  for (int h = 1; h < b->num_hops; ++h) {
    const int64_t f = b->caps[h] - b->caps[h - 1];
    if (f > m) m = f;
  }
  return m;
}
static int64_t max_draws(const hc_fixed_batch* b) {
  int64_t m = 0;
  for (int h = 0; h < b->num_hops; ++h) {
    const int64_t f = (h == 0 ? b->caps[0] : b->caps[h] - b->caps[h - 1]) * (int64_t)b->fanout[h];
    if (f > m) m = f;
  }
  return m;
}

extern "C" int64_t hc_sample_fixed_scratch_bytes(const hc_fixed_batch* b) {
  if (!b || b->num_hops < 1 || b->num_hops > kMaxHops) return 0;
  const int64_t draws = max_draws(b);
  return (16 + (max_frontier(b) + 2) + 2 * (draws + 1) + (draws / 1024 + 2)) * (int64_t)sizeof(int64_t);
}

extern "C" int hc_sample_fixed(const int64_t* gptr, const int64_t* gidx, const int64_t* seeds, int64_t n_seeds,
                               int32_t* local_map, uint64_t seed, int64_t* batch_no,
                               const hc_fixed_batch* b, void* scratch, void* stream) {
  HC_REQUIRE(b != nullptr, HC_ERR_NULL);
  HC_REQUIRE(b->struct_size == sizeof(hc_fixed_batch), HC_ERR_STRUCT);
  HC_REQUIRE(b->num_hops >= 1 && b->num_hops <= kMaxHops, HC_ERR_SIZE);
  HC_REQUIRE(n_seeds >= 0 && n_seeds <= b->caps[0] && b->edge_cap >= 0, HC_ERR_SIZE);
  for (int h = 0; h < b->num_hops; ++h)
    HC_REQUIRE(b->fanout[h] >= 1 && b->caps[h + 1] >= b->caps[h] && b->caps[h] >= 0, HC_ERR_SIZE);
  HC_REQUIRE(b->caps[b->num_hops] < 0x7fffffffLL, HC_ERR_SIZE);
  HC_REQUIRE(gptr && gidx && local_map && batch_no && scratch && b->ptr && b->idx && b->sub_to_full && b->mask &&
                 b->counters && (seeds || n_seeds == 0),
             HC_ERR_NULL);
  HC_REQUIRE(aligned_to(scratch, 8), HC_ERR_ALIGN);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  FixedPlan p;
  p.num_hops = b->num_hops;
  for (int h = 0; h < kMaxHops; ++h) p.fanout[h] = h < b->num_hops ? b->fanout[h] : 0;
  for (int h = 0; h <= kMaxHops; ++h) p.caps[h] = h <= b->num_hops ? b->caps[h] : 0;
  p.edge_cap = b->edge_cap;
  p.ptr = b->ptr; p.idx = b->idx; p.sub_to_full = b->sub_to_full; p.mask = b->mask; p.counters = b->counters;
  const int64_t draws = max_draws(b), mf = max_frontier(b);
  int64_t* w = reinterpret_cast<int64_t*>(scratch);
  p.state = w; w += 16;
  p.cnt = w; w += mf + 2;
  p.nbr = w; w += draws + 1;
  p.new_nodes = w; w += draws + 1;
  p.block_counts = w;
  const int64_t total = p.caps[p.num_hops];
  auto blocks = [](int64_t n, int per) { return (unsigned)ceil_div(n > 0 ? n : 1, per); };
  if (p.edge_cap > 0) HC_CUDA(cudaMemsetAsync(p.idx, 0, (size_t)p.edge_cap * sizeof(int64_t), st));
  fixed_begin_kernel<<<blocks(total, 256), 256, 0, st>>>(p, seeds, n_seeds, local_map, seed, batch_no);
  // state[5] = size of the current frontier (real nodes)
  HC_CUDA(cudaMemcpyAsync(p.state + 5, b->counters, sizeof(int64_t), cudaMemcpyDeviceToDevice, st));
  for (int h = 0; h < p.num_hops; ++h) {
    const int64_t fs = h == 0 ? 0 : p.caps[h - 1];
    const int64_t nf = p.caps[h] - fs;                  // frontier capacity (rows [fs, caps[h]))
    const int64_t row0 = p.caps[h];                     // the new nodes' first row
    const int64_t cap_new = p.caps[h + 1] - p.caps[h];
    const int fan = p.fanout[h];
    const int64_t m = nf * fan;                         // draw capacity of this hop
    if (nf == 0) continue;
    fixed_counts_kernel<<<blocks(nf, 256), 256, 0, st>>>(p, gptr, fs, nf, fan);
    fixed_scan_kernel<<<1, 1024, 0, st>>>(p, nf);
    fixed_picks_kernel<<<blocks(m, 256), 256, 0, st>>>(p, gptr, gidx, fs, nf, fan);
    fixed_claim_kernel<<<blocks(m, 256), 256, 0, st>>>(p, local_map);
    const unsigned nb = blocks(m, 1024);
    fixed_first_count_kernel<<<nb, 1024, 0, st>>>(p, local_map);
    fixed_first_scan_kernel<<<1, 1024, 0, st>>>(p, nb);
    fixed_place_kernel<<<nb, 1024, 0, st>>>(p, local_map, row0, cap_new);
    fixed_assign_kernel<<<blocks(m, 256), 256, 0, st>>>(p, local_map, row0, cap_new);
    fixed_translate_kernel<<<blocks(m, 256), 256, 0, st>>>(p, local_map, fs, nf, fan);
    fixed_unclaim_kernel<<<blocks(m, 256), 256, 0, st>>>(p, local_map);
    fixed_hop_end_kernel<<<1, 1, 0, st>>>(p, cap_new, h == p.num_hops - 1 ? 1 : 0, p.caps[p.num_hops - 1]);
  }
  fixed_finish_kernel<<<blocks(total, 256), 256, 0, st>>>(p, local_map);
  HC_LAUNCH_OK();
  return 0;
}
