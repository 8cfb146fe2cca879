// Backward aggregation as a gather over the transposed block.
//
// The reference (and hc_aggr_bwd) push gradients to the sources with atomic adds
// (src/cpp/src/history_aggr.cu:127-168).  On blocks larger than L2 that scatter is
// bound by read-modify-write DRAM traffic: every reduction that misses L2 moves its
// line DRAM -> L2 -> DRAM, and grad_input needs a zero-fill first.  Here the block is
// transposed once (source -> list of destination rows, each list sorted, so the
// result is reproducible bit for bit) and every source row is then written exactly
// once as the sum of its destinations' gradient rows: no atomics on the data, no
// zero-fill, deterministic.
#include "common.cuh"

namespace hc {

constexpr int kTScan = 1024;

// edges of miss rows whose source takes a gradient
__device__ __forceinline__ bool edge_counts(const hc_aggr_args& a, int64_t r, int64_t s) {
  (void)r;
  return !(a.src_map && a.src_map[s] != -1);
}

__global__ void __launch_bounds__(256) tr_count_kernel(const hc_aggr_args a, long long* cnt) {
  constexpr int G = 8;
  const int gl = threadIdx.x & (G - 1);
  const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (r >= a.num_node) return;
  if (a.hmap && a.hmap[r] != -1) return;
  for (int64_t e = a.ptr[r] + gl; e < a.ptr[r + 1]; e += G) {
    const int64_t s = a.idx[e];
    if (edge_counts(a, r, s)) atomicAdd(reinterpret_cast<unsigned long long*>(cnt + s), 1ull);
  }
}

// three-phase exclusive scan of cnt[0..n) into out[0..n], out[n] = total
__global__ void __launch_bounds__(kTScan)
    tr_block_sum_kernel(const long long* __restrict__ cnt, int64_t n, long long* __restrict__ sums) {
  __shared__ long long sh[kTScan / 32];
  const int64_t i = (int64_t)blockIdx.x * kTScan + threadIdx.x;
  long long v = i < n ? cnt[i] : 0;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFull, v, off);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    long long t = 0;
    for (int w = 0; w < kTScan / 32; ++w) t += sh[w];
    sums[blockIdx.x] = t;
  }
}
__global__ void __launch_bounds__(1024) tr_scan_sums_kernel(long long* sums, int64_t nb) {
  __shared__ long long part[1024];
  __shared__ long long carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < nb; base += 1024) {
    const int64_t b = base + threadIdx.x;
    const long long c = b < nb ? sums[b] : 0;
    part[threadIdx.x] = c;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const long long v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
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
__global__ void __launch_bounds__(kTScan)
    tr_scan_apply_kernel(const long long* __restrict__ cnt, int64_t n, const long long* __restrict__ sums,
                         int64_t* __restrict__ out, long long* __restrict__ cursor) {
  __shared__ long long wsum[kTScan / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t i = (int64_t)blockIdx.x * kTScan + threadIdx.x;
  const long long c = i < n ? cnt[i] : 0;
  long long v = c;  // inclusive scan inside the warp
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const long long t = __shfl_up_sync(kFull, v, off);
    if (lane >= off) v += t;
  }
  if (lane == 31) wsum[warp] = v;
  __syncthreads();
  long long before = sums[blockIdx.x];
  for (int w = 0; w < warp; ++w) before += wsum[w];
  if (i < n) {
    out[i] = before + v - c;
    cursor[i] = before + v - c;
    if (i == n - 1) out[n] = before + v;
  }
}

__global__ void __launch_bounds__(256)
    tr_fill_kernel(const hc_aggr_args a, long long* cursor, int64_t* __restrict__ t_dst) {
  constexpr int G = 8;
  const int gl = threadIdx.x & (G - 1);
  const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
  if (r >= a.num_node) return;
  if (a.hmap && a.hmap[r] != -1) return;
  for (int64_t e = a.ptr[r] + gl; e < a.ptr[r + 1]; e += G) {
    const int64_t s = a.idx[e];
    if (edge_counts(a, r, s)) {
      const long long pos = (long long)atomicAdd(reinterpret_cast<unsigned long long*>(cursor + s), 1ull);
      t_dst[pos] = r;
    }
  }
}

// each source's list ascending by destination row: the order of the atomics above no longer matters
__device__ __forceinline__ void tr_weights(const int64_t* __restrict__ ptr, const int64_t* v, float* w, int64_t k) {
  for (int64_t i = 0; i < k; ++i) w[i] = __frcp_rn((float)(ptr[v[i] + 1] - ptr[v[i]]));
}

__global__ void tr_sort_kernel(const int64_t* __restrict__ ptr, const int64_t* __restrict__ t_ptr,
                               int64_t n_src, int64_t* t_dst, float* t_w) {
  const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_src) return;
  const int64_t b = t_ptr[s], k = t_ptr[s + 1] - b;
  int64_t* v = t_dst + b;
  if (k < 2) {
    tr_weights(ptr, v, t_w + b, k);
    return;
  }
  if (k <= 32) {  // insertion sort
    for (int64_t i = 1; i < k; ++i) {
      const int64_t x = v[i];
      int64_t j = i - 1;
      while (j >= 0 && v[j] > x) { v[j + 1] = v[j]; --j; }
      v[j + 1] = x;
    }
    tr_weights(ptr, v, t_w + b, k);
    return;
  }
  // heap sort for the rare long lists
  for (int64_t start = k / 2 - 1; start >= 0; --start) {
    int64_t root = start;
    for (;;) {
      int64_t child = 2 * root + 1;
      if (child >= k) break;
      if (child + 1 < k && v[child] < v[child + 1]) ++child;
      if (v[root] >= v[child]) break;
      const int64_t t = v[root]; v[root] = v[child]; v[child] = t;
      root = child;
    }
  }
  for (int64_t end = k - 1; end > 0; --end) {
    const int64_t t0 = v[0]; v[0] = v[end]; v[end] = t0;
    int64_t root = 0;
    for (;;) {
      int64_t child = 2 * root + 1;
      if (child >= end) break;
      if (child + 1 < end && v[child] < v[child + 1]) ++child;
      if (v[root] >= v[child]) break;
      const int64_t t = v[root]; v[root] = v[child]; v[child] = t;
      root = child;
    }
  }
  tr_weights(ptr, v, t_w + b, k);
}

// grad_input[s, :] = sum over the transposed list of t_w * grad_out[r, :]; every row written once.
// A warp takes kSW consecutive sources: their lists are one contiguous slice of t_dst / t_w,
// fetched with one coalesced load when it has at most 32 entries, so that each source then
// costs a single round of row loads.
constexpr int kSW = 8;

template <int G, int V>
__global__ void __launch_bounds__(256)
    aggr_bwd_gather_kernel(const int64_t n_src, const int feat, const int64_t* __restrict__ t_ptr,
                           const int64_t* __restrict__ t_dst, const float* __restrict__ t_w,
                           const float* __restrict__ grad_out, float* __restrict__ grad_input,
                           const int nvec) {
  constexpr int EPW = kWarp / G;
  constexpr int U = V == 1 ? 4 : (V == 2 ? 2 : 1);
  const int lane = threadIdx.x & 31;
  const int64_t s0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kSW;
  if (s0 >= n_src) return;
  const int ns = (int)((n_src - s0) < kSW ? (n_src - s0) : kSW);
  const int sub = lane / G, gl = lane % G;
  const int64_t my_p = lane <= ns ? t_ptr[s0 + lane] : 0;
  const int64_t E0 = shfl64(my_p, 0), E1 = shfl64(my_p, ns);
  const bool one_chunk = (E1 - E0) <= kWarp;
  int64_t my_r = 0;
  float my_w = 0.f;
  if (one_chunk && E0 + lane < E1) {
    my_r = t_dst[E0 + lane];
    my_w = t_w[E0 + lane];
  }
  for (int k = 0; k < ns; ++k) {
    const int64_t begin = shfl64(my_p, k), end = shfl64(my_p, k + 1);
    float4 acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t i = begin; i < end; i += EPW * U) {
      float4 buf[U][V];
      float w[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t jj = i + u * EPW + sub;
        const bool ok = jj < end;
        int64_t r;
        if (one_chunk) {
          const int from = (int)(jj - E0) & 31;
          r = shfl64(my_r, from);
          w[u] = __shfl_sync(kFull, my_w, from);
        } else {
          r = ok ? t_dst[jj] : 0;
          w[u] = ok ? t_w[jj] : 0.f;
        }
        if (!ok) w[u] = 0.f;
#pragma unroll
        for (int q = 0; q < V; ++q) {
          const int v = gl + q * G;
          buf[u][q] = (ok && v < nvec) ? __ldg(reinterpret_cast<const float4*>(grad_out + r * feat) + v)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int q = 0; q < V; ++q) {
          acc[q].x = fmaf(w[u], buf[u][q].x, acc[q].x);
          acc[q].y = fmaf(w[u], buf[u][q].y, acc[q].y);
          acc[q].z = fmaf(w[u], buf[u][q].z, acc[q].z);
          acc[q].w = fmaf(w[u], buf[u][q].w, acc[q].w);
        }
    }
    if (EPW > 1) {
#pragma unroll
      for (int off = G; off < kWarp; off <<= 1)
#pragma unroll
        for (int q = 0; q < V; ++q) {
          acc[q].x += __shfl_xor_sync(kFull, acc[q].x, off);
          acc[q].y += __shfl_xor_sync(kFull, acc[q].y, off);
          acc[q].z += __shfl_xor_sync(kFull, acc[q].z, off);
          acc[q].w += __shfl_xor_sync(kFull, acc[q].w, off);
        }
    }
    if (sub == 0) {
#pragma unroll
      for (int q = 0; q < V; ++q) {
        const int v = gl + q * G;
        if (v < nvec) reinterpret_cast<float4*>(grad_input + (s0 + k) * feat)[v] = acc[q];
      }
    }
  }
}

}  // namespace hc

using namespace hc;

extern "C" int64_t hc_transpose_scratch_bytes(int64_t n_src) {
  const int64_t nb = ceil_div(n_src > 0 ? n_src : 1, kTScan);
  return (2 * (n_src + 1) + nb + 8) * (int64_t)sizeof(int64_t);
}

static int check_simple(const hc_aggr_args* a) {
  HC_REQUIRE(a != nullptr, HC_ERR_NULL);
  HC_REQUIRE(a->struct_size == sizeof(hc_aggr_args), HC_ERR_STRUCT);
  HC_REQUIRE(a->num_node >= 0 && a->n_src >= 0 && a->feat > 0, HC_ERR_SIZE);
  HC_REQUIRE(a->num_head == 1 && a->edge_value == nullptr, HC_ERR_UNSUPPORTED);
  return 0;
}

extern "C" int hc_transpose_block(const hc_aggr_args* a, int64_t* t_ptr, int64_t* t_dst,
                                  float* t_w, void* scratch, void* stream) {
  int rc = check_simple(a);
  if (rc) return rc;
  HC_REQUIRE(t_ptr != nullptr, HC_ERR_NULL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->n_src == 0) {
    HC_CUDA(cudaMemsetAsync(t_ptr, 0, sizeof(int64_t), st));
    return 0;
  }
  HC_REQUIRE(scratch != nullptr && aligned_to(scratch, 8), HC_ERR_NULL);
  HC_REQUIRE(a->num_node == 0 || (a->ptr && a->idx && t_dst && t_w), HC_ERR_NULL);
  long long* cnt = reinterpret_cast<long long*>(scratch);
  long long* cursor = cnt + (a->n_src + 1);
  long long* sums = cursor + (a->n_src + 1);
  const int64_t nb = ceil_div(a->n_src, kTScan);
  HC_REQUIRE(nb <= 0x7fffffffLL, HC_ERR_SIZE);
  HC_CUDA(cudaMemsetAsync(cnt, 0, (size_t)(a->n_src + 1) * sizeof(long long), st));
  const int64_t rb = ceil_div((a->num_node > 0 ? a->num_node : 1) * 8, 256);
  HC_REQUIRE(rb <= 0x7fffffffLL, HC_ERR_SIZE);
  if (a->num_node > 0) tr_count_kernel<<<(unsigned)rb, 256, 0, st>>>(*a, cnt);
  tr_block_sum_kernel<<<(unsigned)nb, kTScan, 0, st>>>(cnt, a->n_src, sums);
  tr_scan_sums_kernel<<<1, 1024, 0, st>>>(sums, nb);
  tr_scan_apply_kernel<<<(unsigned)nb, kTScan, 0, st>>>(cnt, a->n_src, sums, t_ptr, cursor);
  if (a->num_node > 0) {
    tr_fill_kernel<<<(unsigned)rb, 256, 0, st>>>(*a, cursor, t_dst);
    tr_sort_kernel<<<(unsigned)ceil_div(a->n_src, 256), 256, 0, st>>>(a->ptr, t_ptr, a->n_src, t_dst, t_w);
  }
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_aggr_bwd_gather(const hc_aggr_args* a, const int64_t* t_ptr, const int64_t* t_dst,
                                  const float* t_w, const float* grad_out, float* grad_input,
                                  void* stream) {
  int rc = check_simple(a);
  if (rc) return rc;
  if (a->n_src == 0) return 0;
  HC_REQUIRE(t_ptr && grad_input, HC_ERR_NULL);
  HC_REQUIRE(a->num_node == 0 || (t_dst && t_w && grad_out), HC_ERR_NULL);
  HC_REQUIRE(a->feat % 4 == 0 && aligned16(grad_out) && aligned16(grad_input), HC_ERR_UNSUPPORTED);
  const int nvec = a->feat / 4;
  int G, V;
  if (nvec <= 8) { G = 8; V = 1; }
  else if (nvec <= 16) { G = 16; V = 1; }
  else if (nvec <= 32) { G = 32; V = 1; }
  else if (nvec <= 64) { G = 32; V = 2; }
  else if (nvec <= 128) { G = 32; V = 4; }
  else if (nvec <= 256) { G = 32; V = 8; }
  else return -HC_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t blocks = ceil_div(ceil_div(a->n_src, kSW), 8);
  HC_REQUIRE(blocks <= 0x7fffffffLL, HC_ERR_SIZE);
  const unsigned g = (unsigned)blocks;
#define HC_GATHER_CASE(gg, vv)                                                                   \
  if (G == gg && V == vv)                                                                        \
    aggr_bwd_gather_kernel<gg, vv><<<g, 256, 0, st>>>(a->n_src, a->feat, t_ptr, t_dst, t_w, grad_out, \
                                                      grad_input, nvec);
  HC_GATHER_CASE(8, 1) HC_GATHER_CASE(16, 1) HC_GATHER_CASE(32, 1) HC_GATHER_CASE(32, 2)
  HC_GATHER_CASE(32, 4) HC_GATHER_CASE(32, 8)
#undef HC_GATHER_CASE
  HC_LAUNCH_OK();
  return 0;
}
