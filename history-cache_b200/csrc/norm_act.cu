// Batch norm (training statistics) + ReLU + dropout as one forward pair and one backward pair.
//
// The dense part of a GraphSAGE / RGCN layer in the reference is torch's BatchNorm1d, relu and
// dropout applied one after the other (hiscache/history_model.py:141-143, :383-385): with
// autograd that is about eight kernels and as many passes over the [rows, hidden] activations
// per layer and direction.  Here the forward is two kernels (column statistics, then
// normalise + affine + ReLU + dropout) and the backward is two (column sums of dz and dz*xhat,
// then dx); the dropout mask is not stored but regenerated from (seed, step counter, element),
// and ReLU's mask is recomputed from x.  Rows can be masked out (padding rows of fixed-shape
// batches): they do not enter the statistics and produce zeros.
//
// Column statistics are reproducible: every block writes its partial sums, the block that
// finishes last adds them in block order in double precision.
#include "common.cuh"

namespace hc {

constexpr int kNormBlock = 256;     // apply kernels
constexpr int kStatsBlock = 1024;   // statistics kernels: one block per SM, 32 warps of loads in flight
constexpr int kNormMaxPartials = 148;   // blocks of the statistics kernels (one per SM)

struct NormGeom {
  int nvec;   // float4 per row
  int rpi;    // rows per block iteration
};
__host__ __device__ inline NormGeom norm_geom(int feat, int threads) {
  NormGeom g;
  g.nvec = feat / 4;
  g.rpi = threads / g.nvec;
  if (g.rpi < 1) g.rpi = 1;
  return g;
}

// keep mask of the four elements of float4 number `vec_index` (bit q set = element q kept)
__device__ __forceinline__ unsigned dropout_keep4(uint64_t seed, int64_t step, int64_t vec_index,
                                                 uint32_t thresh16) {
  const uint64_t h = mix64(mix64(seed ^ (uint64_t)step * 0xD6E8FEB86659FD93ull) ^ (uint64_t)vec_index);
  unsigned m = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) m |= ((uint32_t)((h >> (16 * q)) & 0xFFFFu) >= thresh16 ? 1u : 0u) << q;
  return m;
}

// sum over blocks b of p[b * stride + c], in a fixed order, with eight loads in flight
// Sum over blocks b of p[b * stride + c] in a fixed order, by the whole block: thread t takes
// column t % feat and the blocks b = t / feat, t / feat + parts, ... (eight loads in flight), the
// `parts` partial sums of a column are then added in part order.  red: shared double [2][parts * feat].
// Returns the two column sums (p and p + feat) to the threads with t < feat; all threads must call.
__device__ __forceinline__ void column_sums(const float* p, int feat, unsigned nb, double* red, double* s0,
                                            double* s1) {
  const int parts = blockDim.x / feat > 0 ? blockDim.x / feat : 1;
  const int64_t stride = 2 * (int64_t)feat;
  for (int base = 0; base < feat; base += blockDim.x) {      // feat > blockDim.x: several rounds
    const int t = threadIdx.x;
    const int c = base + (parts > 1 ? t % feat : t);
    const int part = parts > 1 ? t / feat : 0;
    double a0 = 0.0, a1 = 0.0;
    if (c < feat && part < parts) {
      unsigned b = part;
      for (; b + 3u * parts < nb; b += 4u * parts) {
        float v[4], q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[j] = __ldcg(p + (int64_t)(b + j * parts) * stride + c);
          q[j] = __ldcg(p + (int64_t)(b + j * parts) * stride + feat + c);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) { a0 += (double)v[j]; a1 += (double)q[j]; }
      }
      for (; b < nb; b += parts) {
        a0 += (double)__ldcg(p + (int64_t)b * stride + c);
        a1 += (double)__ldcg(p + (int64_t)b * stride + feat + c);
      }
      red[part * feat + (c - base)] = a0;
      red[(parts + part) * feat + (c - base)] = a1;
    }
    __syncthreads();
    if (c < feat && part == 0) {
      double t0 = 0.0, t1 = 0.0;
      for (int k = 0; k < parts; ++k) {
        t0 += red[k * feat + (c - base)];
        t1 += red[(parts + k) * feat + (c - base)];
      }
      s0[base / blockDim.x] = t0;
      s1[base / blockDim.x] = t1;
    }
    __syncthreads();
  }
}

struct NormArgs {
  const float* x; int64_t n; int feat; int64_t stride;
  const uint8_t* valid;
  const float* weight; const float* bias;
  float* running_mean; float* running_var; float momentum; float eps;
  float drop_p; uint64_t seed; int64_t* counter; int64_t* saved_step;   // state[0], state[1]
  float* save_mean; float* save_rstd; float* save_count;
  int relu;
  // scratch
  float* partial;          // [blocks][2][feat]  (+ [blocks] counts behind)
  float* partial_count;    // [blocks]
  unsigned int* ticket;
};

// thread layout shared by all four kernels: column vector `cv`, row slot `rs`
#define HC_NORM_LAYOUT(a)                                  \
  const NormGeom g = norm_geom((a).feat, blockDim.x);      \
  const int cv = threadIdx.x % g.nvec;                     \
  const int rs = threadIdx.x / g.nvec;                     \
  const bool active = rs < g.rpi && threadIdx.x < g.nvec * g.rpi;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// ---- forward 1: column sums -------------------------------------------------
__global__ void __launch_bounds__(kStatsBlock) norm_stats_kernel(const NormArgs a) {
  extern __shared__ __align__(16) float sh[];   // [rpi][nvec] float4 x 2
  __shared__ float sh_cnt[kStatsBlock];
  __shared__ bool is_last;
  HC_NORM_LAYOUT(a)
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f), q = s;
  float cnt = 0.f;
  if (active) {
    for (int64_t r = (int64_t)blockIdx.x * g.rpi + rs; r < a.n; r += (int64_t)gridDim.x * g.rpi) {
      if (a.valid && !a.valid[r]) continue;
      const float4 v = ld4(a.x + r * a.stride + 4 * cv);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      q.x = fmaf(v.x, v.x, q.x); q.y = fmaf(v.y, v.y, q.y);
      q.z = fmaf(v.z, v.z, q.z); q.w = fmaf(v.w, v.w, q.w);
      cnt += 1.f;
    }
  }
  float4* sh_s = reinterpret_cast<float4*>(sh);
  float4* sh_q = sh_s + g.rpi * g.nvec;
  if (active) {
    sh_s[rs * g.nvec + cv] = s;
    sh_q[rs * g.nvec + cv] = q;
  }
  sh_cnt[threadIdx.x] = (active && cv == 0) ? cnt : 0.f;
  __syncthreads();
  if (active && rs == 0) {
    for (int k = 1; k < g.rpi; ++k) {
      const float4 s2 = sh_s[k * g.nvec + cv], q2 = sh_q[k * g.nvec + cv];
      s.x += s2.x; s.y += s2.y; s.z += s2.z; s.w += s2.w;
      q.x += q2.x; q.y += q2.y; q.z += q2.z; q.w += q2.w;
    }
    float* p = a.partial + (int64_t)blockIdx.x * 2 * a.feat;
    *reinterpret_cast<float4*>(p + 4 * cv) = s;
    *reinterpret_cast<float4*>(p + a.feat + 4 * cv) = q;
  }
  if (threadIdx.x == 0) {
    float c = 0.f;
    for (int k = 0; k < g.rpi; ++k) c += sh_cnt[k * g.nvec];
    a.partial_count[blockIdx.x] = c;
  }
  // the block that takes the last ticket reduces all partials in block order
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(a.ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  double n_valid = 0.0;
  for (unsigned b = 0; b < gridDim.x; ++b) n_valid += (double)__ldcg(a.partial_count + b);
  double cs0[1], cs1[1];
  column_sums(a.partial, a.feat, gridDim.x, reinterpret_cast<double*>(sh), cs0, cs1);
  for (int c = threadIdx.x; c < a.feat; c += blockDim.x) {   // feat <= 1024 = blockDim.x: one round
    const double sum = cs0[0], sq = cs1[0];
    const double nn = n_valid > 0.0 ? n_valid : 1.0;
    const double mean = sum / nn;
    double var = sq / nn - mean * mean;
    if (var < 0.0) var = 0.0;
    a.save_mean[c] = (float)mean;
    a.save_rstd[c] = (float)(1.0 / sqrt(var + (double)a.eps));
    if (a.running_mean) {
      const double unb = n_valid > 1.0 ? var * (n_valid / (n_valid - 1.0)) : var;
      a.running_mean[c] = (float)((1.0 - a.momentum) * (double)a.running_mean[c] + a.momentum * mean);
      a.running_var[c] = (float)((1.0 - a.momentum) * (double)a.running_var[c] + a.momentum * unb);
    }
  }
  if (threadIdx.x == 0) {
    a.save_count[0] = (float)n_valid;
    *a.ticket = 0;
    if (a.counter) {      // this call's dropout stream; the next call gets the next one
      a.saved_step[0] = a.counter[0];
      a.counter[0] += 1;
    }
  }
}

// ---- forward 2: y = dropout(relu(xhat * w + b)) -------------------------------
__global__ void __launch_bounds__(kNormBlock) norm_apply_kernel(const NormArgs a, float* __restrict__ y) {
  HC_NORM_LAYOUT(a)
  if (!active) return;
  const float4 mean = ld4(a.save_mean + 4 * cv), rstd = ld4(a.save_rstd + 4 * cv);
  const float4 w = a.weight ? ld4(a.weight + 4 * cv) : make_float4(1.f, 1.f, 1.f, 1.f);
  const float4 b = a.bias ? ld4(a.bias + 4 * cv) : make_float4(0.f, 0.f, 0.f, 0.f);
  const bool drop = a.drop_p > 0.f;
  const float scale = drop ? 1.f / (1.f - a.drop_p) : 1.f;
  const uint32_t thresh = (uint32_t)(a.drop_p * 65536.f);
  const int64_t step = drop ? a.saved_step[0] : 0;
  for (int64_t r = (int64_t)blockIdx.x * g.rpi + rs; r < a.n; r += (int64_t)gridDim.x * g.rpi) {
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!(a.valid && !a.valid[r])) {
      const float4 v = ld4(a.x + r * a.stride + 4 * cv);
      o.x = fmaf((v.x - mean.x) * rstd.x, w.x, b.x);
      o.y = fmaf((v.y - mean.y) * rstd.y, w.y, b.y);
      o.z = fmaf((v.z - mean.z) * rstd.z, w.z, b.z);
      o.w = fmaf((v.w - mean.w) * rstd.w, w.w, b.w);
      if (a.relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
      if (drop) {
        const unsigned k = dropout_keep4(a.seed, step, r * g.nvec + cv, thresh);
        o.x = (k & 1u) ? o.x * scale : 0.f;
        o.y = (k & 2u) ? o.y * scale : 0.f;
        o.z = (k & 4u) ? o.z * scale : 0.f;
        o.w = (k & 8u) ? o.w * scale : 0.f;
      }
    }
    *reinterpret_cast<float4*>(y + r * a.feat + 4 * cv) = o;
  }
}

// dz = dy * dropout * relu'(z) for one float4, and xhat
__device__ __forceinline__ void norm_dz(const NormArgs& a, const float4& v, const float4& dy, const float4& mean,
                                        const float4& rstd, const float4& w, const float4& b, unsigned keep,
                                        float scale, float4* dz, float4* xh) {
  xh->x = (v.x - mean.x) * rstd.x; xh->y = (v.y - mean.y) * rstd.y;
  xh->z = (v.z - mean.z) * rstd.z; xh->w = (v.w - mean.w) * rstd.w;
  const bool px = !a.relu || fmaf(xh->x, w.x, b.x) > 0.f, py = !a.relu || fmaf(xh->y, w.y, b.y) > 0.f;
  const bool pz = !a.relu || fmaf(xh->z, w.z, b.z) > 0.f, pw = !a.relu || fmaf(xh->w, w.w, b.w) > 0.f;
  dz->x = (px && (keep & 1u)) ? dy.x * scale : 0.f;
  dz->y = (py && (keep & 2u)) ? dy.y * scale : 0.f;
  dz->z = (pz && (keep & 4u)) ? dy.z * scale : 0.f;
  dz->w = (pw && (keep & 8u)) ? dy.w * scale : 0.f;
}

// ---- backward 1: column sums of dz and dz * xhat ------------------------------
struct NormBwd {
  const float* grad_y;
  float* grad_weight; float* grad_bias;   // [feat] or NULL
  float* sum_dz; float* sum_dzx;          // [feat] scratch handed to the second kernel
};

__global__ void __launch_bounds__(kStatsBlock) norm_bwd_stats_kernel(const NormArgs a, const NormBwd bw) {
  extern __shared__ __align__(16) float sh[];
  __shared__ bool is_last;
  HC_NORM_LAYOUT(a)
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f), q = s;
  if (active) {
    const float4 mean = ld4(a.save_mean + 4 * cv), rstd = ld4(a.save_rstd + 4 * cv);
    const float4 w = a.weight ? ld4(a.weight + 4 * cv) : make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 b = a.bias ? ld4(a.bias + 4 * cv) : make_float4(0.f, 0.f, 0.f, 0.f);
    const bool drop = a.drop_p > 0.f;
    const float scale = drop ? 1.f / (1.f - a.drop_p) : 1.f;
    const uint32_t thresh = (uint32_t)(a.drop_p * 65536.f);
    const int64_t step = drop ? a.saved_step[0] : 0;
    for (int64_t r = (int64_t)blockIdx.x * g.rpi + rs; r < a.n; r += (int64_t)gridDim.x * g.rpi) {
      if (a.valid && !a.valid[r]) continue;
      const float4 v = ld4(a.x + r * a.stride + 4 * cv);
      const float4 dy = ld4(bw.grad_y + r * a.feat + 4 * cv);
      const unsigned keep = drop ? dropout_keep4(a.seed, step, r * g.nvec + cv, thresh) : 15u;
      float4 dz, xh;
      norm_dz(a, v, dy, mean, rstd, w, b, keep, scale, &dz, &xh);
      s.x += dz.x; s.y += dz.y; s.z += dz.z; s.w += dz.w;
      q.x = fmaf(dz.x, xh.x, q.x); q.y = fmaf(dz.y, xh.y, q.y);
      q.z = fmaf(dz.z, xh.z, q.z); q.w = fmaf(dz.w, xh.w, q.w);
    }
  }
  float4* sh_s = reinterpret_cast<float4*>(sh);
  float4* sh_q = sh_s + g.rpi * g.nvec;
  if (active) {
    sh_s[rs * g.nvec + cv] = s;
    sh_q[rs * g.nvec + cv] = q;
  }
  __syncthreads();
  if (active && rs == 0) {
    for (int k = 1; k < g.rpi; ++k) {
      const float4 s2 = sh_s[k * g.nvec + cv], q2 = sh_q[k * g.nvec + cv];
      s.x += s2.x; s.y += s2.y; s.z += s2.z; s.w += s2.w;
      q.x += q2.x; q.y += q2.y; q.z += q2.z; q.w += q2.w;
    }
    float* p = a.partial + (int64_t)blockIdx.x * 2 * a.feat;
    *reinterpret_cast<float4*>(p + 4 * cv) = s;
    *reinterpret_cast<float4*>(p + a.feat + 4 * cv) = q;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(a.ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  double cs0[1], cs1[1];
  column_sums(a.partial, a.feat, gridDim.x, reinterpret_cast<double*>(sh), cs0, cs1);
  for (int c = threadIdx.x; c < a.feat; c += blockDim.x) {
    const double sum = cs0[0], sq = cs1[0];
    bw.sum_dz[c] = (float)sum;
    bw.sum_dzx[c] = (float)sq;
    if (bw.grad_bias) bw.grad_bias[c] = (float)sum;
    if (bw.grad_weight) bw.grad_weight[c] = (float)sq;
  }
  if (threadIdx.x == 0) *a.ticket = 0;
}

// ---- backward 2: dx = w * rstd * (dz - mean(dz) - xhat * mean(dz * xhat)) -------
__global__ void __launch_bounds__(kNormBlock)
    norm_bwd_apply_kernel(const NormArgs a, const NormBwd bw, float* __restrict__ grad_x) {
  HC_NORM_LAYOUT(a)
  if (!active) return;
  const float4 mean = ld4(a.save_mean + 4 * cv), rstd = ld4(a.save_rstd + 4 * cv);
  const float4 w = a.weight ? ld4(a.weight + 4 * cv) : make_float4(1.f, 1.f, 1.f, 1.f);
  const float4 b = a.bias ? ld4(a.bias + 4 * cv) : make_float4(0.f, 0.f, 0.f, 0.f);
  const float cnt = a.save_count[0] > 0.f ? a.save_count[0] : 1.f;
  const float inv_n = 1.f / cnt;
  float4 m1 = ld4(bw.sum_dz + 4 * cv), m2 = ld4(bw.sum_dzx + 4 * cv);
  m1.x *= inv_n; m1.y *= inv_n; m1.z *= inv_n; m1.w *= inv_n;
  m2.x *= inv_n; m2.y *= inv_n; m2.z *= inv_n; m2.w *= inv_n;
  const bool drop = a.drop_p > 0.f;
  const float scale = drop ? 1.f / (1.f - a.drop_p) : 1.f;
  const uint32_t thresh = (uint32_t)(a.drop_p * 65536.f);
  const int64_t step = drop ? a.saved_step[0] : 0;
  for (int64_t r = (int64_t)blockIdx.x * g.rpi + rs; r < a.n; r += (int64_t)gridDim.x * g.rpi) {
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!(a.valid && !a.valid[r])) {
      const float4 v = ld4(a.x + r * a.stride + 4 * cv);
      const float4 dy = ld4(bw.grad_y + r * a.feat + 4 * cv);
      const unsigned keep = drop ? dropout_keep4(a.seed, step, r * g.nvec + cv, thresh) : 15u;
      float4 dz, xh;
      norm_dz(a, v, dy, mean, rstd, w, b, keep, scale, &dz, &xh);
      o.x = w.x * rstd.x * (dz.x - m1.x - xh.x * m2.x);
      o.y = w.y * rstd.y * (dz.y - m1.y - xh.y * m2.y);
      o.z = w.z * rstd.z * (dz.z - m1.z - xh.z * m2.z);
      o.w = w.w * rstd.w * (dz.w - m1.w - xh.w * m2.w);
    }
    *reinterpret_cast<float4*>(grad_x + r * a.feat + 4 * cv) = o;
  }
}


static int fill(const hc_norm_args* p, void* scratch, NormArgs* a, NormBwd* bw) {
  HC_REQUIRE(p != nullptr, HC_ERR_NULL);
  HC_REQUIRE(p->struct_size == sizeof(hc_norm_args), HC_ERR_STRUCT);
  HC_REQUIRE(p->n >= 0 && p->feat > 0, HC_ERR_SIZE);
  HC_REQUIRE(p->feat % 4 == 0 && p->feat <= 1024, HC_ERR_UNSUPPORTED);
  HC_REQUIRE(p->drop_p >= 0.f && p->drop_p < 1.f && p->eps > 0.f, HC_ERR_SIZE);
  HC_REQUIRE(p->x && p->state && p->save_mean && p->save_rstd && p->save_count && scratch, HC_ERR_NULL);
  const int64_t stride = p->x_stride ? p->x_stride : p->feat;
  HC_REQUIRE(stride >= p->feat && stride % 4 == 0 && aligned16(p->x) && aligned16(scratch), HC_ERR_UNSUPPORTED);
  HC_REQUIRE((!p->weight || aligned16(p->weight)) && (!p->bias || aligned16(p->bias)) &&
                 aligned16(p->save_mean) && aligned16(p->save_rstd), HC_ERR_UNSUPPORTED);
  HC_REQUIRE((p->running_mean == nullptr) == (p->running_var == nullptr), HC_ERR_NULL);
  a->x = p->x; a->n = p->n; a->feat = p->feat; a->stride = stride; a->valid = p->valid;
  a->weight = p->weight; a->bias = p->bias;
  a->running_mean = p->running_mean; a->running_var = p->running_var;
  a->momentum = p->momentum; a->eps = p->eps; a->drop_p = p->drop_p; a->seed = p->seed;
  a->counter = p->drop_p > 0.f ? p->state : nullptr;
  a->saved_step = p->state + 1;
  a->ticket = reinterpret_cast<unsigned int*>(p->state + 2);
  a->save_mean = p->save_mean; a->save_rstd = p->save_rstd; a->save_count = p->save_count;
  a->relu = p->relu ? 1 : 0;
  float* f = reinterpret_cast<float*>(scratch);
  a->partial = f;
  a->partial_count = f + (int64_t)kNormMaxPartials * 2 * p->feat;
  bw->sum_dz = a->partial_count + kNormMaxPartials;
  bw->sum_dzx = bw->sum_dz + p->feat;
  return 0;
}

static void grids(const NormArgs& a, unsigned* stats_blocks, unsigned* apply_blocks, size_t* smem) {
  const NormGeom gs = norm_geom(a.feat, kStatsBlock), ga = norm_geom(a.feat, kNormBlock);
  const int64_t n = a.n > 0 ? a.n : 1;
  const int64_t si = ceil_div(n, gs.rpi), ai = ceil_div(n, ga.rpi);
  *stats_blocks = (unsigned)(si < kNormMaxPartials ? si : kNormMaxPartials);
  *apply_blocks = (unsigned)(ai < 148 * 8 ? ai : 148 * 8);
  // block partial sums (float4 x 2 per row slot), reused by the last block for the column sums
  size_t need = (size_t)2 * gs.rpi * gs.nvec * sizeof(float4);
  const int parts = kStatsBlock / a.feat > 0 ? kStatsBlock / a.feat : 1;
  const size_t fin = (size_t)2 * parts * a.feat * sizeof(double);
  *smem = need > fin ? need : fin;
}

}  // namespace hc

using namespace hc;

extern "C" int64_t hc_norm_scratch_bytes(int32_t feat) {
  if (feat < 1) feat = 1;
  return ((int64_t)kNormMaxPartials * (2 * feat + 1) + 2 * feat) * (int64_t)sizeof(float) + 64;
}

extern "C" int hc_norm_act_fwd(const hc_norm_args* p, float* y, void* scratch, void* stream) {
  NormArgs a;
  NormBwd bw;
  int rc = fill(p, scratch, &a, &bw);
  if (rc) return rc;
  if (a.n == 0) return 0;
  HC_REQUIRE(y && aligned16(y), HC_ERR_NULL);
  unsigned sb, ab;
  size_t smem;
  grids(a, &sb, &ab, &smem);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  norm_stats_kernel<<<sb, kStatsBlock, smem, st>>>(a);
  norm_apply_kernel<<<ab, kNormBlock, 0, st>>>(a, y);
  HC_LAUNCH_OK();
  return 0;
}

extern "C" int hc_norm_act_bwd(const hc_norm_args* p, const float* grad_y, float* grad_x, float* grad_weight,
                               float* grad_bias, void* scratch, void* stream) {
  NormArgs a;
  NormBwd bw;
  int rc = fill(p, scratch, &a, &bw);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a.n == 0) {
    if (grad_weight) HC_CUDA(cudaMemsetAsync(grad_weight, 0, (size_t)a.feat * sizeof(float), st));
    if (grad_bias) HC_CUDA(cudaMemsetAsync(grad_bias, 0, (size_t)a.feat * sizeof(float), st));
    return 0;
  }
  HC_REQUIRE(grad_y && grad_x && aligned16(grad_y) && aligned16(grad_x), HC_ERR_NULL);
  a.counter = nullptr;          // the backward pass reads this call's dropout stream, it does not advance it
  a.running_mean = a.running_var = nullptr;
  bw.grad_y = grad_y;
  bw.grad_weight = grad_weight;
  bw.grad_bias = grad_bias;
  unsigned sb, ab;
  size_t smem;
  grids(a, &sb, &ab, &smem);
  norm_bwd_stats_kernel<<<sb, kStatsBlock, smem, st>>>(a, bw);
  norm_bwd_apply_kernel<<<ab, kNormBlock, 0, st>>>(a, bw, grad_x);
  HC_LAUNCH_OK();
  return 0;
}
