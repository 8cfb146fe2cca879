// Shared device/host helpers for libhiscache_b200 (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "hiscache_b200.h"

#define HC_CUDA(call)                        \
  do {                                       \
    cudaError_t hc_e_ = (call);              \
    if (hc_e_ != cudaSuccess) return (int)hc_e_; \
  } while (0)

// Launch errors are read with cudaPeekAtLastError so that a sticky error left
// by somebody else's kernel is reported, not swallowed.
#define HC_LAUNCH_OK()                           \
  do {                                           \
    cudaError_t hc_e_ = cudaPeekAtLastError();   \
    if (hc_e_ != cudaSuccess) return (int)hc_e_; \
  } while (0)

#define HC_REQUIRE(cond, err) \
  do {                        \
    if (!(cond)) return -(err); \
  } while (0)

namespace hc {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline int dtype_size(int dt) { return dt == HC_F32 ? 4 : (dt == HC_F16 ? 2 : 0); }

// 64-bit shuffle (two 32-bit shuffles).
__device__ __forceinline__ int64_t shfl64(int64_t v, int src) {
  return __shfl_sync(kFull, (long long)v, src);
}

// Element load with run-time dtype, converted to fp32.
__device__ __forceinline__ float load_as_f32(const void* base, int dt, int64_t off) {
  return dt == HC_F16 ? __half2float(reinterpret_cast<const __half*>(base)[off])
                      : reinterpret_cast<const float*>(base)[off];
}
__device__ __forceinline__ void store_from_f32(void* base, int dt, int64_t off, float v) {
  if (dt == HC_F16)
    reinterpret_cast<__half*>(base)[off] = __float2half_rn(v);
  else
    reinterpret_cast<float*>(base)[off] = v;
}

// 16-byte read-only load.
__device__ __forceinline__ uint4 ldg16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// Unpack a 16-byte vector of T into fp32 values.
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
};
template <>
struct Vec16<__half> {
  static constexpr int kElems = 8;
  __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
    float2 c = __half22float2(h[2]), d = __half22float2(h[3]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
};

// acc[0..EL) += the EL elements of a 16-byte vector of T.  For fp16 this uses the
// mixed-precision add of sm_100 (f32 += f16 in one instruction; the widening is exact, so
// the result equals convert-then-add).
template <typename T>
__device__ __forceinline__ void accumulate_vec(float* acc, const uint4& v);
template <>
__device__ __forceinline__ void accumulate_vec<float>(float* acc, const uint4& v) {
  acc[0] += __uint_as_float(v.x);
  acc[1] += __uint_as_float(v.y);
  acc[2] += __uint_as_float(v.z);
  acc[3] += __uint_as_float(v.w);
}
#define HC_MIXED_ADD2(a0, a1, word)                                                   \
  asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %2; add.f32.f16 %0, lo, %0; "             \
      "add.f32.f16 %1, hi, %1;}"                                                      \
      : "+f"(a0), "+f"(a1)                                                            \
      : "r"(word))
template <>
__device__ __forceinline__ void accumulate_vec<__half>(float* acc, const uint4& v) {
  HC_MIXED_ADD2(acc[0], acc[1], v.x);
  HC_MIXED_ADD2(acc[2], acc[3], v.y);
  HC_MIXED_ADD2(acc[4], acc[5], v.z);
  HC_MIXED_ADD2(acc[6], acc[7], v.w);
}

// Vectorised fp32 reduction into global memory (one 16-byte transaction).
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

// ---- bulk-copy engine (TMA, untiled cp.async.bulk) and mbarrier helpers -----
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem),
               "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}


// ---- the library's fixed score reduction --------------------------------
// Element e of a row belongs to lane (e/4) mod 32; a lane adds its terms in
// increasing e with separately rounded multiply and add; partial sums are
// combined by an xor butterfly; L2 ends with a correctly rounded sqrt.
__device__ __forceinline__ float score_term(float acc, float x, int kind) {
  return kind == HC_SCORE_L2 ? __fadd_rn(acc, __fmul_rn(x, x)) : __fadd_rn(acc, fabsf(x));
}
__device__ __forceinline__ float score_finish(float partial, int kind) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) partial = __fadd_rn(partial, __shfl_xor_sync(kFull, partial, off));
  return kind == HC_SCORE_L2 ? __fsqrt_rn(partial) : partial;
}
__device__ __forceinline__ float row_score(const float* row, int feat, int kind, int lane) {
  float acc = 0.f;
  for (int c0 = 0; c0 < feat; c0 += 128) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      int e = c0 + 4 * lane + k;
      if (e < feat) acc = score_term(acc, row[e], kind);
    }
  }
  return score_finish(acc, kind);
}

// splitmix64 finaliser: the owner hash of the sharded table.
__host__ __device__ inline uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

}  // namespace hc
