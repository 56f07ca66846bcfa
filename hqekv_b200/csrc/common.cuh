// Shared host/device helpers of libhqkv (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "hqkv.h"

namespace hqkv {

// ---- host-side error reporting ---------------------------------------------------------------
int fail(int code, const char* fmt, ...);  // records the message for hqkv_last_error(), returns code
int check_cuda(cudaError_t e, const char* what);

#define HQKV_REQUIRE(cond, ...)                                \
  do {                                                         \
    if (!(cond)) return ::hqkv::fail(HQKV_E_INVALID, __VA_ARGS__); \
  } while (0)

#define HQKV_CUDA(call)                                        \
  do {                                                         \
    int rc_ = ::hqkv::check_cuda((call), #call);               \
    if (rc_) return rc_;                                       \
  } while (0)

#define HQKV_LAUNCH_CHECK(name) HQKV_CUDA((cudaGetLastError()))

// ---- bounds-check build (-DHQKV_CHECKS) --------------------------------------------------------
// Every index that comes out of a caller-supplied list (logical positions of the decode, token ids of the
// flush plan) is range-checked before it addresses memory; a violation is counted in a device counter of
// the translation unit and the access is skipped - no trap.  hqkv_check_failures() reports the sum.  The
// regular build compiles the checks away.  (The stand-in for compute-sanitizer's memcheck on small cases.)
#ifdef HQKV_CHECKS
#define HQKV_CHECKS_ENABLED 1
#define HQKV_DEFINE_CHECK_COUNTER static __device__ unsigned int g_check_failures = 0u;
#define HQKV_INDEX_OK(idx, bound) \
  ((static_cast<unsigned long long>(idx) < static_cast<unsigned long long>(bound)) ? true : (atomicAdd(&g_check_failures, 1u), false))
#else
#define HQKV_CHECKS_ENABLED 0
#define HQKV_DEFINE_CHECK_COUNTER
#define HQKV_INDEX_OK(idx, bound) true
#endif
unsigned decode_check_failures(bool reset);  // decode.cu
unsigned policy_check_failures(bool reset);  // policy.cu

static inline bool valid_group(int g) { return g == 32 || g == 64 || g == 128; }
static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- fp16 arithmetic with one rounding per operation -----------------------------------------
// "One torch op on fp16 tensors": widen to fp32, operate, round to nearest-even fp16.  The
// intrinsics with explicit rounding keep the compiler from contracting separate operations
// into an FMA, which would drop an intermediate rounding.
__device__ __forceinline__ __half h_sub(__half a, __half b) {
  return __float2half_rn(__fsub_rn(__half2float(a), __half2float(b)));
}
__device__ __forceinline__ __half h_div(__half a, __half b) {
  return __float2half_rn(__fdiv_rn(__half2float(a), __half2float(b)));
}
__device__ __forceinline__ __half h_divf(__half a, float b) {
  return __float2half_rn(__fdiv_rn(__half2float(a), b));
}
__device__ __forceinline__ __half h_mul(__half a, __half b) {
  return __float2half_rn(__fmul_rn(__half2float(a), __half2float(b)));
}
__device__ __forceinline__ __half h_add(__half a, __half b) {
  return __float2half_rn(__fadd_rn(__half2float(a), __half2float(b)));
}

// Code of one element: clamp(half(half(x - mn) / scale), 0, levels) rounded half-to-even.
// A NaN quotient (constant group: scale == 0) gives code 0, as the float->int conversion on
// the GPU does for the reference.
__device__ __forceinline__ uint32_t quant_code(__half x, __half mn, __half scale, float levels) {
  float u = __half2float(h_div(h_sub(x, mn), scale));
  u = fminf(fmaxf(u, 0.f), levels);  // fmaxf(NaN, 0) == 0
  return static_cast<uint32_t>(__float2int_rn(u));
}

// The same code for many elements of one group.  x - mn with the native fp16 subtract (one rounding
// of the exact difference equals the two roundings of "widen, subtract, narrow": fp32 carries 2*11 + 2
// bits).  The quotient by Markstein's sequence: r = RN(1/scale) once per group, q0 = RN(d*r),
// e = d - q0*scale (exact in one FMA), q1 = RN(q0 + e*r) is the correctly rounded fp32 quotient (the
// scale has an 11-bit significand, never the all-ones fp32 significand the theorem excludes), so
// half(q1) is what h_div returns; three FP32 instructions per element instead of a full IEEE divide.
// A NaN or infinite intermediate (scale 0 or inf) ends as code 0 exactly as in quant_code.
struct QuantGroup {
  __half mn;
  float scale, rcp, levels;
};
__device__ __forceinline__ QuantGroup quant_group(__half mn, __half scale, float levels) {
  QuantGroup g;
  g.mn = mn;
  g.scale = __half2float(scale);
  g.rcp = __frcp_rn(g.scale);
  g.levels = levels;
  return g;
}
__device__ __forceinline__ float quant_quotient(float d, const QuantGroup& g) {
  const float q0 = __fmul_rn(d, g.rcp);
  const float e = __fmaf_rn(-q0, g.scale, d);
  return __fmaf_rn(e, g.rcp, q0);
}
__device__ __forceinline__ uint32_t quant_code_fast(__half x, const QuantGroup& g) {
  float u = __half2float(__float2half_rn(quant_quotient(__half2float(__hsub(x, g.mn)), g)));
  u = fminf(fmaxf(u, 0.f), g.levels);  // fmaxf(NaN, 0) == 0
  return static_cast<uint32_t>(__float2int_rn(u));
}
// two elements (low half in group g, high half in group gh): codes in bits [0,10) and [16,26)
__device__ __forceinline__ uint32_t quant_code_fast2(__half2 x, const QuantGroup& g, const QuantGroup& gh) {
  const float2 d = __half22float2(__hsub2(x, __halves2half2(g.mn, gh.mn)));
  __half2 u = __floats2half2_rn(quant_quotient(d.x, g), quant_quotient(d.y, gh));
  u = __hmin2(__hmax2(u, __float2half2_rn(0.f)), __float2half2_rn(g.levels));  // max(NaN, 0) == 0
  u = __hadd2(u, __float2half2_rn(1024.f));  // 1024 + rint(u): fp16 has unit spacing there, ties to even
  return *reinterpret_cast<uint32_t*>(&u) & 0x03FF03FFu;
}
__device__ __forceinline__ uint32_t quant_code_fast2(__half2 x, const QuantGroup& g) { return quant_code_fast2(x, g, g); }

// scale = half(half(mx - mn) / levels)
__device__ __forceinline__ __half quant_scale(__half mn, __half mx, float levels) {
  return h_divf(h_sub(mx, mn), levels);
}

// Two-rounding dequantisation: half(half(code * scale) + mn).
__device__ __forceinline__ __half dequant_2r(uint32_t code, __half scale, __half mn) {
  return h_add(h_mul(__uint2half_rn(code), scale), mn);
}

// Gaussian-codebook codec at 1 bit.  std and mean of a group are torch.std_mean (unbiased) of its fp16
// values: computed in fp64 (the sum of up to 128 fp16 values is exact there) and rounded once to fp16.
__device__ __forceinline__ __half normal1_sd(double sum_sq_dev, int group) {
  return __double2half(sqrt(sum_sq_dev / (group - 1)));
}
// code = 1 where half(half(x - mean) / std) > 0 (decision bounds [0, inf]); a NaN quotient gives 0
__device__ __forceinline__ uint32_t normal1_code(__half x, __half mean, __half sd) {
  return __half2float(h_div(h_sub(x, mean), sd)) > 0.f ? 1u : 0u;
}
#define HQKV_NORMAL1_CENTER 0.67448974f

__device__ __forceinline__ __half h_min(__half a, __half b) { return __half2float(b) < __half2float(a) ? b : a; }
__device__ __forceinline__ __half h_max(__half a, __half b) { return __half2float(b) > __half2float(a) ? b : a; }

}  // namespace hqkv
