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

// scale = half(half(mx - mn) / levels)
__device__ __forceinline__ __half quant_scale(__half mn, __half mx, float levels) {
  return h_divf(h_sub(mx, mn), levels);
}

// Two-rounding dequantisation: half(half(code * scale) + mn).
__device__ __forceinline__ __half dequant_2r(uint32_t code, __half scale, __half mn) {
  return h_add(h_mul(__uint2half_rn(code), scale), mn);
}

__device__ __forceinline__ __half h_min(__half a, __half b) { return __half2float(b) < __half2float(a) ? b : a; }
__device__ __forceinline__ __half h_max(__half a, __half b) { return __half2float(b) > __half2float(a) ? b : a; }

}  // namespace hqkv
