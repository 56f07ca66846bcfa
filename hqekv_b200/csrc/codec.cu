// Group quantise + bit-pack, unpack + dequantise (sm_100a).
//
// HBM-bound elementwise work: every element is read once and every packed word written once.
// Algorithmic bytes per element: 2 in, bits/8 + 4/group out.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace hqkv {

// ------------------------------------------------------------------------------------------------
// error plumbing shared by all translation units
// ------------------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  return fail(HQKV_E_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
}

// ------------------------------------------------------------------------------------------------
// Row path: groups are contiguous in memory (t_stride == 1).  One thread owns 8 consecutive
// elements (one 16-byte load when aligned), GROUP/8 adjacent lanes own one group.
// ------------------------------------------------------------------------------------------------
template <int BITS, int GROUP>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const __half* __restrict__ x, int64_t rows, int64_t T,
                                                            int64_t inner, int64_t outer_stride,
                                                            int64_t inner_stride, bool vec_ok,
                                                            uint32_t* __restrict__ code, __half* __restrict__ scale,
                                                            __half* __restrict__ mn_out) {
  constexpr int LPG = GROUP / 8;  // lanes per group
  const float levels = static_cast<float>((1 << BITS) - 1);
  const int64_t units_per_row = T / 8;
  const int64_t total_units = rows * units_per_row;
  // all lanes of a warp take part in the shuffles: iterate in whole-warp steps; two units per thread and step, both
  // loads issued before either is worked on (one 16-byte load in flight per thread did not cover the memory latency)
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t n_iter = (total_units + 2 * stride - 1) / (2 * stride);
  // packed source (the usual case): unit u is elements [8u, 8u+8) and no 64-bit division is needed;
  // (row*T + t0) below is 8u either way
  const bool packed = inner_stride == T && outer_stride == inner * T;
  const int lane = threadIdx.x & 31;
  for (int64_t it = 0; it < n_iter; ++it) {
    __half v[2][8];
    int64_t row[2], t0[2];
    bool live[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int64_t u = (2 * it + k) * stride + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
      live[k] = u < total_units;
      row[k] = 0;
      t0[k] = live[k] ? u * 8 : 0;
      if (!packed && live[k]) {
        row[k] = u / units_per_row;
        t0[k] = (u % units_per_row) * 8;
      }
      if (live[k]) {
        const __half* src = packed ? x + t0[k] : x + (row[k] / inner) * outer_stride + (row[k] % inner) * inner_stride + t0[k];
        if (vec_ok) {
          *reinterpret_cast<uint4*>(v[k]) = *reinterpret_cast<const uint4*>(src);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[k][i] = src[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[k][i] = __float2half(0.f);
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      // min / max of the group on half2 pairs (NaN propagates, as in torch.min / torch.max)
      const __half2* v2 = reinterpret_cast<const __half2*>(v[k]);
      __half2 lo2 = __hmin2_nan(__hmin2_nan(v2[0], v2[1]), __hmin2_nan(v2[2], v2[3]));
      __half2 hi2 = __hmax2_nan(__hmax2_nan(v2[0], v2[1]), __hmax2_nan(v2[2], v2[3]));
#pragma unroll
      for (int off = 1; off < LPG; off <<= 1) {
        lo2 = __hmin2_nan(lo2, __shfl_xor_sync(0xffffffffu, lo2, off));
        hi2 = __hmax2_nan(hi2, __shfl_xor_sync(0xffffffffu, hi2, off));
      }
      lo2 = __hmin2_nan(lo2, __lowhigh2highlow(lo2));
      hi2 = __hmax2_nan(hi2, __lowhigh2highlow(hi2));
      const __half lo = __low2half(lo2), hi = __low2half(hi2);
      const __half sc = quant_scale(lo, hi, levels);
      const QuantGroup qg = quant_group(lo, sc, levels);
      uint64_t part = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t c2 = quant_code_fast2(v2[i], qg);
        part |= static_cast<uint64_t>((c2 & 0xFFFFu) | ((c2 >> 16) << BITS)) << (2 * i * BITS);
      }
      const int64_t out_bit = (row[k] * T + t0[k]) * BITS;  // bit offset of this unit in the packed row-major stream
      if constexpr (BITS == 8) {
        if (live[k]) {
          uint2 w;
          w.x = static_cast<uint32_t>(part);
          w.y = static_cast<uint32_t>(part >> 32);
          *reinterpret_cast<uint2*>(code + out_bit / 32) = w;
        }
      } else if constexpr (BITS == 4) {
        if (live[k]) code[out_bit / 32] = static_cast<uint32_t>(part);
      } else {
        // 2 bits: 16 bits per thread, two lanes per word; 1 bit: 8 bits per thread, four lanes per word
        constexpr int LPW = 32 / (8 * BITS);  // lanes per word
        uint32_t w = static_cast<uint32_t>(part);
#pragma unroll
        for (int off = 1; off < LPW; off <<= 1) {
          const uint32_t other = __shfl_down_sync(0xffffffffu, w, off);
          w |= other << (8 * BITS * off);
        }
        if (live[k] && (lane % LPW) == 0) code[out_bit / 32] = w;
      }
      if (live[k] && (lane % LPG) == 0) {
        const int64_t gi = (row[k] * T + t0[k]) / GROUP;
        scale[gi] = sc;
        mn_out[gi] = lo;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Column path (K): source is token-major [outer, T, inner] and is quantised as [outer*inner, T] with
// groups of GROUP tokens per channel — the transposed view, never materialised.  One thread owns
// one channel; a warp reads 64 contiguous bytes per token.  Two passes over the group (the second
// hits L1/L2): min/max, then codes.
// ------------------------------------------------------------------------------------------------
template <int BITS>
__global__ void __launch_bounds__(128) quantize_cols_kernel(const __half* __restrict__ x, int64_t inner, int64_t T,
                                                            int64_t outer_stride, int64_t t_stride, int group,
                                                            uint32_t* __restrict__ code, __half* __restrict__ scale,
                                                            __half* __restrict__ mn_out) {
  constexpr int FPI = 32 / BITS;
  const float levels = static_cast<float>((1 << BITS) - 1);
  const int64_t d = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
  if (d >= inner) return;
  const int64_t o = blockIdx.z;
  const int64_t gi = blockIdx.x;  // group index along T
  const __half* src = x + o * outer_stride + d + gi * group * t_stride;
  __half lo = src[0], hi = src[0];
  for (int t = 1; t < group; ++t) {
    const __half v = src[t * t_stride];
    lo = h_min(lo, v);
    hi = h_max(hi, v);
  }
  const __half sc = quant_scale(lo, hi, levels);
  const QuantGroup qg = quant_group(lo, sc, levels);
  const int64_t row = o * inner + d;
  const int64_t W = T / FPI;
  uint32_t* dst = code + row * W + gi * (group / FPI);
  for (int w = 0; w < group / FPI; ++w) {
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < FPI; ++i) word |= quant_code_fast(src[(w * FPI + i) * t_stride], qg) << (i * BITS);
    dst[w] = word;
  }
  const int64_t G = T / group;
  scale[row * G + gi] = sc;
  mn_out[row * G + gi] = lo;
}

// Same, two adjacent channels per thread (4-byte loads, half2 arithmetic): the usual case of an even,
// 4-byte aligned channel count.  A warp reads 128 contiguous bytes per token.
template <int BITS>
__global__ void __launch_bounds__(64) quantize_cols2_kernel(const __half* __restrict__ x, int64_t inner, int64_t T,
                                                            int64_t outer_stride, int64_t t_stride, int group,
                                                            uint32_t* __restrict__ code, __half* __restrict__ scale,
                                                            __half* __restrict__ mn_out) {
  constexpr int FPI = 32 / BITS;
  const float levels = static_cast<float>((1 << BITS) - 1);
  const int64_t d = 2 * (static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x);
  if (d >= inner) return;
  const int64_t o = blockIdx.z;
  const int64_t gi = blockIdx.x;  // group index along T
  const __half* src = x + o * outer_stride + d + gi * group * t_stride;
  auto at = [&](int t) { return *reinterpret_cast<const __half2*>(src + t * t_stride); };
  __half2 lo = at(0), hi = lo;
#pragma unroll 8
  for (int t = 1; t < group; ++t) {
    const __half2 v = at(t);
    lo = __hmin2_nan(lo, v);
    hi = __hmax2_nan(hi, v);
  }
  const __half sc0 = quant_scale(__low2half(lo), __low2half(hi), levels);
  const __half sc1 = quant_scale(__high2half(lo), __high2half(hi), levels);
  const QuantGroup g0 = quant_group(__low2half(lo), sc0, levels), g1 = quant_group(__high2half(lo), sc1, levels);
  const int64_t row = o * inner + d;
  const int64_t W = T / FPI;
  uint32_t* dst0 = code + row * W + gi * (group / FPI);
  uint32_t* dst1 = dst0 + W;
  for (int w = 0; w < group / FPI; ++w) {
    uint32_t word0 = 0, word1 = 0;
#pragma unroll
    for (int i = 0; i < FPI; ++i) {
      const uint32_t c2 = quant_code_fast2(at(w * FPI + i), g0, g1);
      word0 |= (c2 & 0xFFFFu) << (i * BITS);
      word1 |= (c2 >> 16) << (i * BITS);
    }
    dst0[w] = word0;
    dst1[w] = word1;
  }
  const int64_t G = T / group;
  scale[row * G + gi] = sc0;
  mn_out[row * G + gi] = __low2half(lo);
  scale[(row + 1) * G + gi] = sc1;
  mn_out[(row + 1) * G + gi] = __high2half(lo);
}

// The same for groups of 32 tokens, a tile of 8 groups x 128 channels per CTA.  The kernel above writes every word
// with its own 4-byte store one code row apart from its neighbour's and reads every value twice; here a thread
// keeps the 32 values of a group in registers (one pass), the tile's words and scale / zero halfs meet in shared
// memory, and the CTA stores each channel's 8 groups as one contiguous run (32 x BITS bytes of codes, 16 bytes of
// scales), consecutive threads on consecutive words.  256 threads: thread = (channel pair cp, group lane gl), groups
// gl and gl + 4 of the tile.  Arithmetic and results are those of the kernel above.
constexpr int QT_GROUPS = 8;     // groups per tile
constexpr int QT_CH = 128;       // channels per tile
template <int BITS>
__global__ void __launch_bounds__(256) quantize_cols_tile_kernel(const __half* __restrict__ x, int64_t inner, int64_t T,
                                                                 int64_t outer_stride, int64_t t_stride,
                                                                 uint32_t* __restrict__ code, __half* __restrict__ scale,
                                                                 __half* __restrict__ mn_out) {
  constexpr int GROUP = 32;
  constexpr int FPI = 32 / BITS;          // codes per word
  constexpr int WPG = GROUP / FPI;        // words per group = BITS
  constexpr int ROW = QT_GROUPS * WPG + 1;  // words per staged channel row (+1: rows land in different banks)
  __shared__ uint32_t s_words[QT_CH * ROW];
  __shared__ __half s_scale[QT_CH * QT_GROUPS], s_min[QT_CH * QT_GROUPS];
  const float levels = static_cast<float>((1 << BITS) - 1);
  const int tid = threadIdx.x, cp = tid & 63, gl = tid >> 6;
  const int64_t G = T / GROUP;
  const int64_t g_first = static_cast<int64_t>(blockIdx.x) * QT_GROUPS;
  const int ngr = static_cast<int>(G - g_first < QT_GROUPS ? G - g_first : QT_GROUPS);
  const int64_t d0 = static_cast<int64_t>(blockIdx.y) * QT_CH;
  const int nch = static_cast<int>(inner - d0 < QT_CH ? inner - d0 : QT_CH);  // even: the host checks inner % 2 == 0
  const int64_t o = blockIdx.z;
  const int ch = 2 * cp;
  if (ch < nch) {
    for (int gq = gl; gq < ngr; gq += 4) {
      const __half* src = x + o * outer_stride + d0 + ch + (g_first + gq) * GROUP * t_stride;
      __half2 v[GROUP];
#pragma unroll
      for (int t = 0; t < GROUP; ++t) v[t] = *reinterpret_cast<const __half2*>(src + t * t_stride);
      __half2 lo = v[0], hi = v[0];
#pragma unroll
      for (int t = 1; t < GROUP; ++t) {
        lo = __hmin2_nan(lo, v[t]);
        hi = __hmax2_nan(hi, v[t]);
      }
      const __half sc0 = quant_scale(__low2half(lo), __low2half(hi), levels);
      const __half sc1 = quant_scale(__high2half(lo), __high2half(hi), levels);
      const QuantGroup g0 = quant_group(__low2half(lo), sc0, levels), g1 = quant_group(__high2half(lo), sc1, levels);
      uint32_t* w0 = s_words + ch * ROW + gq * WPG;
      uint32_t* w1 = w0 + ROW;
#pragma unroll
      for (int w = 0; w < WPG; ++w) {
        uint32_t word0 = 0, word1 = 0;
#pragma unroll
        for (int i = 0; i < FPI; ++i) {
          const uint32_t c2 = quant_code_fast2(v[w * FPI + i], g0, g1);
          word0 |= (c2 & 0xFFFFu) << (i * BITS);
          word1 |= (c2 >> 16) << (i * BITS);
        }
        w0[w] = word0;
        w1[w] = word1;
      }
      s_scale[ch * QT_GROUPS + gq] = sc0;
      s_min[ch * QT_GROUPS + gq] = __low2half(lo);
      s_scale[(ch + 1) * QT_GROUPS + gq] = sc1;
      s_min[(ch + 1) * QT_GROUPS + gq] = __high2half(lo);
    }
  }
  __syncthreads();
  const int64_t row0 = o * inner + d0;
  const int64_t W = T / FPI;
  const int wpr = ngr * WPG;  // words of one channel row in this tile
  for (int i = tid; i < nch * wpr; i += 256) {
    const int r = i / wpr, w = i - r * wpr;
    code[(row0 + r) * W + g_first * WPG + w] = s_words[r * ROW + w];
  }
  for (int i = tid; i < nch * ngr; i += 256) {
    const int r = i / ngr, g = i - r * ngr;
    scale[(row0 + r) * G + g_first + g] = s_scale[r * QT_GROUPS + g];
    mn_out[(row0 + r) * G + g_first + g] = s_min[r * QT_GROUPS + g];
  }
}

// ------------------------------------------------------------------------------------------------
// unpack + two-rounding dequantise; one thread writes 8 consecutive fp16 values (16 bytes)
// ------------------------------------------------------------------------------------------------
template <int BITS>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint32_t* __restrict__ code,
                                                         const __half* __restrict__ scale,
                                                         const __half* __restrict__ mn, int64_t n_units, int group,
                                                         __half* __restrict__ out) {
  const int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t e0 = u * 8;  // first element (row-major over [rows, T]; T is a multiple of the group, group of 8)
  const int64_t bit0 = e0 * BITS;
  uint64_t bits = code[bit0 / 32];
  if (BITS == 8) bits |= static_cast<uint64_t>(code[bit0 / 32 + 1]) << 32;
  bits >>= (bit0 % 32);
  const __half sc = scale[e0 / group], z = mn[e0 / group];
  __half v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = dequant_2r(static_cast<uint32_t>(bits >> (i * BITS)) & ((1u << BITS) - 1), sc, z);
  *reinterpret_cast<uint4*>(out + e0) = *reinterpret_cast<const uint4*>(v);
}

template <int BITS>
__global__ void __launch_bounds__(256) pack_kernel(const int32_t* __restrict__ codes, int64_t n_words,
                                                   uint32_t* __restrict__ words) {
  constexpr int FPI = 32 / BITS;
  const int64_t w = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  uint32_t word = 0;
#pragma unroll
  for (int i = 0; i < FPI; ++i) word |= static_cast<uint32_t>(codes[w * FPI + i]) << (i * BITS);
  words[w] = word;
}

template <int BITS>
__global__ void __launch_bounds__(256) unpack_kernel(const uint32_t* __restrict__ words, int64_t n_words,
                                                     __half* __restrict__ out) {
  constexpr int FPI = 32 / BITS;
  const int64_t w = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  const uint32_t word = words[w];
#pragma unroll
  for (int i = 0; i < FPI; ++i) out[w * FPI + i] = __uint2half_rn((word >> (i * BITS)) & ((1u << BITS) - 1));
}

template <int BITS>
static int launch_quant_rows(const __half* x, int64_t rows, int64_t T, int64_t inner, int64_t os, int64_t is,
                             int group, bool vec_ok, uint32_t* code, __half* scale, __half* mn, cudaStream_t st) {
  const int64_t units = rows * (T / 8);
  const int threads = 256;
  // two units per thread and step; beyond 64 CTAs per SM the grid strides, sized so that every step is full
  // (a last step that only some CTAs take costs a whole step's time)
  const int64_t per_step = 2 * threads;
  const int64_t steps = ceil_div(units, per_step * 148 * 64);
  int64_t blocks = ceil_div(units, per_step * (steps < 1 ? 1 : steps));
  if (blocks < 1) blocks = 1;
  switch (group) {
    case 32:
      quantize_rows_kernel<BITS, 32><<<blocks, threads, 0, st>>>(x, rows, T, inner, os, is, vec_ok, code, scale, mn);
      break;
    case 64:
      quantize_rows_kernel<BITS, 64><<<blocks, threads, 0, st>>>(x, rows, T, inner, os, is, vec_ok, code, scale, mn);
      break;
    default:
      quantize_rows_kernel<BITS, 128><<<blocks, threads, 0, st>>>(x, rows, T, inner, os, is, vec_ok, code, scale, mn);
      break;
  }
  return 0;
}


// ------------------------------------------------------------------------------------------------
// Gaussian-codebook codec at 1 bit (the low tier of 'high_uniform_group_low_normal_group')
// ------------------------------------------------------------------------------------------------
// One thread per group, two passes over its `group` elements.  std and mean are the unbiased
// torch.std_mean of the group computed in fp64 (the sum of fp16 values is exact there) and rounded ONCE
// to fp16, which is what torch returns for fp16 input; then (x - mean) / std in fp16 with a rounding after
// each step, code = 1 where the quotient is > 0 (decision bounds [0, inf]; NaN gives 0).
__global__ void __launch_bounds__(128) normal1_quantize_kernel(const __half* __restrict__ x, int64_t rows, int64_t T,
                                                               int64_t inner, int64_t outer_stride, int64_t inner_stride,
                                                               int64_t t_stride, int group, uint32_t* __restrict__ code,
                                                               __half* __restrict__ std_out, __half* __restrict__ mean_out) {
  const int64_t G = T / group;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= rows * G) return;
  const int64_t row = gid / G, gi = gid - row * G;
  const __half* src = x + (row / inner) * outer_stride + (row % inner) * inner_stride + gi * group * t_stride;
  double sum = 0.0;
  for (int t = 0; t < group; ++t) sum += static_cast<double>(__half2float(src[t * t_stride]));
  const double mean64 = sum / group;
  double ss = 0.0;
  for (int t = 0; t < group; ++t) {
    const double d = static_cast<double>(__half2float(src[t * t_stride])) - mean64;
    ss += d * d;
  }
  const __half mean = __double2half(mean64);
  const __half sd = normal1_sd(ss, group);
  uint32_t* dst = code + (row * T + gi * group) / 32;
  for (int w = 0; w < group / 32; ++w) {
    uint32_t word = 0;
    for (int i = 0; i < 32; ++i) {
      word |= normal1_code(src[(w * 32 + i) * t_stride], mean, sd) << i;
    }
    dst[w] = word;
  }
  std_out[gid] = sd;
  mean_out[gid] = mean;
}

// x = half(half(center[code] * std) + mean), center = +-fp16(0.67448974); one thread per packed word
__global__ void __launch_bounds__(256) normal1_dequantize_kernel(const uint32_t* __restrict__ code,
                                                                 const __half* __restrict__ sd,
                                                                 const __half* __restrict__ mean, int64_t n_words,
                                                                 int group, __half* __restrict__ out) {
  const int64_t w = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  const uint32_t word = code[w];
  const int64_t gi = (w * 32) / group;
  const __half s = sd[gi], m = mean[gi];
  const __half cpos = __float2half_rn(HQKV_NORMAL1_CENTER), cneg = __float2half_rn(-HQKV_NORMAL1_CENTER);
  __half* dst = out + w * 32;
  for (int i = 0; i < 32; ++i) dst[i] = h_add(h_mul((word >> i) & 1u ? cpos : cneg, s), m);
}

}  // namespace hqkv

using namespace hqkv;

extern "C" const char* hqkv_last_error(void) { return g_err; }
extern "C" int hqkv_version(void) { return 100; }
#ifndef HQKV_BUILD_ID
#define HQKV_BUILD_ID "unstamped"
#endif
// the marker lets a build script read the stamp out of the file without loading the library
static const char g_build_stamp[] = "HQKV_BUILD_ID=" HQKV_BUILD_ID;
extern "C" const char* hqkv_build_id(void) { return g_build_stamp + 14; }

extern "C" int hqkv_quantize_pack(const void* x, int64_t rows, int64_t T, int64_t inner, int64_t outer_stride,
                                  int64_t inner_stride, int64_t t_stride, int group, int bits, void* code,
                                  void* scale, void* mn, void* stream) {
  HQKV_REQUIRE(bits == 8 || bits == 4 || bits == 2 || bits == 1, "quantize_pack: bits must be 8, 4, 2 or 1 (got %d)", bits);
  HQKV_REQUIRE(valid_group(group), "quantize_pack: group must be 32, 64 or 128 (got %d)", group);
  HQKV_REQUIRE(rows >= 0 && T >= 0 && inner > 0, "quantize_pack: negative size");
  HQKV_REQUIRE(T % group == 0, "quantize_pack: T (%lld) is not a multiple of the group size %d", (long long)T, group);
  HQKV_REQUIRE(rows % inner == 0, "quantize_pack: rows (%lld) is not a multiple of inner (%lld)", (long long)rows,
               (long long)inner);
  if (rows == 0 || T == 0) return HQKV_OK;
  HQKV_REQUIRE(x && code && scale && mn, "quantize_pack: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half* xs = static_cast<const __half*>(x);
  uint32_t* c = static_cast<uint32_t*>(code);
  __half* s = static_cast<__half*>(scale);
  __half* m = static_cast<__half*>(mn);
  if (t_stride == 1) {
    const bool vec_ok = aligned(x, 16) && outer_stride % 8 == 0 && inner_stride % 8 == 0;
    switch (bits) {
      case 8: launch_quant_rows<8>(xs, rows, T, inner, outer_stride, inner_stride, group, vec_ok, c, s, m, st); break;
      case 4: launch_quant_rows<4>(xs, rows, T, inner, outer_stride, inner_stride, group, vec_ok, c, s, m, st); break;
      case 2: launch_quant_rows<2>(xs, rows, T, inner, outer_stride, inner_stride, group, vec_ok, c, s, m, st); break;
      default: launch_quant_rows<1>(xs, rows, T, inner, outer_stride, inner_stride, group, vec_ok, c, s, m, st); break;
    }
  } else if (inner_stride == 1) {
    const int64_t outer = rows / inner;
    HQKV_REQUIRE(outer <= 65535 && ceil_div(inner, 128) <= 65535, "quantize_pack: too many rows for the column path");
    dim3 grid(static_cast<unsigned>(T / group), static_cast<unsigned>(ceil_div(inner, 128)),
              static_cast<unsigned>(outer));
    if (group == 32 && inner % 2 == 0 && aligned(x, 4) && outer_stride % 2 == 0 && t_stride % 2 == 0) {
      dim3 gridt(static_cast<unsigned>(ceil_div(T / group, QT_GROUPS)), static_cast<unsigned>(ceil_div(inner, QT_CH)),
                 static_cast<unsigned>(outer));
      switch (bits) {
        case 8: quantize_cols_tile_kernel<8><<<gridt, 256, 0, st>>>(xs, inner, T, outer_stride, t_stride, c, s, m); break;
        case 4: quantize_cols_tile_kernel<4><<<gridt, 256, 0, st>>>(xs, inner, T, outer_stride, t_stride, c, s, m); break;
        case 2: quantize_cols_tile_kernel<2><<<gridt, 256, 0, st>>>(xs, inner, T, outer_stride, t_stride, c, s, m); break;
        default: quantize_cols_tile_kernel<1><<<gridt, 256, 0, st>>>(xs, inner, T, outer_stride, t_stride, c, s, m); break;
      }
    } else if (inner % 2 == 0 && aligned(x, 4) && outer_stride % 2 == 0 && t_stride % 2 == 0) {
      dim3 grid2(static_cast<unsigned>(T / group), static_cast<unsigned>(ceil_div(inner, 128)),
                 static_cast<unsigned>(outer));
      switch (bits) {
        case 8: quantize_cols2_kernel<8><<<grid2, 64, 0, st>>>(xs, inner, T, outer_stride, t_stride, group, c, s, m); break;
        case 4: quantize_cols2_kernel<4><<<grid2, 64, 0, st>>>(xs, inner, T, outer_stride, t_stride, group, c, s, m); break;
        case 2: quantize_cols2_kernel<2><<<grid2, 64, 0, st>>>(xs, inner, T, outer_stride, t_stride, group, c, s, m); break;
        default: quantize_cols2_kernel<1><<<grid2, 64, 0, st>>>(xs, inner, T, outer_stride, t_stride, group, c, s, m); break;
      }
    } else
    switch (bits) {
      case 8: quantize_cols_kernel<8><<<grid, 128, 0, st>>>(xs, inner, T, outer_stride, t_stride, group, c, s, m); break;
      case 4: quantize_cols_kernel<4><<<grid, 128, 0, st>>>(xs, inner, T, outer_stride, t_stride, group, c, s, m); break;
      case 2: quantize_cols_kernel<2><<<grid, 128, 0, st>>>(xs, inner, T, outer_stride, t_stride, group, c, s, m); break;
      default: quantize_cols_kernel<1><<<grid, 128, 0, st>>>(xs, inner, T, outer_stride, t_stride, group, c, s, m); break;
    }
  } else {
    return fail(HQKV_E_INVALID, "quantize_pack: unsupported strides (need t_stride == 1 or inner_stride == 1)");
  }
  HQKV_LAUNCH_CHECK("quantize_pack");
  return HQKV_OK;
}

extern "C" int hqkv_dequantize_unpack(const void* code, const void* scale, const void* mn, int64_t rows, int64_t T,
                                      int group, int bits, void* out, void* stream) {
  HQKV_REQUIRE(bits == 8 || bits == 4 || bits == 2 || bits == 1, "dequantize_unpack: bits must be 8, 4, 2 or 1");
  HQKV_REQUIRE(valid_group(group), "dequantize_unpack: group must be 32, 64 or 128");
  HQKV_REQUIRE(rows >= 0 && T >= 0 && T % group == 0, "dequantize_unpack: T is not a multiple of the group size");
  if (rows == 0 || T == 0) return HQKV_OK;
  HQKV_REQUIRE(code && scale && mn && out, "dequantize_unpack: null pointer");
  HQKV_REQUIRE(aligned(out, 16), "dequantize_unpack: output must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t units = rows * T / 8;
  const unsigned blocks = static_cast<unsigned>(ceil_div(units, 256));
  const uint32_t* c = static_cast<const uint32_t*>(code);
  const __half* s = static_cast<const __half*>(scale);
  const __half* m = static_cast<const __half*>(mn);
  __half* o = static_cast<__half*>(out);
  switch (bits) {
    case 8: dequantize_kernel<8><<<blocks, 256, 0, st>>>(c, s, m, units, group, o); break;
    case 4: dequantize_kernel<4><<<blocks, 256, 0, st>>>(c, s, m, units, group, o); break;
    case 2: dequantize_kernel<2><<<blocks, 256, 0, st>>>(c, s, m, units, group, o); break;
    default: dequantize_kernel<1><<<blocks, 256, 0, st>>>(c, s, m, units, group, o); break;
  }
  HQKV_LAUNCH_CHECK("dequantize_unpack");
  return HQKV_OK;
}

extern "C" int hqkv_pack(const void* codes_i32, int64_t rows, int64_t T, int bits, void* words, void* stream) {
  HQKV_REQUIRE(bits == 8 || bits == 4 || bits == 2 || bits == 1, "pack: bits must be 8, 4, 2 or 1");
  HQKV_REQUIRE(rows >= 0 && T >= 0 && T % (32 / bits) == 0, "pack: T is not a multiple of 32/bits");
  const int64_t n_words = rows * T / (32 / bits);
  if (n_words == 0) return HQKV_OK;
  HQKV_REQUIRE(codes_i32 && words, "pack: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>(ceil_div(n_words, 256));
  const int32_t* c = static_cast<const int32_t*>(codes_i32);
  uint32_t* w = static_cast<uint32_t*>(words);
  switch (bits) {
    case 8: pack_kernel<8><<<blocks, 256, 0, st>>>(c, n_words, w); break;
    case 4: pack_kernel<4><<<blocks, 256, 0, st>>>(c, n_words, w); break;
    case 2: pack_kernel<2><<<blocks, 256, 0, st>>>(c, n_words, w); break;
    default: pack_kernel<1><<<blocks, 256, 0, st>>>(c, n_words, w); break;
  }
  HQKV_LAUNCH_CHECK("pack");
  return HQKV_OK;
}

extern "C" int hqkv_unpack(const void* words, int64_t rows, int64_t W, int bits, void* out_f16, void* stream) {
  HQKV_REQUIRE(bits == 8 || bits == 4 || bits == 2 || bits == 1, "unpack: bits must be 8, 4, 2 or 1");
  HQKV_REQUIRE(rows >= 0 && W >= 0, "unpack: negative size");
  const int64_t n_words = rows * W;
  if (n_words == 0) return HQKV_OK;
  HQKV_REQUIRE(words && out_f16, "unpack: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>(ceil_div(n_words, 256));
  const uint32_t* w = static_cast<const uint32_t*>(words);
  __half* o = static_cast<__half*>(out_f16);
  switch (bits) {
    case 8: unpack_kernel<8><<<blocks, 256, 0, st>>>(w, n_words, o); break;
    case 4: unpack_kernel<4><<<blocks, 256, 0, st>>>(w, n_words, o); break;
    case 2: unpack_kernel<2><<<blocks, 256, 0, st>>>(w, n_words, o); break;
    default: unpack_kernel<1><<<blocks, 256, 0, st>>>(w, n_words, o); break;
  }
  HQKV_LAUNCH_CHECK("unpack");
  return HQKV_OK;
}

extern "C" int hqkv_normal1_quantize_pack(const void* x, int64_t rows, int64_t T, int64_t inner, int64_t outer_stride,
                                          int64_t inner_stride, int64_t t_stride, int group, void* code, void* std_out,
                                          void* mean_out, void* stream) {
  HQKV_REQUIRE(valid_group(group), "normal1_quantize_pack: group size must be 32, 64 or 128 (got %d)", group);
  HQKV_REQUIRE(rows >= 0 && T >= 0 && inner > 0, "normal1_quantize_pack: negative size");
  HQKV_REQUIRE(T % group == 0, "normal1_quantize_pack: T (%lld) is not a multiple of the group size %d", (long long)T, group);
  HQKV_REQUIRE(rows % inner == 0, "normal1_quantize_pack: rows is not a multiple of inner");
  if (rows == 0 || T == 0) return HQKV_OK;
  HQKV_REQUIRE(x && code && std_out && mean_out, "normal1_quantize_pack: null pointer");
  const int64_t groups = rows * (T / group);
  normal1_quantize_kernel<<<static_cast<unsigned>(ceil_div(groups, 128)), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(x), rows, T, inner, outer_stride, inner_stride, t_stride, group,
      static_cast<uint32_t*>(code), static_cast<__half*>(std_out), static_cast<__half*>(mean_out));
  HQKV_LAUNCH_CHECK("normal1_quantize_pack");
  return HQKV_OK;
}

extern "C" int hqkv_normal1_dequantize_unpack(const void* code, const void* std_in, const void* mean_in, int64_t rows,
                                              int64_t T, int group, void* out, void* stream) {
  HQKV_REQUIRE(valid_group(group), "normal1_dequantize_unpack: group size must be 32, 64 or 128 (got %d)", group);
  HQKV_REQUIRE(rows >= 0 && T >= 0 && T % group == 0, "normal1_dequantize_unpack: bad sizes");
  if (rows == 0 || T == 0) return HQKV_OK;
  HQKV_REQUIRE(code && std_in && mean_in && out, "normal1_dequantize_unpack: null pointer");
  const int64_t n_words = rows * T / 32;
  normal1_dequantize_kernel<<<static_cast<unsigned>(ceil_div(n_words, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(code), static_cast<const __half*>(std_in), static_cast<const __half*>(mean_in),
      n_words, group, static_cast<__half*>(out));
  HQKV_LAUNCH_CHECK("normal1_dequantize_unpack");
  return HQKV_OK;
}
