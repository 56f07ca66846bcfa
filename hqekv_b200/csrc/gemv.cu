// Stand-alone batched GEMV over one packed tier in the reference's un-transposed layout (sm_100a):
//   out[b, hq, n] = sum_k fA[b, hq, k] * (scale[b, h, k, n/group] * code[b, h, k, n] + zero[b, h, k, n/group])
// qB is [B, nh_kv, K, N/fpi]: the contraction runs over ROWS, the packed axis is the output axis.
// One thread owns one packed word column (fpi outputs; half a word = 16 outputs at 1 bit) for all query
// heads of its kv head, so every word is read once (twice at 1 bit) and shared by the GQA group; K is split over the threadIdx.y slices of the CTA,
// which are added in index order through shared memory.  fp32 accumulation, fp16 result.
// NORMAL (1 bit only): the Gaussian-codebook tier, value = std * (code ? C : -C) + mean with the float32
// centre, as the reference's kernel evaluates it.
#include "common.cuh"

namespace hqkv {

constexpr int GEMV_WC = 32;     // word columns per CTA
constexpr int GEMV_KS = 8;      // K slices per CTA

template <int BITS, int REP, bool NORMAL>
__global__ void __launch_bounds__(GEMV_WC* GEMV_KS) gemv_group_kernel(
    const __half* __restrict__ fA, const uint32_t* __restrict__ qB, const __half* __restrict__ scales,
    const __half* __restrict__ zeros, int nh_q, int nh_kv, int64_t K, int64_t N, int gshift,
    __half* __restrict__ out) {
  constexpr int VPW = 32 / BITS;            // values per packed word
  constexpr int FPI = VPW > 16 ? 16 : VPW;  // outputs per thread
  constexpr int TPW = VPW / FPI;            // threads per word
  __shared__ float red[GEMV_KS][GEMV_WC][REP];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t W = N / FPI, G = N >> gshift;  // W = thread columns
  const int64_t wc = static_cast<int64_t>(blockIdx.x) * GEMV_WC + tx;
  const int bh = blockIdx.y, b = bh / nh_kv, h = bh - b * nh_kv;
  const bool live = wc < W;
  const __half* a = fA + (static_cast<int64_t>(b) * nh_q + h * REP) * K;
  const uint32_t* w = qB + static_cast<int64_t>(bh) * K * (W / TPW) + wc / TPW;
  const int shift0 = static_cast<int>(wc % TPW) * FPI * BITS;
  const int64_t gi = live ? (wc * FPI) >> gshift : 0;
  const __half* s = scales + static_cast<int64_t>(bh) * K * G + gi;
  const __half* z = zeros + static_cast<int64_t>(bh) * K * G + gi;
  float acc[REP][FPI];
#pragma unroll
  for (int r = 0; r < REP; ++r)
#pragma unroll
    for (int i = 0; i < FPI; ++i) acc[r][i] = 0.f;
  if (live) {
    for (int64_t k = ty; k < K; k += GEMV_KS) {
      const uint32_t word = w[k * (W / TPW)] >> shift0;
      const float sc = __half2float(s[k * G]), zp = __half2float(z[k * G]);
      float av[REP];
#pragma unroll
      for (int r = 0; r < REP; ++r) av[r] = __half2float(a[r * K + k]);
#pragma unroll
      for (int i = 0; i < FPI; ++i) {
        const uint32_t code = (word >> (i * BITS)) & ((1u << BITS) - 1u);
        const float wv = NORMAL ? fmaf(sc, code ? HQKV_NORMAL1_CENTER : -HQKV_NORMAL1_CENTER, zp)
                                : fmaf(sc, static_cast<float>(code), zp);
#pragma unroll
        for (int r = 0; r < REP; ++r) acc[r][i] = fmaf(av[r], wv, acc[r][i]);
      }
    }
  }
  // add the K slices in index order, one output value at a time to keep shared memory small
#pragma unroll
  for (int i = 0; i < FPI; ++i) {
#pragma unroll
    for (int r = 0; r < REP; ++r) red[ty][tx][r] = acc[r][i];
    __syncthreads();
    if (ty == 0 && live) {
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        float v = red[0][tx][r];
#pragma unroll
        for (int y = 1; y < GEMV_KS; ++y) v += red[y][tx][r];
        out[(static_cast<int64_t>(b) * nh_q + h * REP + r) * N + wc * FPI + i] = __float2half_rn(v);
      }
    }
    __syncthreads();
  }
}

template <int BITS, bool NORMAL = false>
static int launch_gemv(int rep, dim3 grid, cudaStream_t st, const __half* fA, const uint32_t* qB, const __half* s,
                       const __half* z, int nh_q, int nh_kv, int64_t K, int64_t N, int gshift, __half* out) {
  const dim3 block(GEMV_WC, GEMV_KS);
  switch (rep) {
    case 1: gemv_group_kernel<BITS, 1, NORMAL><<<grid, block, 0, st>>>(fA, qB, s, z, nh_q, nh_kv, K, N, gshift, out); break;
    case 2: gemv_group_kernel<BITS, 2, NORMAL><<<grid, block, 0, st>>>(fA, qB, s, z, nh_q, nh_kv, K, N, gshift, out); break;
    case 4: gemv_group_kernel<BITS, 4, NORMAL><<<grid, block, 0, st>>>(fA, qB, s, z, nh_q, nh_kv, K, N, gshift, out); break;
    case 8: gemv_group_kernel<BITS, 8, NORMAL><<<grid, block, 0, st>>>(fA, qB, s, z, nh_q, nh_kv, K, N, gshift, out); break;
    default: return fail(HQKV_E_INVALID, "gemv: nh_q/nh_kv must be 1, 2, 4 or 8 (got %d)", rep);
  }
  return HQKV_OK;
}

}  // namespace hqkv

using namespace hqkv;

static int gemv_entry(const void* fA, const void* qB, const void* scales, const void* zeros, int B, int nh_q, int nh_kv,
                      int64_t K, int64_t N, int group, int bits, bool normal, void* out, void* stream) {
  HQKV_REQUIRE(bits == 8 || bits == 4 || bits == 2 || bits == 1, "gemv: bits must be 8, 4, 2 or 1 (got %d)", bits);
  HQKV_REQUIRE(!normal || bits == 1, "gemv: the Gaussian-codebook codec is built at 1 bit only (got %d)", bits);
  HQKV_REQUIRE(valid_group(group), "gemv: group must be 32, 64 or 128 (got %d)", group);
  HQKV_REQUIRE(B > 0 && nh_q > 0 && nh_kv > 0 && nh_q % nh_kv == 0, "gemv: nh_q must be a positive multiple of nh_kv");
  HQKV_REQUIRE(K >= 0 && N >= 0 && N % group == 0, "gemv: N (%lld) is not a multiple of the group size %d", (long long)N,
               group);
  HQKV_REQUIRE(static_cast<int64_t>(B) * nh_kv <= 65535, "gemv: B*nh_kv too large");
  if (N == 0) return HQKV_OK;
  HQKV_REQUIRE(fA && qB && scales && zeros && out, "gemv: null pointer");
  int gshift = 0;
  while ((1 << gshift) < group) ++gshift;
  const int64_t W = N / (bits == 1 ? 16 : 32 / bits);  // thread columns
  const dim3 grid(static_cast<unsigned>(ceil_div(W, GEMV_WC)), static_cast<unsigned>(B * nh_kv));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rep = nh_q / nh_kv;
  int rc;
  const __half* a = static_cast<const __half*>(fA);
  const uint32_t* w = static_cast<const uint32_t*>(qB);
  const __half* s = static_cast<const __half*>(scales);
  const __half* z = static_cast<const __half*>(zeros);
  __half* o = static_cast<__half*>(out);
  if (bits == 8) rc = launch_gemv<8>(rep, grid, st, a, w, s, z, nh_q, nh_kv, K, N, gshift, o);
  else if (bits == 4) rc = launch_gemv<4>(rep, grid, st, a, w, s, z, nh_q, nh_kv, K, N, gshift, o);
  else if (bits == 2) rc = launch_gemv<2>(rep, grid, st, a, w, s, z, nh_q, nh_kv, K, N, gshift, o);
  else if (normal) rc = launch_gemv<1, true>(rep, grid, st, a, w, s, z, nh_q, nh_kv, K, N, gshift, o);
  else rc = launch_gemv<1>(rep, grid, st, a, w, s, z, nh_q, nh_kv, K, N, gshift, o);
  if (rc) return rc;
  HQKV_LAUNCH_CHECK("gemv_group");
  return HQKV_OK;
}

extern "C" int hqkv_gemv_uniform_group(const void* fA, const void* qB, const void* scales, const void* zeros, int B,
                                       int nh_q, int nh_kv, int64_t K, int64_t N, int group, int bits, void* out,
                                       void* stream) {
  return gemv_entry(fA, qB, scales, zeros, B, nh_q, nh_kv, K, N, group, bits, false, out, stream);
}

extern "C" int hqkv_gemv_normal_group(const void* fA, const void* qB, const void* stds, const void* means, int B,
                                      int nh_q, int nh_kv, int64_t K, int64_t N, int group, int bits, void* out,
                                      void* stream) {
  return gemv_entry(fA, qB, stds, means, B, nh_q, nh_kv, K, N, group, bits, true, out, stream);
}
