// Tile-level device code of the fused decode attention (sm_100a): what ONE WARP does with one tile of a
// K tier or a V tier.  The kernel that schedules the tiles lives in decode.cu.
//
// The roofline is HBM: every packed word, scale and zero is read exactly once per call and is shared
// by all query heads of its kv head (GQA).  At 2-4 bits there are 1.6-2.7 codes per byte; four query
// heads need four FMAs per code, more than the FP32 pipes can issue at HBM speed, so the dot products
// run on the tensor pipe (mma.sync m16n8k16, fp32 accumulation).  Tiles of codes are staged in shared
// memory with 16-byte cp.async and read back with ldmatrix.trans, which delivers the two K-neighbours
// of an A fragment in one register; the codes enter the MMA as fp16 subnormals (one AND per pair) and
// the scale is folded into the B operand, carried exactly as hi + lo.
#pragma once

#include <math.h>

#include "common.cuh"

namespace hqkv {

HQKV_DEFINE_CHECK_COUNTER

constexpr int D = 128;      // head dim
constexpr int MAX_REP = 8;  // query heads per kv head (n of the m16n8k16 tile)
constexpr float LOG2E = 1.4426950408889634f;

struct TierDev {
  const void* k_data;
  const __half* k_scale;
  const __half* k_zero;
  const int64_t* k_idx;
  const void* v_data;
  const __half* v_scale;
  const __half* v_zero;
  const int64_t* v_idx;
  int n_k, n_v;
  int bits;
  int normal;  // 1-bit tier in the Gaussian-codebook codec: value = std * (+-C) + mean, scale slots = std, zero = mean
  // work items of this tier per (batch, kv head): tokens per tile, tiles, weight of a tile, first weight
  int k_tile_tokens, k_tiles, k_w, k_w0;
  int v_tile_tokens, v_tiles, v_w, v_w0;
};

// ------------------------------------------------------------------------------------------------
// per-warp shared memory: byte offsets inside the warp's region
// ------------------------------------------------------------------------------------------------
// Every warp owns one region.  While it works on K tiles the region holds the tile's codes and its
// scale / zero rows; while it works on V tiles, the codes, the per-token scales and zeros, the staged
// exp(logit - max) rows and the warp's partial output.
constexpr int WS_CODES = 0;                      // 8192: codes of the current tile (plain K tiles: the logit tile)
constexpr int WS_K_S = 8192;                     // 2048: K scale rows [128 channels][8 halfs]
constexpr int WS_K_Z = WS_K_S + 2048;            // 2048: K zero rows
constexpr int WS_K_ZQ = WS_K_Z + 2048;           // 128: sum_c zero*q per group of the tile and head, float [4][8]
constexpr int WS_K_END = WS_K_ZQ + 128;          // 12416
constexpr int WS_KSTAT = WS_K_END;               // 512: (max, sum-exp) per (batch, kv head) slot and head, float2 [8][8]
constexpr int WS_KPOS = WS_KSTAT + 512;          // 256: logical positions of the 64 tokens of a sub-span, uint32 [64]
constexpr int WS_V_S = 8192;                     // 1024: V scales of the tile as in memory [token][group]
constexpr int WS_V_Z = WS_V_S + 1024;            // 1024
constexpr int WS_V_P = WS_V_Z + 1024;            // 1088: exp(logit - max) of heads 0-3, half [4][136]
constexpr int V_PROW = 128 + 8;                  // halfs per staged probability row (pitch 68 words: rows 4 banks apart)
constexpr int WS_V_P_BYTES = 4 * V_PROW * 2;     // 1088
// after the probability rows (one set for up to four query heads per kv head, two for eight):
//   out  float [rep4][128]  partial output of the warp for its current (batch, kv head); rep4 = 4 or 8
//   zt   float [4][8]       sum_t p*zero per channel group and head
__host__ __device__ constexpr int ws_v_out(bool rep8) { return WS_V_P + (rep8 ? 2 : 1) * WS_V_P_BYTES; }
__host__ __device__ constexpr int ws_v_zt(bool rep8) { return ws_v_out(rep8) + (rep8 ? 8 : 4) * D * 4; }
__host__ __device__ constexpr int ws_bytes(bool rep8) { return ws_v_zt(rep8) + 128; }
static_assert(WS_KPOS + 256 <= ws_bytes(false), "K statistics and positions fit the region");
static_assert(WS_KSTAT >= ws_v_out(false) && WS_KSTAT >= WS_V_P + WS_V_P_BYTES, "K statistics do not overlap a V tile's staged inputs");

// ------------------------------------------------------------------------------------------------
// fragments and small helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Streaming loads: the cache is read once per call, keep it out of L1.
__device__ __forceinline__ uint2 ld_stream(const uint2* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// low word of an int64 list entry (logical positions are below 2^30)
__device__ __forceinline__ uint32_t ld_pos(const int64_t* p) {
  return static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned long long*>(p)));
}

// 2^x on the special-function unit (about 2 ulp; 2^-inf = 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void softmax_merge(float& m, float& l, float m2, float l2) {
  const float mx = fmaxf(m, m2);
  if (mx == -INFINITY) return;  // both empty
  l = l * fast_exp2((m - mx) * LOG2E) + l2 * fast_exp2((m2 - mx) * LOG2E);
  m = mx;
}

// global -> shared copies without a register round trip; completion = wait_group + __syncwarp
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
               "l"(src));
}
__device__ __forceinline__ void cp_async_8(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
               "l"(src));
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
               "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// four 8x8 matrices of 16-bit elements, transposed: lane (g, tig) gets elements (row 2*tig, col g) and
// (row 2*tig+1, col g) of matrix i in r[i]; lanes 8*i .. 8*i+7 supply the row addresses of matrix i
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(row_ptr))));
}

// 16-bit halves of two words -> one half2 register (low half from a)
__device__ __forceinline__ uint32_t pack_lo16(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x5410); }

// q of one (batch, kv head) in shared memory: one row of Q_PITCH halfs per query head (rows beyond the heads that
// exist are zero).  The pitch of 68 words puts the rows of four heads four banks apart, so the B-fragment reads of
// a warp (head g & 3 or g, channels 16*kt + 2*tig + (0,1 | 8,9)) are free of bank conflicts.
constexpr int Q_PITCH = D + 8;
// B fragment of q for the 16-channel step kt: column n = g is the query head of row qrow (set per lane), rows are
// channels 16*kt + 2*tig + (0,1) in .x and + (8,9) in .y
__device__ __forceinline__ uint2 q_frag(const __half* qrow_tig, int kt) {
  return make_uint2(*reinterpret_cast<const uint32_t*>(qrow_tig + 16 * kt),
                    *reinterpret_cast<const uint32_t*>(qrow_tig + 16 * kt + 8));
}

// ------------------------------------------------------------------------------------------------
// K tiles
// ------------------------------------------------------------------------------------------------
// Quantised K tier: rows = channels, packed words along tokens.  A TILE is all 128 channel rows x
// 64 bytes of codes (32 bytes at 2 bits, 16 at 1 bit), i.e. 64 / 128 / 128 / 128 tokens at 8 / 4 / 2 / 1
// bits, with the scale / zero rows of its (up to four) token groups.  All of it is copied global ->
// shared with cp.async as the first action (no registers are tied up) and the warp then works out
// of shared memory in sub-spans of 64 tokens.  Wide copies in, ldmatrix out: the L1 data pipe moves
// 128 bytes per wavefront both ways.
//
// ldmatrix.trans over 8 channel rows x 16 bytes hands lane (g, tig) the 16-bit block g of channels
// 2*tig and 2*tig+1 in one register: exactly the two K-neighbours of an m16n8k16 A fragment for the
// tokens of block g (2 / 4 / 8 tokens at 8 / 4 / 2 bits).  What keeps the instruction count low:
//  * the integer codes enter the tensor pipe as they are: a masked field at bit k < 10 of a 16-bit
//    lane IS the fp16 subnormal code * 2^(k-24), exactly, so one AND per pair of codes builds an A
//    fragment register; the power of two comes back out in the epilogue;
//  * the scale lives in the B operand: logit = sum_c (q_c * scale_c) * code_c + sum_c q_c * zero_c.
//    A sub-span holds two 32-token scale groups; B columns 0-3 hold q*scale of the first group for
//    four query heads and columns 4-7 that of the second, and each fragment row keeps the half of
//    its accumulators whose group matches.  With eight query heads per kv head the warp walks its
//    tile once per half of the heads;
//  * q*scale (11 x 11 significant bits) is carried EXACTLY as hi = fp16(q*scale) and
//    lo = q*scale - hi, two MMAs into the same fp32 accumulator.  (One fp16 rounding of it - or of
//    the dequantised K value - costs ~2e-3 on the attention output with x10 outlier channels.)
//  * the zero point enters through Zq[group][head] = sum_c zero_c * q_c, one small MMA per tile;
//  * every lane scatters its own logits from registers and keeps a running (max, sum-exp).
constexpr int K_SPAN = 64;           // tokens per sub-span: four M-tiles of 16
constexpr int K_SLOT = 4;            // fp16 tier: tokens per 8-byte slot
constexpr int K_SROW = 8;            // staged halfs per channel row of scales: two aligned 8-byte pieces
constexpr int K_TROW = MAX_REP + 1;  // floats per token row of the logit tile (odd: no bank conflicts)

template <int BITS>
struct KTile {
  static constexpr int PITCH = BITS == 1 ? 16 : BITS == 2 ? 32 : 64;  // bytes per channel row
  static constexpr int TOKENS = PITCH * 8 / BITS;         // 64, 128, 128, 128 at 8, 4, 2, 1 bits
  static constexpr int NSUB = TOKENS / K_SPAN;            // sub-spans: 1, 2, 2, 2
  static constexpr int TPC = 128 / BITS;                  // tokens per 16-byte piece: 16, 32, 64, 128
  static constexpr int CPS = BITS == 1 ? 1 : K_SPAN / TPC;  // pieces of a row per sub-span: 4, 2, 1 (1 bit: half a piece)
  // byte offset of 16-byte piece c of a channel row.  The piece index is XORed with row bits so that
  // the eight rows of an ldmatrix (same logical piece) and the pieces a cp.async instruction writes
  // both spread over all banks.
  static __device__ __forceinline__ uint32_t offset(uint32_t row, uint32_t c) {
    if constexpr (PITCH == 64) {
      return row * 64u + ((c ^ ((row >> 1) & 3u)) << 4);
    } else if constexpr (PITCH == 32) {
      return row * 32u + ((c ^ ((row >> 2) & 1u)) << 4);
    } else {
      return row * 16u;  // 1 bit: read with 2-byte loads, see k_tile_compute
    }
  }
};

// Requests of a tile's parts.  They are written once for all bit widths (the width is a run-time argument) and
// are not inlined: with one tile per warp every instruction of this kernel is fetched about once per launch, so
// what a launch costs is first of all the amount of code it walks through.
//
// Scale / zero rows: group gamma of channel c (of G per row) is half ((bh*128 + c)*G + g0) of its plane, at any
// 2-byte alignment; the two aligned 8-byte pieces that cover the tile's (up to four) groups go to shared memory
// as they are, so group gamma of the tile sits at half ((c*G + g0) & 3) + gamma of row c.  (The planes hold
// B*H*128*G halfs, a multiple of 4, and start 8-byte aligned, so an aligned piece that begins inside a plane also
// ends inside it.)  ntok = valid tokens of the tile (a multiple of 32).  Commits one group.
__device__ __noinline__ void k_scales_request(const __half* k_scale, const __half* k_zero, unsigned char* wsm, int bh, int G,
                                              int g0, int ng) {
  const int lane = threadIdx.x & 31;
  __half* s = reinterpret_cast<__half*>(wsm + WS_K_S);
  __half* z = reinterpret_cast<__half*>(wsm + WS_K_Z);
#pragma unroll 1
  for (int j = 0; j < 4; ++j) {
    const int ch = lane + 32 * j;
    const int64_t e0 = (static_cast<int64_t>(bh) * D + ch) * G + g0;
    const int64_t a = e0 & ~static_cast<int64_t>(3);
    cp_async_8(s + ch * K_SROW, k_scale + a);
    cp_async_8(z + ch * K_SROW, k_zero + a);
    if (a + 4 < e0 + ng) {
      cp_async_8(s + ch * K_SROW + 4, k_scale + a + 4);
      cp_async_8(z + ch * K_SROW + 4, k_zero + a + 4);
    }
  }
  cp_async_commit();
}
// Codes of channel rows 32*quarter .. 32*quarter + 31 (two 16-channel steps).  src: byte address of (row 0, first
// token of the tile).  A row holds `pitch` bytes in shared memory (64, 64, 32, 16 at 8, 4, 2, 1 bits); four lanes
// share a row, each copies pitch / 4 bytes (16, 16, 8, 4 - also the alignment rows of that width are sure to
// have in memory), so one copy instruction moves 8 rows.  The shared-memory layout is KTile<BITS>::offset.
// Commits one group.
__device__ __noinline__ void k_codes_request(const unsigned char* src, int64_t row_bytes, unsigned char* codes, int pitch,
                                             int valid_bytes, int quarter) {
  const int lane = threadIdx.x & 31;
  const int piece = pitch >> 2, r0 = lane >> 2, cb = (lane & 3) * piece;  // byte of the row this lane copies
  if (cb < valid_bytes) {
#pragma unroll 1
    for (int i = 0; i < 4; ++i) {
      const uint32_t row = quarter * 32 + i * 8 + r0;
      const uint32_t swz = pitch == 64 ? ((row >> 1) & 3u) : pitch == 32 ? ((row >> 2) & 1u) : 0u;
      unsigned char* d = codes + row * pitch + (((static_cast<uint32_t>(cb) >> 4) ^ swz) << 4) + (cb & 15);
      const unsigned char* s = src + row * row_bytes + cb;
      if (piece == 16) cp_async_16(d, s);
      else if (piece == 8) cp_async_8(d, s);
      else cp_async_4(d, s);
    }
  }
  cp_async_commit();
}
__device__ __forceinline__ int k_pitch(int bits) { return bits == 1 ? 16 : bits == 2 ? 32 : 64; }
__device__ __forceinline__ const unsigned char* k_tile_src(const TierDev& T, int bh, int tile_t0, int64_t& row_bytes) {
  row_bytes = static_cast<int64_t>(T.n_k) * T.bits / 8;
  return reinterpret_cast<const unsigned char*>(T.k_data) + static_cast<int64_t>(bh) * D * row_bytes +
         static_cast<int64_t>(tile_t0) * T.bits / 8;
}
// A whole tile: the scale / zero rows in the oldest commit group, then one group per quarter of the codes.
__device__ __noinline__ void k_tile_request(const TierDev& T, unsigned char* wsm, int bh, int tile_t0, int ntok, int gk_shift) {
  const int g0 = tile_t0 >> gk_shift;
  k_scales_request(T.k_scale, T.k_zero, wsm, bh, T.n_k >> gk_shift, g0, ((tile_t0 + ntok - 1) >> gk_shift) - g0 + 1);
  int64_t row_bytes;
  const unsigned char* src = k_tile_src(T, bh, tile_t0, row_bytes);
#pragma unroll 1
  for (int quarter = 0; quarter < 4; ++quarter)
    k_codes_request(src, row_bytes, wsm + WS_CODES, k_pitch(T.bits), ntok * T.bits / 8, quarter);
}

// Zq[group][head] of the tile for the heads in qf: rows of the A operand are the tile's groups
// (at most four; rows 4-7 repeat them, rows 8-15 are zero).  z_even / z_odd: this lane's two staged
// zero rows (channels 2*tig and 2*tig+1) at the half of the tile's first group.
// Gaussian-codebook tier (s_even / s_odd non-null: the std rows at the same halves): a value is
// std * C * (2 code - 1) + mean, so the term that does not depend on the code is sum_c (mean - C std) q.
__device__ __forceinline__ void k_tile_zq(float* zq, const __half* qrow_tig, const __half* z_even, const __half* z_odd,
                                          const __half* s_even = nullptr, const __half* s_odd = nullptr) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int gam = g & 3;
  float zacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
  for (int kt = 0; kt < 8; ++kt) {
    const int o = (16 * kt) * K_SROW + gam;
    const uint32_t a0 = pack_lo16(__half_as_ushort(z_even[o]), __half_as_ushort(z_odd[o]));
    const uint32_t a2 = pack_lo16(__half_as_ushort(z_even[o + 8 * K_SROW]), __half_as_ushort(z_odd[o + 8 * K_SROW]));
    const uint2 bq = q_frag(qrow_tig, kt);
    mma16816(zacc, a0, 0u, a2, 0u, bq.x, bq.y);
  }
  if (s_even) {
    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
    for (int kt = 0; kt < 8; ++kt) {
      const int o = (16 * kt) * K_SROW + gam;
      const uint32_t a0 = pack_lo16(__half_as_ushort(s_even[o]), __half_as_ushort(s_odd[o]));
      const uint32_t a2 = pack_lo16(__half_as_ushort(s_even[o + 8 * K_SROW]), __half_as_ushort(s_odd[o + 8 * K_SROW]));
      const uint2 bq = q_frag(qrow_tig, kt);
      mma16816(sacc, a0, 0u, a2, 0u, bq.x, bq.y);
    }
    zacc[0] = fmaf(-HQKV_NORMAL1_CENTER, sacc[0], zacc[0]);
    zacc[1] = fmaf(-HQKV_NORMAL1_CENTER, sacc[1], zacc[1]);
  }
  __syncwarp();  // readers of the previous half are done
  if (g < 4 && tig < 2) {  // columns 0-3 are the four heads of this half; 4-7 repeat them
    zq[g * MAX_REP + 2 * tig] = zacc[0];
    zq[g * MAX_REP + 2 * tig + 1] = zacc[1];
  }
  __syncwarp();
}

// A fragment registers of the four M-tiles of a sub-span from the ldmatrix registers of one 8-channel
// octet.  R[c]: 16-byte piece c of the sub-span; each 16-bit half = block g of one channel.
// lo[i] -> fragment row g of M-tile i, hi[i] -> row g+8.  Fields are fp16 subnormals code * 2^(k-24);
// KField<BITS>::shift(i) gives k of M-tile i.
//   8 bits: block = 2 tokens.  M-tile i = (piece p = i>>1, token e = i&1): row g <- piece p, row g+8 <-
//           piece p+2.  Tokens: row g = 16p + 2g + e, row g+8 = 32 + 16p + 2g + e.
//   4 bits: block = 4 tokens.  M-tile i: row g <- piece 0 token i, row g+8 <- piece 1 token i.
//           Tokens: row g = 4g + i, row g+8 = 32 + 4g + i.
//   2 bits: block = 8 tokens, one piece.  M-tile i: row g <- token i, row g+8 <- token 4+i of block g.
//           Tokens: row g = 8g + i, row g+8 = 8g + 4 + i.
//   1 bit:  block = 16 tokens, four blocks per sub-span (no ldmatrix: lane g reads block g & 3 with a
//           2-byte load).  M-tile i: row g <- token 4*(g>>2) + i, row g+8 <- token 8 + 4*(g>>2) + i of
//           block g & 3.  Tokens: row g = 16*(g&3) + 4*(g>>2) + i, row g+8 = +8.
template <int BITS>
struct KField {
  static __host__ __device__ constexpr int shift(int i) {
    return BITS == 8 ? 0 : BITS == 4 ? 4 * (i & 1) : BITS == 2 ? 2 * i : i;
  }
};
template <int BITS>
__device__ __forceinline__ void octet_frags(const uint32_t* R, uint32_t (&lo)[4], uint32_t (&hi)[4]) {
  if constexpr (BITS == 8) {
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      lo[2 * p] = R[p] & 0x00FF00FFu;
      lo[2 * p + 1] = __byte_perm(R[p], 0u, 0x4341);
      hi[2 * p] = R[p + 2] & 0x00FF00FFu;
      hi[2 * p + 1] = __byte_perm(R[p + 2], 0u, 0x4341);
    }
  } else if constexpr (BITS == 4) {
    const uint32_t a = R[0], as = R[0] >> 8, b = R[1], bs = R[1] >> 8;
    lo[0] = a & 0x000F000Fu;
    lo[1] = a & 0x00F000F0u;
    lo[2] = as & 0x000F000Fu;
    lo[3] = as & 0x00F000F0u;
    hi[0] = b & 0x000F000Fu;
    hi[1] = b & 0x00F000F0u;
    hi[2] = bs & 0x000F000Fu;
    hi[3] = bs & 0x00F000F0u;
  } else {
    const uint32_t a = R[0], as = R[0] >> 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo[i] = a & (0x00030003u << (2 * i));
      hi[i] = as & (0x00030003u << (2 * i));
    }
  }
}

// running (max, sum-exp) of a lane over values it produces four at a time; -inf marks "no value"
__device__ __forceinline__ void softmax_push4(float& m, float& l, const float (&x)[4]) {
  const float mn = fmaxf(fmaxf(m, fmaxf(x[0], x[1])), fmaxf(x[2], x[3]));
  const float ref = (mn == -INFINITY ? 0.f : mn) * LOG2E;
  l = l * fast_exp2(fmaf(m, LOG2E, -ref)) + (fast_exp2(fmaf(x[0], LOG2E, -ref)) + fast_exp2(fmaf(x[1], LOG2E, -ref))) +
      (fast_exp2(fmaf(x[2], LOG2E, -ref)) + fast_exp2(fmaf(x[3], LOG2E, -ref)));
  m = mn;
}

// What a warp carries from tile to tile while it stays on one (batch, kv head) of the K side.
struct KWarpState {
  float m[2][2];     // quantised tiles: this lane's running (max, sum-exp), [half of the heads][e] for head
  float l[2][2];     //   4*half + 2*(tig & 1) + e
  float pm, pl;      // fp16 tiles: this lane's running pair for head lane & (rep - 1)
  const __half* mask0;     // additive mask row of head 0 of this kv head (fp16, indexed by logical position), or null
  int64_t mask_hstride;    // elements between the mask rows of consecutive query heads (0: one row for all heads)
};

// One tile of a quantised tier, already requested: all heads of this kv head.
// row0: logit row of head 0 of this kv head; qs: q rows of this kv head in shared memory (Q_PITCH halfs each).
// Streaming: with next_ntok > 0 the NEXT tile of the same tier and (batch, kv head) - tokens next_t0 .. - is
// requested into the same buffer while this one is computed: a quarter of its code rows as soon as the last
// walk over this tile is done with that quarter, its scale / zero rows after the last step.  A tile that was
// requested that way (streamed_in) finds all its parts issued, the scale rows last.
template <int BITS>
__device__ __forceinline__ void k_tile_compute(const TierDev& T, unsigned char* wsm, KWarpState& st, const __half* qs,
                                               int bh, int rep, int L, int gk_shift, float qk_scale, int tile_t0, int ntok,
                                               float* row0, bool streamed_in, int next_t0, int next_ntok) {
  using TL = KTile<BITS>;
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int G = T.n_k >> gk_shift;
  const int g0 = tile_t0 >> gk_shift;  // first group of the tile
  const int nh = rep > 4 ? 2 : 1;
  // staged scale / zero rows of this lane's channels 2*tig (even) and 2*tig+1 (odd) of step 0, at the
  // half of the tile's first group; a step adds 16 rows, the +8 channels add 8 rows
  const int sh_even = static_cast<int>((static_cast<int64_t>(2 * tig) * G + g0) & 3);
  const int sh_odd = static_cast<int>((static_cast<int64_t>(2 * tig + 1) * G + g0) & 3);
  const __half* srow = reinterpret_cast<const __half*>(wsm + WS_K_S);
  const __half* zrow = reinterpret_cast<const __half*>(wsm + WS_K_Z);
  float* zq = reinterpret_cast<float*>(wsm + WS_K_ZQ);
  const unsigned char* codes = wsm + WS_CODES;
  // ldmatrix row address of this lane for step 0 / sub-span 0 (see the loop for the matrix order)
  uint32_t lm_off;
  {
    const int mi = lane >> 3, rr = lane & 7;
    if constexpr (BITS == 8) {
      lm_off = TL::offset(rr, mi);                           // octet 0; pieces 0..3
    } else if constexpr (BITS == 4) {
      lm_off = TL::offset(8 * (mi >> 1) + rr, mi & 1);       // (octet 0, piece 0), (0,1), (1,0), (1,1)
    } else if constexpr (BITS == 2) {
      lm_off = TL::offset(8 * mi + rr, 0);                   // steps kt, kt+1: octets 0..3 of 32 channels
    } else {
      lm_off = (2 * tig) * 16 + 2 * (g & 3);                 // 1 bit: this lane's block of channel 2*tig
    }
  }
  const int hp = tig & 1;
  // Gaussian-codebook 1-bit tier: the code term carries the factor 2C
  const bool normal = BITS == 1 && T.normal != 0;
  const float pscale = normal ? qk_scale * (2.f * HQKV_NORMAL1_CENTER) : qk_scale;

  const bool stream_out = next_ntok > 0;
  if (streamed_in) cp_async_wait<0>();  // everything of this tile was requested during the previous one
  else cp_async_wait<4>();              // the scale / zero rows
  __syncwarp();
  for (int hh = 0; hh < nh; ++hh) {
    // as a B column this lane is n = g: query head 4*hh + (g & 3) (columns 4-7 repeat 0-3)
    const __half* qrow_tig = qs + (4 * hh + (g & 3)) * Q_PITCH + 2 * tig;
    if (normal)
      k_tile_zq(zq, qrow_tig, zrow + (2 * tig) * K_SROW + sh_even, zrow + (2 * tig + 1) * K_SROW + sh_odd,
                srow + (2 * tig) * K_SROW + sh_even, srow + (2 * tig + 1) * K_SROW + sh_odd);
    else
      k_tile_zq(zq, qrow_tig, zrow + (2 * tig) * K_SROW + sh_even, zrow + (2 * tig + 1) * K_SROW + sh_odd);
#pragma unroll 1
    for (int j = 0; j < TL::NSUB; ++j) {
      const int sub_t0 = j * K_SPAN;
      // Epilogue ownership (decided here so that the positions can be requested before the MMA loop):
      // a lane keeps the accumulator columns whose scale group is its row's, and every lane ends up
      // with four tokens x two heads (heads 2*(tig&1), +1).
      //  8 / 4 bits: rows 0-7 are tokens 0-31, rows 8-15 tokens 32-63: lanes tig 0,1 own row g, lanes
      //              tig 2,3 own row g+8.
      //  2 bits:     rows g and g+8 are the eight tokens of block g, valid in the lanes with
      //              (g < 4) == (tig < 2); such a lane keeps the row of its tig half and hands the
      //              other row to lane tig ^ 2, whose own accumulators belong to the wrong scale group.
      //  1 bit:      the same with block g & 3: valid where ((g & 3) < 2) == (tig < 2).
      const int r = tig >> 1;
      // first of this lane's tokens (8 bits: tokens my_tok, +1, +16, +17; 4, 2 and 1 bits: my_tok .. my_tok+3)
      const int my_tok = sub_t0 + (BITS == 8 ? 32 * r + 2 * g : BITS == 4 ? 32 * r + 4 * g : BITS == 2 ? 8 * g + 4 * r
                                                                : 16 * (g & 3) + 4 * (g >> 2) + 8 * r);
      const bool live = my_tok < ntok;
      // the sub-span's logical positions: requested now (one coalesced 8-byte load per token), handed to the
      // lanes that own the tokens through shared memory after the MMA loop
      uint32_t pos_a = 0u, pos_b = 0u;
      if (sub_t0 + lane < ntok) pos_a = ld_pos(T.k_idx + tile_t0 + sub_t0 + lane);
      if (sub_t0 + 32 + lane < ntok) pos_b = ld_pos(T.k_idx + tile_t0 + sub_t0 + 32 + lane);
      // as a B column this lane is n = g: columns 0-3 carry the scale group of tokens 0-31 of the
      // sub-span, columns 4-7 that of tokens 32-63
      const int gam = ((tile_t0 + sub_t0 + 32 * (g >> 2)) >> gk_shift) - g0;
      const __half* s_even = srow + (2 * tig) * K_SROW + sh_even + gam;
      const __half* s_odd = srow + (2 * tig + 1) * K_SROW + sh_odd + gam;
      const unsigned char* kb = codes + (BITS == 1 ? lm_off + j * 8 : (lm_off ^ (j * TL::CPS * 16)));
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
      // two 16-channel steps per iteration (short loop body: with one tile per warp every warp runs this code
      // once, so it is fetched rather than reused)
#pragma unroll 1
      for (int kk = 0; kk < 4; ++kk) {
        const bool last_walk = hh == nh - 1 && j == TL::NSUB - 1;
        if (hh == 0 && j == 0 && !streamed_in) {  // the codes arrive two steps at a time
          // groups younger than this quarter: the later quarters of this tile, and - when this only walk is also
          // the last one and streams the next tile in - the kk quarters of the next tile requested so far
          if (kk == 0 || (last_walk && stream_out)) cp_async_wait<3>();
          else if (kk == 1) cp_async_wait<2>();
          else if (kk == 2) cp_async_wait<1>();
          else cp_async_wait<0>();
          __syncwarp();
        }
        uint32_t R2[4];  // 2 bits: one ldmatrix feeds both steps
        if constexpr (BITS == 2) ldmatrix_x4_trans(R2, kb + kk * 32 * TL::PITCH);
        (void)R2;
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
          const unsigned char* kbs = kb + (kk * 32 + k2 * 16) * TL::PITCH;
          // A fragments: lo/hi of octet 0 -> registers 0/1 (channels 2tig, 2tig+1), of octet 1 -> 2/3 (+8)
          uint32_t a[4][4];  // [register][M-tile]
          if constexpr (BITS == 8) {
            uint32_t R[4];
            ldmatrix_x4_trans(R, kbs);
            octet_frags<8>(R, a[0], a[1]);
            ldmatrix_x4_trans(R, kbs + 8 * TL::PITCH);
            octet_frags<8>(R, a[2], a[3]);
          } else if constexpr (BITS == 4) {
            uint32_t R[4];
            ldmatrix_x4_trans(R, kbs);
            octet_frags<4>(R, a[0], a[1]);
            octet_frags<4>(R + 2, a[2], a[3]);
          } else if constexpr (BITS == 2) {
            octet_frags<2>(R2 + 2 * k2, a[0], a[1]);
            octet_frags<2>(R2 + 2 * k2 + 1, a[2], a[3]);
          } else {
#pragma unroll
            for (int o = 0; o < 2; ++o) {  // channels 2tig, 2tig+1 (o = 0) and +8, +9 (o = 1)
              const unsigned char* cb = kbs + o * 8 * 16;
              const uint32_t t = pack_lo16(*reinterpret_cast<const uint16_t*>(cb), *reinterpret_cast<const uint16_t*>(cb + 16));
              const uint32_t lo = t >> (4 * (g >> 2)), hi = lo >> 8;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                a[2 * o][i] = lo & (0x00010001u << i);
                a[2 * o + 1][i] = hi & (0x00010001u << i);
              }
            }
          }
          const int o = (kk * 32 + k2 * 16) * K_SROW;
          const __half2 s0 = u32_as_h2(pack_lo16(__half_as_ushort(s_even[o]), __half_as_ushort(s_odd[o])));
          const __half2 s1 = u32_as_h2(pack_lo16(__half_as_ushort(s_even[o + 8 * K_SROW]),
                                                 __half_as_ushort(s_odd[o + 8 * K_SROW])));
          const uint2 qv = q_frag(qrow_tig, 2 * kk + k2);
          const __half2 hi0 = __hmul2(u32_as_h2(qv.x), s0);
          const __half2 hi1 = __hmul2(u32_as_h2(qv.y), s1);
          const __half2 lo0 = __hfma2(u32_as_h2(qv.x), s0, __hneg2(hi0));  // exact remainder
          const __half2 lo1 = __hfma2(u32_as_h2(qv.y), s1, __hneg2(hi1));
          // the two MMAs into one accumulator are issued four apart (they depend on each other)
#pragma unroll
          for (int i = 0; i < 4; ++i) mma16816(acc[i], a[0][i], a[1][i], a[2][i], a[3][i], h2_as_u32(hi0), h2_as_u32(hi1));
#pragma unroll
          for (int i = 0; i < 4; ++i) mma16816(acc[i], a[0][i], a[1][i], a[2][i], a[3][i], h2_as_u32(lo0), h2_as_u32(lo1));
        }
        if (last_walk && stream_out) {  // nobody reads these 32 channel rows of this tile again
          __syncwarp();
          int64_t row_bytes;
          const unsigned char* src = k_tile_src(T, bh, next_t0, row_bytes);
          k_codes_request(src, row_bytes, wsm + WS_CODES, TL::PITCH, next_ntok * BITS / 8, kk);
        }
      }
      if (hh == nh - 1 && j == TL::NSUB - 1 && stream_out) {  // the scale / zero rows are free as well
        __syncwarp();
        const int ng0 = next_t0 >> gk_shift;
        k_scales_request(T.k_scale, T.k_zero, wsm, bh, G, ng0, ((next_t0 + next_ntok - 1) >> gk_shift) - ng0 + 1);
      }
      // Epilogue from registers.
      uint32_t pos[4];
      {
        uint32_t* kpos = reinterpret_cast<uint32_t*>(wsm + WS_KPOS);
        __syncwarp();  // the previous sub-span's readers are done
        kpos[lane] = pos_a;
        kpos[lane + 32] = pos_b;
        __syncwarp();
        const int o = my_tok - sub_t0;
        if constexpr (BITS == 8) {
          const uint2 p01 = *reinterpret_cast<const uint2*>(kpos + o), p23 = *reinterpret_cast<const uint2*>(kpos + o + 16);
          pos[0] = p01.x, pos[1] = p01.y, pos[2] = p23.x, pos[3] = p23.y;
        } else {
          const uint4 p = *reinterpret_cast<const uint4*>(kpos + o);
          pos[0] = p.x, pos[1] = p.y, pos[2] = p.z, pos[3] = p.w;
        }
      }
      float val[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int e = 0; e < 2; ++e) val[i][e] = r ? acc[i][2 + e] : acc[i][e];
      if constexpr (BITS <= 2) {
        const bool valid = BITS == 2 ? (g < 4) == (tig < 2) : ((g & 3) < 2) == (tig < 2);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, r ? acc[i][e] : acc[i][2 + e], 2);
            if (!valid) val[i][e] = other;
          }
      }
      const int my_gam = ((tile_t0 + my_tok) >> gk_shift) - g0;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int head = 4 * hh + 2 * hp + e;
        const bool on = live && head < rep;
        const float zqs = zq[(my_gam & 3) * MAX_REP + 2 * hp + e] * qk_scale;
        float* row = row0 + static_cast<int64_t>(head) * L;
        float x[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float unscale = static_cast<float>(1 << (24 - KField<BITS>::shift(i)));
          x[i] = on ? fmaf(val[i][e], pscale * unscale, zqs) : -INFINITY;
        }
        if (st.mask0 != nullptr && on) {
          const __half* mrow = st.mask0 + head * st.mask_hstride;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (HQKV_INDEX_OK(pos[i], L)) x[i] += __half2float(mrow[pos[i]]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (on && HQKV_INDEX_OK(pos[i], L)) row[pos[i]] = x[i];
        softmax_push4(st.m[hh][e], st.l[hh][e], x);
      }
    }
  }
}

// Write out a warp's logit tile [ntok][K_TROW] (already scaled) at the tokens' logical positions and
// fold it into the lane's running (max, sum-exp).  Element = (token, head) with the head fastest
// across lanes, so every lane owns ONE head for the whole call (rep divides 32) and index loads and
// stores are spread over all 32 lanes.  (fp16 tier and residual window only; the quantised tiers
// write from registers.)
__device__ __forceinline__ void k_write_tile(KWarpState& st, const float* tile, int ntok, const int64_t* idx, int64_t first_pos,
                                             int rep, int rep_shift, int L, float* row0) {
  const int lane = threadIdx.x & 31;
  const int h = lane & (rep - 1);
  float* row = row0 + static_cast<int64_t>(h) * L;
  const int tpr = 32 >> rep_shift;  // tokens per round
  float mx = st.pm;
#pragma unroll 2
  for (int t = lane >> rep_shift; t < ntok; t += tpr) {
    const int64_t pos = idx ? static_cast<int64_t>(ld_pos(idx + t)) : first_pos + t;
    float x = tile[t * K_TROW + h];
    if (!HQKV_INDEX_OK(pos, L)) continue;
    if (st.mask0 != nullptr) {
      x += __half2float(st.mask0[h * st.mask_hstride + pos]);
      const_cast<float*>(tile)[t * K_TROW + h] = x;  // the second pass reads it back (own element: no race)
    }
    row[pos] = x;
    mx = fmaxf(mx, x);
  }
  if (mx == -INFINITY) return;  // this lane has seen no token yet
  float sum = st.pl * fast_exp2((st.pm - mx) * LOG2E);
#pragma unroll 2
  for (int t = lane >> rep_shift; t < ntok; t += tpr) sum += fast_exp2((tile[t * K_TROW + h] - mx) * LOG2E);
  st.pm = mx;
  st.pl = sum;
}

// fp16 tier, channel-major rows [D][n]: four tokens per 8-byte slot, no scales; B = q exactly.
// One span of 64 tokens per call.
__device__ __forceinline__ void k_f16_span(const TierDev& T, unsigned char* wsm, KWarpState& st, const __half* qs, int bh, int rep,
                                           int rep_shift, int L, float qk_scale, int span_t0, float* row0) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  // B column n = g is query head g (with at most four heads the rows 4-7 do not exist: columns 4-7 repeat 0-3)
  const __half* qrow_tig = qs + (rep > 4 ? g : (g & 3)) * Q_PITCH + 2 * tig;
  const int n = T.n_k;
  const int64_t nslot = n / K_SLOT;
  const uint2* base = reinterpret_cast<const uint2*>(T.k_data) + static_cast<int64_t>(bh) * D * nslot;
  int64_t sl[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) sl[r] = min(static_cast<int64_t>(span_t0 / K_SLOT + r * 8 + g), nslot - 1);
  float acc[K_SLOT][4];
#pragma unroll
  for (int i = 0; i < K_SLOT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll 2
  for (int kt = 0; kt < 8; ++kt) {
    uint2 w[4][2];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int ch = 16 * kt + 8 * (e >> 1) + 2 * tig + (e & 1);
#pragma unroll
      for (int r = 0; r < 2; ++r) w[e][r] = ld_stream(base + ch * nslot + sl[r]);
    }
    // token i of a slot: halfs (x.lo, x.hi, y.lo, y.hi); pair the same token of two channel rows
    uint32_t a[K_SLOT][4];
#pragma unroll
    for (int q = 0; q < 2; ++q)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint2 wa = w[2 * q][r], wb = w[2 * q + 1][r];
        a[0][q * 2 + r] = __byte_perm(wa.x, wb.x, 0x5410);
        a[1][q * 2 + r] = __byte_perm(wa.x, wb.x, 0x7632);
        a[2][q * 2 + r] = __byte_perm(wa.y, wb.y, 0x5410);
        a[3][q * 2 + r] = __byte_perm(wa.y, wb.y, 0x7632);
      }
    const uint2 bq = q_frag(qrow_tig, kt);
#pragma unroll
    for (int i = 0; i < K_SLOT; ++i) mma16816(acc[i], a[i][0], a[i][1], a[i][2], a[i][3], bq.x, bq.y);
  }
  float* tile = reinterpret_cast<float*>(wsm + WS_CODES);
  __syncwarp();
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int e = 0; e < 2; ++e)
#pragma unroll
      for (int i = 0; i < K_SLOT; ++i)
        tile[((r * 8 + g) * K_SLOT + i) * K_TROW + 2 * tig + e] = acc[i][r * 2 + e] * qk_scale;
  __syncwarp();
  k_write_tile(st, tile, min(K_SPAN, n - span_t0), T.k_idx + span_t0, 0, rep, rep_shift, L, row0);
  __syncwarp();
}

// fp16 residual window, token-major [r][D]: A fragments are read directly; one 16-token tile per call.
__device__ __forceinline__ void k_residual_tile(const TierDev& T, unsigned char* wsm, KWarpState& st, const __half* qs, int bh,
                                                int rep, int rep_shift, int L, float qk_scale, int tile_t0, float* row0) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const __half* qrow_tig = qs + (rep > 4 ? g : (g & 3)) * Q_PITCH + 2 * tig;
  const int n = T.n_k;
  const __half* base = reinterpret_cast<const __half*>(T.k_data) + static_cast<int64_t>(bh) * n * D;
  const int t[2] = {min(tile_t0 + g, n - 1), min(tile_t0 + g + 8, n - 1)};
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  uint32_t a[8][4];
#pragma unroll
  for (int kt = 0; kt < 8; ++kt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const __half* p = base + static_cast<int64_t>(t[r]) * D + 16 * kt + 2 * tig;
      a[kt][r] = *reinterpret_cast<const uint32_t*>(p);
      a[kt][2 + r] = *reinterpret_cast<const uint32_t*>(p + 8);
    }
#pragma unroll
  for (int kt = 0; kt < 8; ++kt) {
    const uint2 bq = q_frag(qrow_tig, kt);
    mma16816(acc, a[kt][0], a[kt][1], a[kt][2], a[kt][3], bq.x, bq.y);
  }
  float* tile = reinterpret_cast<float*>(wsm + WS_CODES);
  __syncwarp();
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int e = 0; e < 2; ++e) tile[(r * 8 + g) * K_TROW + 2 * tig + e] = acc[r * 2 + e] * qk_scale;
  __syncwarp();
  k_write_tile(st, tile, min(16, n - tile_t0), nullptr, static_cast<int64_t>(L) - n + tile_t0, rep, rep_shift, L, row0);
  __syncwarp();
}

// The warp's (max, sum-exp) per head for the (batch, kv head) it has just finished -> kstat[head]
// (float2 [8]); the running pairs start over.  tmp: eight float2 of scratch in the warp's region.
__device__ __forceinline__ void k_emit_stats(KWarpState& st, float2* kstat, float2* tmp, int rep) {
  const int lane = threadIdx.x & 31;
  // quantised tiles: lanes that share tig & 1 hold pairs of the same two heads
#pragma unroll
  for (int hh = 0; hh < 2; ++hh)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float mx = st.m[hh][e];
#pragma unroll
      for (int o = 2; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = st.l[hh][e] * fast_exp2((st.m[hh][e] - (mx == -INFINITY ? 0.f : mx)) * LOG2E);
#pragma unroll
      for (int o = 2; o < 32; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane < 2) tmp[4 * hh + 2 * lane + e] = make_float2(mx, sum);
      st.m[hh][e] = -INFINITY;
      st.l[hh][e] = 0.f;
    }
  // fp16 tiles: lane owns head lane & (rep - 1)
  float pm = st.pm;
  for (int off = rep; off < 32; off <<= 1) pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, off));
  float pl = st.pl * fast_exp2((st.pm - (pm == -INFINITY ? 0.f : pm)) * LOG2E);
  for (int off = rep; off < 32; off <<= 1) pl += __shfl_xor_sync(0xffffffffu, pl, off);
  st.pm = -INFINITY;
  st.pl = 0.f;
  __syncwarp();
  if (lane < MAX_REP) {
    float m = -INFINITY, l = 0.f;
    if (lane < rep) {
      const float2 t = tmp[lane];
      m = t.x;
      l = t.y;
      softmax_merge(m, l, pm, pl);
    }
    kstat[lane] = make_float2(m, l);
  }
  __syncwarp();
}

// ------------------------------------------------------------------------------------------------
// V tiles
// ------------------------------------------------------------------------------------------------
// V tier, token-major rows of 128 channels.  A TILE is a run of consecutive tokens (8 KB of codes at
// 8 / 4 bits = 64 / 128 tokens, 4 KB at 2 bits = 128 tokens) with their scales and zeros, all copied
// global -> shared with cp.async before anything else.  The contraction runs over tokens, 16 per step.
// ldmatrix.trans over 8 token rows x 16 bytes hands lane (g, tig) the 16-bit block g (2 / 4 / 8 channels)
// of tokens 2*tig and 2*tig+1 in one register: the two K-neighbours of an m16n8k16 A fragment.  As on
// the K side the codes enter the tensor pipe as fp16 subnormals (one AND per pair of codes) and the
// scale - here per token and 32-channel group - is folded into the B operand:
// out[h][c] = sum_t (p_t * scale_t,G) * code_t,c + sum_t p_t * zero_t,G, with p*scale carried exactly as
// hi + lo and B columns 0-3 / 4-7 holding the two channel groups of a 64-channel half.  The zero term
// is one small MMA per step (rows = groups).
constexpr int V_MAX_TT = 128;  // tokens per tile at most

template <int BITS>
struct VTile {
  static constexpr int PITCH = 16 * BITS;                  // bytes per token row: 128, 64, 32, 16
  static constexpr int TOKENS = BITS == 8 ? 64 : 128;
  static constexpr int STEPS = TOKENS / 16;
  static constexpr int NPIECE = PITCH / 16;                // 16-byte pieces per row: 8, 4, 2, 1
  static __device__ __forceinline__ uint32_t offset(uint32_t row, uint32_t c) {
    if constexpr (PITCH == 128) {
      return row * 128u + ((c ^ (row & 7u)) << 4);
    } else if constexpr (PITCH == 64) {
      return row * 64u + ((c ^ ((row >> 1) & 3u)) << 4);
    } else if constexpr (PITCH == 32) {
      return row * 32u + ((c ^ ((row >> 2) & 1u)) << 4);
    } else {
      return row * 16u;  // 1 bit: read with 2-byte loads
    }
  }
};

// A fragment registers from one ldmatrix quad R[0..3] = sources of fragment registers a0..a3
// (a0: row g, tokens 2tig,2tig+1; a1: row g+8; a2 / a3: the same rows, tokens +8).
//   field f of a 16-bit block as the fp16 subnormal code * 2^(k-24); VField<BITS>::shift(f) gives k.
template <int BITS>
struct VField {
  static constexpr int N = BITS == 8 ? 2 : 4;  // fields taken from one register per fragment row
  static __host__ __device__ constexpr int shift(int f) {
    return BITS == 8 ? 0 : BITS == 4 ? 4 * (f & 1) : BITS == 2 ? 2 * f : f;
  }
};
template <int BITS>
__device__ __forceinline__ uint32_t v_field(uint32_t r, uint32_t r_shr8, int f) {
  if constexpr (BITS == 8) {
    return f == 0 ? (r & 0x00FF00FFu) : __byte_perm(r, 0u, 0x4341);
  } else if constexpr (BITS == 4) {
    return (f < 2 ? r : r_shr8) & (0x000F000Fu << (4 * (f & 1)));
  } else {
    return r & (0x00030003u << (2 * f));  // 2 bits: fields 0-3 of r (row g) or of r >> 8 (row g+8)
  }
}

// Request of one quarter of a tile's tokens (16 consecutive rows at 8 bits, 32 otherwise): their scales and zeros
// (ng halfs per token each, contiguous in memory) and their code rows of 16 * bits bytes, laid out as
// VTile<BITS>::offset.  ntok = valid tokens of the tile (a multiple of 32).  Written once for all widths, not
// inlined (see k_scales_request).  Commits one group.
__device__ __noinline__ void v_quarter_request(const TierDev& T, unsigned char* wsm, int bh, int tile_t0, int ntok, int ng,
                                               int quarter) {
  const int lane = threadIdx.x & 31;
  const int bits = T.bits;
  const int64_t tok0 = static_cast<int64_t>(bh) * T.n_v + tile_t0;
  const int qtok = bits == 8 ? 16 : 32;  // tokens per quarter
  {
    // 8-byte pieces: a quarter holds qtok * ng * 2 bytes = 32 .. 256
    const int o = quarter * qtok * ng * 2 + lane * 8, bytes = min(ntok, (quarter + 1) * qtok) * ng * 2;
    if (lane * 8 < qtok * ng * 2 && o < bytes) {
      cp_async_8(wsm + WS_V_S + o, reinterpret_cast<const unsigned char*>(T.v_scale + tok0 * ng) + o);
      cp_async_8(wsm + WS_V_Z + o, reinterpret_cast<const unsigned char*>(T.v_zero + tok0 * ng) + o);
    }
  }
  unsigned char* codes = wsm + WS_CODES;
  const uint32_t pitch = 16u * bits;
  const unsigned char* src = reinterpret_cast<const unsigned char*>(T.v_data) + tok0 * pitch;
  const int np_shift = bits == 8 ? 3 : bits == 4 ? 2 : bits == 2 ? 1 : 0;  // log2(16-byte pieces per row)
  const int per_q = (qtok << np_shift) >> 5;                                // copies per lane and quarter: 4, 4, 2, 1
#pragma unroll 1
  for (int i = 0; i < per_q; ++i) {
    const uint32_t id = (quarter * per_q + i) * 32 + lane;
    const uint32_t row = id >> np_shift, c = id & ((1u << np_shift) - 1u);
    const uint32_t swz = bits == 8 ? (row & 7u) : bits == 4 ? ((row >> 1) & 3u) : bits == 2 ? ((row >> 2) & 1u) : 0u;
    if (static_cast<int>(row) < ntok) cp_async_16(codes + row * pitch + ((c ^ swz) << 4), src + static_cast<int64_t>(id) * 16);
  }
  cp_async_commit();
}
// logical positions of the lane's tokens (lane + 32 j) of a tile of `tile_tokens` tokens
__device__ __forceinline__ void v_tile_positions(const TierDev& T, int tile_t0, int ntok, uint32_t (&pos)[4]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int t = lane + 32 * j;
    pos[j] = t < ntok ? ld_pos(T.v_idx + tile_t0 + t) : 0u;
  }
}
// A whole tile: four commit groups, one per quarter of the tokens.
__device__ __noinline__ void v_tile_request(const TierDev& T, unsigned char* wsm, int bh, int tile_t0, int ntok, int ng) {
#pragma unroll 1
  for (int quarter = 0; quarter < 4; ++quarter) v_quarter_request(T, wsm, bh, tile_t0, ntok, ng, quarter);
}

// exp(logit - max) of the tile's tokens for heads h0..h0+3 into prow[0..3][token], and the
// normalised probabilities into the output rows; the gathers of four heads are in flight together.
// pos[j]: logical position of token lane + 32 j.  gm / gl: global max / sum-exp per head of this kv head.
// logit0 / w0: logit and probability rows of head 0 of this kv head.
// With pin0 != nullptr (rows of caller-supplied weights, fp16) those are staged instead - the p.V product
// of given weights - and no probabilities are written.
template <int PER>
__device__ __forceinline__ void v_tile_probs(const float* gm, const float* gl, const uint32_t (&pos)[4], __half (*prow)[V_PROW],
                                             const float* logit0, __half* w0, const __half* pin0, int L, int rep, int h0,
                                             int ntok) {
  const int lane = threadIdx.x & 31;
  if (pin0) {
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      const int h = h0 + hh;
      const unsigned short* row = reinterpret_cast<const unsigned short*>(pin0) + static_cast<int64_t>(min(h, rep - 1)) * L;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int t = lane + 32 * j;
        const unsigned short v = (h < rep && t < ntok && HQKV_INDEX_OK(pos[j], L)) ? __ldcg(row + pos[j]) : static_cast<unsigned short>(0);
        prow[hh][t] = __ushort_as_half(v);
      }
    }
    return;
  }
  float x[4][PER];
#pragma unroll
  for (int hh = 0; hh < 4; ++hh) {
    const int h = min(h0 + hh, rep - 1);
    const float* row = logit0 + static_cast<int64_t>(h) * L;
#pragma unroll
    for (int j = 0; j < PER; ++j) x[hh][j] = (lane + 32 * j < ntok && HQKV_INDEX_OK(pos[j], L)) ? __ldcg(row + pos[j]) : -INFINITY;
  }
#pragma unroll
  for (int hh = 0; hh < 4; ++hh) {
    const int h = h0 + hh;
    const bool on = h < rep;
    const float mh = on ? gm[h] * LOG2E : 0.f, inv = on ? 1.f / gl[h] : 0.f;
    __half* wrow = w0 + static_cast<int64_t>(min(h, rep - 1)) * L;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int t = lane + 32 * j;
      const float e = on ? fast_exp2(fmaf(x[hh][j], LOG2E, -mh)) : 0.f;  // exp2(-inf) = 0 beyond the tile
      prow[hh][t] = __float2half_rn(e);
      if (on && t < ntok && HQKV_INDEX_OK(pos[j], L)) wrow[pos[j]] = __float2half_rn(e * inv);
    }
  }
}

// One tile of a quantised V tier for one half of the heads: acc[mt] = M-tile mt of the output
// (channels x heads, see the channel map in v_tile_store), zacc = zero term rows.
// With next_ntok > 0 the quarters of the NEXT tile of the same tier and (batch, kv head) (tokens next_t0 ..) are
// requested into the same buffer as soon as this walk is done with the rows they replace.
template <int BITS>
__device__ __forceinline__ void v_tile_walk(const TierDev& T, unsigned char* wsm, int gv_shift, const __half (*prow)[V_PROW],
                                            int ntok, float (&acc)[8][4], float (&zacc)[4], bool normal, int bh, int next_t0,
                                            int next_ntok) {
  using TL = VTile<BITS>;
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int ng_shift = 7 - gv_shift;  // log2(groups per token): 2, 1, 0
  const __half* vs = reinterpret_cast<const __half*>(wsm + WS_V_S);
  const __half* vz = reinterpret_cast<const __half*>(wsm + WS_V_Z);
  // ldmatrix row address of this lane for step 0, quad 0: matrices (token octet, piece) =
  //   8/4 bits: (0, c), (0, c'), (1, c), (1, c');  2 bits: (0, 0), (0, 1), (1, 0), (1, 1)
  // with (c, c') = the quad's two pieces: 4 bits (2pp, 2pp+1); 8 bits (4q+u, 4q+2+u)
  const int mi = lane >> 3, rr = lane & 7;
  const int lm_row = 8 * (mi >> 1) + rr;
  // as a B column this lane is n = g: head (n & 3) of this half, channel group of channels
  // 64q + 32*(n >> 2) for quad set q
  const __half* pr = &prow[g & 3][2 * tig];
  int gq[2];
#pragma unroll
  for (int q = 0; q < 2; ++q) gq[q] = (64 * q + 32 * (g >> 2)) >> gv_shift;
  const int zg = (g & 3) & ((1 << ng_shift) - 1);  // zero-term row g = group g (rows beyond ng repeat)
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  zacc[0] = zacc[1] = zacc[2] = zacc[3] = 0.f;
  float sacc[4] = {0.f, 0.f, 0.f, 0.f};  // Gaussian-codebook tier: sum_t p * std per channel group

  const int nsteps = ntok >> 4;
#pragma unroll 1
  for (int st = 0; st < nsteps; ++st) {
    const int t0 = st * 16;
    // B operands: p pairs of tokens (2tig, 2tig+1) and (+8, +9); scales of the same tokens
    const uint32_t p0 = *reinterpret_cast<const uint32_t*>(pr + t0);
    const uint32_t p1 = *reinterpret_cast<const uint32_t*>(pr + t0 + 8);
    const __half* sb = vs + ((t0 + 2 * tig) << ng_shift);
    const __half* zb = vz + ((t0 + 2 * tig) << ng_shift);
    uint32_t bh_[2][2], bl_[2][2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const __half2 s0 = u32_as_h2(pack_lo16(__half_as_ushort(sb[gq[q]]), __half_as_ushort(sb[(1 << ng_shift) + gq[q]])));
      const __half2 s1 = u32_as_h2(pack_lo16(__half_as_ushort(sb[(8 << ng_shift) + gq[q]]),
                                             __half_as_ushort(sb[(9 << ng_shift) + gq[q]])));
      const __half2 h0 = __hmul2(u32_as_h2(p0), s0), h1 = __hmul2(u32_as_h2(p1), s1);
      bh_[q][0] = h2_as_u32(h0);
      bh_[q][1] = h2_as_u32(h1);
      bl_[q][0] = h2_as_u32(__hfma2(u32_as_h2(p0), s0, __hneg2(h0)));  // exact remainder
      bl_[q][1] = h2_as_u32(__hfma2(u32_as_h2(p1), s1, __hneg2(h1)));
    }
    {  // zero term: A rows = channel groups, exact fp16 x fp16 products
      const uint32_t a0 = pack_lo16(__half_as_ushort(zb[zg]), __half_as_ushort(zb[(1 << ng_shift) + zg]));
      const uint32_t a2 = pack_lo16(__half_as_ushort(zb[(8 << ng_shift) + zg]), __half_as_ushort(zb[(9 << ng_shift) + zg]));
      mma16816(zacc, a0, 0u, a2, 0u, p0, p1);
    }
    if (BITS == 1 && normal) {
      const uint32_t a0 = pack_lo16(__half_as_ushort(sb[zg]), __half_as_ushort(sb[(1 << ng_shift) + zg]));
      const uint32_t a2 = pack_lo16(__half_as_ushort(sb[(8 << ng_shift) + zg]), __half_as_ushort(sb[(9 << ng_shift) + zg]));
      mma16816(sacc, a0, 0u, a2, 0u, p0, p1);
    }
    const unsigned char* rowp = wsm + WS_CODES;
    if constexpr (BITS == 1) {
      // block = 16 channels, four blocks per 64-channel half c; lane g reads block 4c + (g & 3) of tokens
      // 2tig, 2tig+1 (+8, +9) with 2-byte loads; rows g / g+8 of M-tile f are channels 4*(g>>2) + f and +8
      const unsigned char* tb = rowp + (t0 + 2 * tig) * 16 + 2 * (g & 3);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t r0 = pack_lo16(*reinterpret_cast<const uint16_t*>(tb + 8 * c), *reinterpret_cast<const uint16_t*>(tb + 8 * c + 16));
        const uint32_t r1 = pack_lo16(*reinterpret_cast<const uint16_t*>(tb + 8 * c + 128), *reinterpret_cast<const uint16_t*>(tb + 8 * c + 144));
        const uint32_t lo0 = r0 >> (4 * (g >> 2)), hi0 = lo0 >> 8, lo1 = r1 >> (4 * (g >> 2)), hi1 = lo1 >> 8;
#pragma unroll
        for (int f = 0; f < 4; ++f) {
          const uint32_t msk = 0x00010001u << f;
          mma16816(acc[4 * c + f], lo0 & msk, hi0 & msk, lo1 & msk, hi1 & msk, bh_[c][0], bh_[c][1]);
        }
#pragma unroll
        for (int f = 0; f < 4; ++f) {
          const uint32_t msk = 0x00010001u << f;
          mma16816(acc[4 * c + f], lo0 & msk, hi0 & msk, lo1 & msk, hi1 & msk, bl_[c][0], bl_[c][1]);
        }
      }
    } else if constexpr (BITS == 2) {
      uint32_t R[4];
      ldmatrix_x4_trans(R, rowp + TL::offset(t0 + lm_row, mi & 1));
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t lo0 = R[c], hi0 = R[c] >> 8, lo1 = R[2 + c], hi1 = R[2 + c] >> 8;
        uint32_t fa[4][4];
#pragma unroll
        for (int f = 0; f < 4; ++f) {
          fa[f][0] = v_field<2>(lo0, 0u, f), fa[f][1] = v_field<2>(hi0, 0u, f);
          fa[f][2] = v_field<2>(lo1, 0u, f), fa[f][3] = v_field<2>(hi1, 0u, f);
        }
#pragma unroll
        for (int f = 0; f < 4; ++f) mma16816(acc[4 * c + f], fa[f][0], fa[f][1], fa[f][2], fa[f][3], bh_[c][0], bh_[c][1]);
#pragma unroll
        for (int f = 0; f < 4; ++f) mma16816(acc[4 * c + f], fa[f][0], fa[f][1], fa[f][2], fa[f][3], bl_[c][0], bl_[c][1]);
      }
    } else if constexpr (BITS == 4) {
#pragma unroll
      for (int pp = 0; pp < 2; ++pp) {
        uint32_t R[4], S[4];
        ldmatrix_x4_trans(R, rowp + TL::offset(t0 + lm_row, 2 * pp + (mi & 1)));
#pragma unroll
        for (int k = 0; k < 4; ++k) S[k] = R[k] >> 8;
        uint32_t fa[4][4];
#pragma unroll
        for (int f = 0; f < 4; ++f)
#pragma unroll
          for (int k = 0; k < 4; ++k) fa[f][k] = v_field<4>(R[k], S[k], f);
#pragma unroll
        for (int f = 0; f < 4; ++f) mma16816(acc[4 * pp + f], fa[f][0], fa[f][1], fa[f][2], fa[f][3], bh_[pp][0], bh_[pp][1]);
#pragma unroll
        for (int f = 0; f < 4; ++f) mma16816(acc[4 * pp + f], fa[f][0], fa[f][1], fa[f][2], fa[f][3], bl_[pp][0], bl_[pp][1]);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          uint32_t R[4];
          ldmatrix_x4_trans(R, rowp + TL::offset(t0 + lm_row, 4 * q + u + 2 * (mi & 1)));
          uint32_t fa[2][4];
#pragma unroll
          for (int f = 0; f < 2; ++f)
#pragma unroll
            for (int k = 0; k < 4; ++k) fa[f][k] = v_field<8>(R[k], 0u, f);
#pragma unroll
          for (int f = 0; f < 2; ++f) mma16816(acc[4 * q + 2 * u + f], fa[f][0], fa[f][1], fa[f][2], fa[f][3], bh_[q][0], bh_[q][1]);
#pragma unroll
          for (int f = 0; f < 2; ++f) mma16816(acc[4 * q + 2 * u + f], fa[f][0], fa[f][1], fa[f][2], fa[f][3], bl_[q][0], bl_[q][1]);
        }
    }
    if (next_ntok > 0) {  // a quarter of this tile's rows is behind the walk: the next tile's rows may take their place
      constexpr int SPQ = TL::STEPS / 4;  // steps per quarter: 1 (8 bits) or 2
      if ((st + 1) % SPQ == 0) {
        __syncwarp();
        v_quarter_request(T, wsm, bh, next_t0, next_ntok, 128 >> gv_shift, st / SPQ);
      }
    }
  }
  if (BITS == 1 && normal) {  // value = std * C * (2 code - 1) + mean: the code-free term is sum_t p (mean - C std)
#pragma unroll
    for (int i = 0; i < 4; ++i) zacc[i] = fmaf(-HQKV_NORMAL1_CENTER, sacc[i], zacc[i]);
  }
  (void)T;
  (void)bh;
}

// Accumulators of one walk are ADDED to out[head of this half][channel] (every element has exactly one owner).
//   8 / 4 bits: rows 0-7 and 8-15 of an M-tile are two different channel groups: lanes tig 0,1 own row g
//               (columns 0-3), lanes tig 2,3 own row g+8 (columns 4-7).
//   2 bits:     rows g and g+8 are channels of the same block: lanes with (g < 4) == (tig < 2) own both.
// M-tile -> channels:  8 bits  mt = 4q + 2u + f : row g = 64q + 16u + 2g + f,  row g+8 = +32
//                      4 bits  mt = 4pp + f     : row g = 64pp + 4g + f,        row g+8 = +32
//                      2 bits  mt = 4c + f      : row g = 64c + 8g + f,         row g+8 = +4
//                      1 bit   mt = 4c + f      : row g = 64c + 16(g&3) + 4(g>>2) + f, row g+8 = +8
//                              (owned by the lanes with ((g & 3) < 2) == (tig < 2))
template <int BITS>
__device__ __forceinline__ void v_tile_store(float (*out)[D], const float (&acc)[8][4], float gain) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int hp = tig & 1, r = tig >> 1;
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    const int f = BITS == 8 ? (mt & 1) : (mt & 3);
    const float unscale = static_cast<float>(1 << (24 - VField<BITS>::shift(f))) * gain;
    if constexpr (BITS <= 2) {
      const bool mine = BITS == 2 ? (g < 4) == (tig < 2) : ((g & 3) < 2) == (tig < 2);
      if (mine) {
        const int ch = 64 * (mt >> 2) + (BITS == 2 ? 8 * g : 16 * (g & 3) + 4 * (g >> 2)) + f;
        constexpr int UP = BITS == 2 ? 4 : 8;  // channel distance of row g+8
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          out[2 * hp + e][ch] = fmaf(acc[mt][e], unscale, out[2 * hp + e][ch]);
          out[2 * hp + e][ch + UP] = fmaf(acc[mt][2 + e], unscale, out[2 * hp + e][ch + UP]);
        }
      }
    } else {
      const int ch = BITS == 8 ? 64 * (mt >> 2) + 16 * ((mt >> 1) & 1) + 2 * g + f + 32 * r
                               : 64 * (mt >> 2) + 4 * g + f + 32 * r;
#pragma unroll
      for (int e = 0; e < 2; ++e) out[2 * hp + e][ch] = fmaf(r ? acc[mt][2 + e] : acc[mt][e], unscale, out[2 * hp + e][ch]);
    }
  }
}

// Everything a warp does for one tile of a quantised V tier, already requested: probabilities of its
// tokens, then sum_t p_t * V_t added to the warp's partial output.
// Streaming (next_ntok > 0, only for a full tile): the next tile of the same tier and (batch, kv head) is requested
// into the same buffer during the last walk over this one.
template <int BITS>
__device__ __forceinline__ void v_tile(const TierDev& T, unsigned char* wsm, bool rep8, int rep, int L, int gv_shift,
                                       const float* gm, const float* gl, const uint32_t (&pos)[4], const float* logit0,
                                       __half* w0, const __half* pin0, int ntok, int bh, int next_t0, int next_ntok) {
  using TL = VTile<BITS>;
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int nh = rep8 ? 2 : 1;
  __half(*p_lo)[V_PROW] = reinterpret_cast<__half(*)[V_PROW]>(wsm + WS_V_P);
  __half(*p_hi)[V_PROW] = reinterpret_cast<__half(*)[V_PROW]>(wsm + WS_V_P + WS_V_P_BYTES);
  float(*out)[D] = reinterpret_cast<float(*)[D]>(wsm + ws_v_out(rep8));
  float* zt = reinterpret_cast<float*>(wsm + ws_v_zt(rep8));
  for (int hh = 0; hh < nh; ++hh)
    v_tile_probs<TL::TOKENS / 32>(gm, gl, pos, hh ? p_hi : p_lo, logit0, w0, pin0, L, rep, 4 * hh, ntok);
  cp_async_wait<0>();  // scales, zeros and codes (the gathers above took at least as long)
  __syncwarp();
  const bool normal = BITS == 1 && T.normal != 0;
  for (int hh = 0; hh < nh; ++hh) {
    float acc[8][4], zacc[4];
    v_tile_walk<BITS>(T, wsm, gv_shift, hh ? p_hi : p_lo, ntok, acc, zacc, normal, bh, next_t0, hh == nh - 1 ? next_ntok : 0);
    v_tile_store<BITS>(out + 4 * hh, acc, normal ? 2.f * HQKV_NORMAL1_CENTER : 1.f);
    if (g < 4 && tig < 2) {
      zt[g * MAX_REP + 4 * hh + 2 * tig] += zacc[0];
      zt[g * MAX_REP + 4 * hh + 2 * tig + 1] += zacc[1];
    }
  }
  __syncwarp();  // all lanes are done with the codes, the scales and the probability rows
}

// Storage format of the fp16 tiles: a "word" is what one thread loads for one (row, column) slot: eight halfs.
// One 16-deep contraction step over all M-tiles of a thread's slots:
//   w[p][r]: word of row-pair member p (0,1 -> fragment columns 2tig,2tig+1; 2,3 -> +8,+9) and row
//            slot r (0 -> fragment row g, 1 -> row g+8);  M-tile index = 2 * (32-bit lane of the word) + k.
template <int SUBI>
__device__ __forceinline__ void mma_f16_sub(float (&acc)[8][4], const uint4 (&w)[4][2], uint32_t b0, uint32_t b1) {
  auto pick = [](const uint4& v) { return SUBI == 0 ? v.x : SUBI == 1 ? v.y : SUBI == 2 ? v.z : v.w; };
  uint32_t a[2][4];
#pragma unroll
  for (int q = 0; q < 2; ++q)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint32_t x = pick(w[2 * q][r]), y = pick(w[2 * q + 1][r]);
      a[0][2 * q + r] = __byte_perm(x, y, 0x5410);
      a[1][2 * q + r] = __byte_perm(x, y, 0x7632);
    }
#pragma unroll
  for (int k = 0; k < 2; ++k) mma16816(acc[SUBI * 2 + k], a[k][0], a[k][1], a[k][2], a[k][3], b0, b1);
}

// fp16 tier and residual window, token-major rows [n][D] halfs: one 16-token step straight from global
// memory; B = p.  Adds the partial outputs of all (up to eight) heads to the warp's partial output.
__device__ __forceinline__ void v_plain_tile(const TierDev& T, unsigned char* wsm, bool rep8, int rep, int L, const float* gm,
                                             const float* gl, int bh, const float* logit0, __half* w0, const __half* pin0,
                                             int t0, int ntok, bool is_res) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  __half(*p_lo)[V_PROW] = reinterpret_cast<__half(*)[V_PROW]>(wsm + WS_V_P);
  __half(*p_hi)[V_PROW] = reinterpret_cast<__half(*)[V_PROW]>(wsm + WS_V_P + WS_V_P_BYTES);
  float(*out)[D] = reinterpret_cast<float(*)[D]>(wsm + ws_v_out(rep8));
  const uint4* base = reinterpret_cast<const uint4*>(T.v_data) + static_cast<int64_t>(bh) * T.n_v * 16;
  uint4 w[4][2];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int tl = 2 * tig + (p & 1) + (p >> 1) * 8;
    const int64_t tok = t0 + min(tl, ntok - 1);
#pragma unroll
    for (int s = 0; s < 2; ++s) w[p][s] = ld_stream(base + tok * 16 + s * 8 + g);
  }
  uint32_t pos[4] = {0u, 0u, 0u, 0u};
  if (lane < ntok) pos[0] = is_res ? static_cast<uint32_t>(L - T.n_v + t0 + lane) : ld_pos(T.v_idx + t0 + lane);
  for (int hh = 0; hh < (rep8 ? 2 : 1); ++hh)
    v_tile_probs<1>(gm, gl, pos, hh ? p_hi : p_lo, logit0, w0, pin0, L, rep, 4 * hh, ntok);
  __syncwarp();
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  uint32_t b0 = 0u, b1 = 0u;
  if (g < rep) {
    const __half* pr = g < 4 ? p_lo[g] : p_hi[g - 4];
    b0 = *reinterpret_cast<const uint32_t*>(pr + 2 * tig);
    b1 = *reinterpret_cast<const uint32_t*>(pr + 2 * tig + 8);
  }
  mma_f16_sub<0>(acc, w, b0, b1);
  mma_f16_sub<1>(acc, w, b0, b1);
  mma_f16_sub<2>(acc, w, b0, b1);
  mma_f16_sub<3>(acc, w, b0, b1);
  // M-tile mt, slot s: channel 8*(8s + g) + mt; columns 2tig, 2tig+1 = heads
#pragma unroll
  for (int mt = 0; mt < 8; ++mt)
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int ch = 8 * (s * 8 + g) + mt;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int h = 2 * tig + e;
        if (h < rep) out[h][ch] += acc[mt][s * 2 + e];
      }
    }
  __syncwarp();
}

}  // namespace hqkv
