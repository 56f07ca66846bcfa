// Fused mixed-precision decode attention over the tiered KV cache (sm_100a).
//
// Two launches per call:
//   k_pass : logits[h, pos] = scale * q_h . K^_pos for every tier (8/4/2/1-bit packed, fp16 tier,
//            fp16 residual), written to an fp32 scratch row at the tokens' logical positions,
//            plus one (max, sum-exp) pair per CTA and head.
//   v_pass : every CTA first folds the k_pass pairs into the global (max, sum) of its heads; each
//            warp then writes the normalised probabilities of its own tokens and accumulates
//            sum_t exp(logit_t - max) * V^_t over them; the CTA's partial output joins fp64
//            accumulators, and the last CTA of each (batch, kv head) normalises and writes fp16.
//
// The roofline is HBM: every packed word, scale and zero is read exactly once per call and is
// shared by all query heads of its kv head (GQA).  At 2-4 bits there are 1.6-2.7 codes per byte;
// four query heads need four FMAs per code, more than the FP32 pipes can issue at HBM speed, so the
// dot products run on the tensor pipe (mma.sync m16n8k16, fp32 accumulation).  Tiles of codes are
// staged in shared memory with 16-byte cp.async and read back with ldmatrix.trans, which delivers the
// two K-neighbours of an A fragment in one register; the codes enter the MMA as fp16 subnormals (one
// AND per pair) and the scale is folded into the B operand, carried exactly as hi + lo.
// Both kernels are chained with programmatic dependent launch: whatever a kernel needs only from the
// cache is requested before it waits for the kernel ahead of it.
#include <math.h>
#include <string.h>

#include "common.cuh"

namespace hqkv {

HQKV_DEFINE_CHECK_COUNTER

constexpr int D = 128;           // head dim
constexpr int MAX_REP = 8;       // query heads per kv head (n of the m16n8k16 tile)

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
  int k_chunk0, k_chunk_tokens;  // first chunk id of this tier in the k_pass grid, tokens per chunk
  int v_chunk0, v_chunk_tokens;
};

struct DecodeParams {
  TierDev tier[HQKV_NUM_TIERS + 1];  // [5] = fp16 residual window (token-major K and V)
  int B, H, nh_q, rep, rep_shift, L;
  int gk_shift, gv_shift;
  int nk_chunks, nv_chunks;
  float scale;
  const __half* q;
  const __half* mask;      // additive mask on the logits (null: none); element (b, head, pos) at b*bstride + head*hstride + pos
  long long mask_bstride, mask_hstride;
  const __half* probs_in;  // V pass on caller-supplied weights [B*nh_q][L] (null: softmax of the scratch logits)
  __half* head_sum;        // [L] sum of the probabilities over batch and heads, written by the V pass (null: not wanted)
  unsigned* hs_count;      // [nv_chunks] arrival counters of that sum
  __half* weights;
  __half* out;
  float* logits;   // [B*nh_q][L]
  float2* k_part;  // [B*H][nk_chunks][MAX_REP]
  double* v_acc;   // [B*H][rep][D] output accumulators: cleared by the K pass, summed into by the V pass
  __half* peer_out[HQKV_MAX_PEERS];  // copies of `out` in other GPUs' memory (kv-head sharding), n_peers used
  int n_peers;
  int peer_flagged;  // 1: peer_out are flagged 8-byte entries {two fp16 values, call number}, see peer_unpack_kernel
  // cross-GPU barrier run by the last CTA of the V pass (world == 0: none)
  unsigned* pad[HQKV_MAX_PEERS + 1];  // the ranks' signal pads, own one included
  int rank, world;
  unsigned* peer_state;  // call number, status, finished (batch, kv head) count
  long long max_spins;
  unsigned* counters;  // [B*H]
};


// ------------------------------------------------------------------------------------------------
// fragments
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

// Storage formats.  A "word" is what one thread loads for one (row, column) slot; it holds FPI
// values of one row.  SUB = independently decoded sub-units of a word (bytes of a packed word,
// 32-bit lanes of a uint4 of halfs), CPS = values per sub-unit.
template <int BITS>
struct Fmt;
template <>
struct Fmt<16> {
  using word_t = uint4;  // eight halfs
  static constexpr int FPI = 8, SUB = 4, CPS = 2;
};

// Decode sub-unit `sub` of the words wa (first row of the pair) and wb (second row) into CPS
// half2 values (value of row a in the low half, row b in the high half): v = code*scale + zero
// with one fp16 rounding; `sz` packs the scales of the two rows, `zz` their zeros.
template <int BITS>
struct Decode;

template <>
struct Decode<16> {
  template <int SUBI>
  static __device__ __forceinline__ void run(const uint4& wa, const uint4& wb, __half2, __half2, uint32_t (&out)[2]) {
    const uint32_t a = SUBI == 0 ? wa.x : SUBI == 1 ? wa.y : SUBI == 2 ? wa.z : wa.w;
    const uint32_t b = SUBI == 0 ? wb.x : SUBI == 1 ? wb.y : SUBI == 2 ? wb.z : wb.w;
    out[0] = __byte_perm(a, b, 0x5410);
    out[1] = __byte_perm(a, b, 0x7632);
  }
};

// One 16-deep contraction step over all M-tiles of a thread's slots.
//   w[p][r]: word of row-pair member p (0,1 -> fragment columns 2tig,2tig+1; 2,3 -> +8,+9) and row
//            slot r (0 -> fragment row g, 1 -> row g+8)
//   sz/zz[q][r]: scales/zeros of pair q (0: p=0,1; 1: p=2,3) for slot r
// M-tile index of sub-unit s, value k: s*CPS + k.
template <int BITS, int SUBI, int NM>
__device__ __forceinline__ void mma_sub(float (&acc)[NM][4], const typename Fmt<BITS>::word_t (&w)[4][2],
                                        const __half2 (&sz)[2][2], const __half2 (&zz)[2][2], uint32_t b0,
                                        uint32_t b1) {
  constexpr int CPS = Fmt<BITS>::CPS;
  uint32_t a0[CPS], a1[CPS], a2[CPS], a3[CPS];
  Decode<BITS>::template run<SUBI>(w[0][0], w[1][0], sz[0][0], zz[0][0], a0);
  Decode<BITS>::template run<SUBI>(w[0][1], w[1][1], sz[0][1], zz[0][1], a1);
  Decode<BITS>::template run<SUBI>(w[2][0], w[3][0], sz[1][0], zz[1][0], a2);
  Decode<BITS>::template run<SUBI>(w[2][1], w[3][1], sz[1][1], zz[1][1], a3);
#pragma unroll
  for (int k = 0; k < CPS; ++k) mma16816(acc[SUBI * CPS + k], a0[k], a1[k], a2[k], a3[k], b0, b1);
}

template <int BITS, int NM>
__device__ __forceinline__ void mma_words(float (&acc)[NM][4], const typename Fmt<BITS>::word_t (&w)[4][2],
                                          const __half2 (&sz)[2][2], const __half2 (&zz)[2][2], uint32_t b0,
                                          uint32_t b1) {
  constexpr int SUB = Fmt<BITS>::SUB;
  mma_sub<BITS, 0, NM>(acc, w, sz, zz, b0, b1);
  mma_sub<BITS, 1, NM>(acc, w, sz, zz, b0, b1);
  mma_sub<BITS, 2, NM>(acc, w, sz, zz, b0, b1);
  mma_sub<BITS, 3, NM>(acc, w, sz, zz, b0, b1);
  if constexpr (SUB == 8) {
    mma_sub<BITS, 4, NM>(acc, w, sz, zz, b0, b1);
    mma_sub<BITS, 5, NM>(acc, w, sz, zz, b0, b1);
    mma_sub<BITS, 6, NM>(acc, w, sz, zz, b0, b1);
    mma_sub<BITS, 7, NM>(acc, w, sz, zz, b0, b1);
  }
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
  l = l * fast_exp2((m - mx) * 1.4426950408889634f) + l2 * fast_exp2((m2 - mx) * 1.4426950408889634f);
  m = mx;
}


// ------------------------------------------------------------------------------------------------
// k_pass
// ------------------------------------------------------------------------------------------------
// Quantised K tier: rows = channels, packed words along tokens.  Every warp of a CTA owns one TILE:
// all 128 channel rows x 64 bytes of codes (32 bytes at 2 bits), i.e. 64 / 128 / 128 tokens at
// 8 / 4 / 2 bits, plus the tile's logical positions; the CTA shares the scale / zero rows of its 256
// or 512 tokens and q.  All of it is copied global -> shared with 16-byte cp.async as the first
// action (no registers are tied up, ~45 KB per CTA are in flight at once) and each warp then works
// out of shared memory in sub-spans of 64 tokens.  Wide copies in, ldmatrix out: the L1 data pipe
// moves 128 bytes per wavefront both ways.  (Per-lane loads of the 1-4 bytes a thread needs - from
// global or from shared memory - saturate that pipe at a quarter of the HBM bandwidth.)
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
constexpr int K_MIN_CTAS = 4;  // CTAs per SM the K pass is compiled for
constexpr int KWARPS = 4;
constexpr int KTHREADS = KWARPS * 32;
constexpr int K_SPAN = 64;                   // tokens per sub-span: four M-tiles of 16
constexpr int K_SLOT = 4;                    // fp16 tier: tokens per 8-byte slot
constexpr int K_TILE_BYTES = D * 64;         // codes of one tile
constexpr int K_MAX_TT = 128;                // tokens per tile at most
constexpr int K_CHUNK_GROUPS = KWARPS * K_MAX_TT / 32;  // scale groups per CTA at most (group size 32)
constexpr int K_RAW_HALFS = K_CHUNK_GROUPS + 8;         // staged halfs per channel row: three aligned 16-byte pieces
constexpr int K_TROW = MAX_REP + 1;          // floats per token row of the logit tile (odd: no bank conflicts)
constexpr float LOG2E = 1.4426950408889634f;

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

// global -> shared copies without a register round trip; completion = wait_group + barrier
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
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
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

struct KWarpShared {
  union {
    unsigned char codes[K_TILE_BYTES];
    float tile[64 * K_TROW];  // fp16 tier / residual: logits [token][head]
  } u;
  int64_t idx[K_MAX_TT];      // logical positions of the tile's tokens
  float zq[4][MAX_REP];       // sum_c zero*q per group of the tile and head
};

struct KShared {
  // B fragments of q per 16-channel step and lane: channels 16*kt + 2*tig + (0,1 | 8,9).  fp16 tier /
  // residual CTAs: [0] with column n = head n.  Quantised CTAs: [hh] with column n = head
  // 4*hh + (n & 3) (columns 4-7 repeat 0-3).
  uint2 qb[2][8][32];
  // scale / zero rows of the CTA's tokens as they lie in memory: channel c, three aligned 16-byte
  // pieces starting at or before the chunk's first group
  __half s[D][K_RAW_HALFS];
  __half z[D][K_RAW_HALFS];
  float red_m[KWARPS][MAX_REP], red_l[KWARPS][MAX_REP];
  KWarpShared w[KWARPS];
};

// Request the scale / zero rows of the CTA's chunk: thread t copies channel t.  The chunk's groups
// [g0c, g0c + ngc) of a channel are 2*ngc bytes at any 2-byte alignment; the (up to) three aligned
// 16-byte pieces that cover them go to shared memory as they are, so group gamma of channel c is
// half ((c*G + g0c) & 7) + gamma of row c.  (The planes hold B*H*128*G halfs, a multiple of 8, and
// start 16-byte aligned, so every aligned piece that begins inside a plane also ends inside it.)
__device__ __forceinline__ void k_scales_request(const DecodeParams& P, const TierDev& T, KShared& sh, int bh, int g0c,
                                                 int ngc) {
  const int ch = threadIdx.x;  // KTHREADS == D
  const int G = T.n_k >> P.gk_shift;
  const int64_t e0 = (static_cast<int64_t>(bh) * D + ch) * G + g0c;
  const int64_t a = e0 & ~static_cast<int64_t>(7);
#pragma unroll
  for (int p = 0; p < K_RAW_HALFS / 8; ++p)
    if (a + 8 * p < e0 + ngc) {
      cp_async_16(&sh.s[ch][8 * p], T.k_scale + a + 8 * p);
      cp_async_16(&sh.z[ch][8 * p], T.k_zero + a + 8 * p);
    }
}
static_assert(KTHREADS == D, "one thread per channel row");

// Request a tile: four commit groups, the codes of channel rows 0-31 (with the positions), 32-63,
// 64-95, 96-127 (two 16-channel steps each).  ntok = valid tokens of the tile (a multiple of 32).
template <int BITS>
__device__ __forceinline__ void k_tile_request(const TierDev& T, KWarpShared& ws, int bh, int tile_t0, int ntok) {
  using TL = KTile<BITS>;
  const int lane = threadIdx.x & 31;
  const int n = T.n_k;
#pragma unroll
  for (int j = 0; j < TL::TOKENS / 32; ++j) {
    const int t = lane + 32 * j;
    if (t < ntok) cp_async_8(&ws.idx[t], T.k_idx + tile_t0 + t);
  }
  const int64_t row_bytes = static_cast<int64_t>(n) * BITS / 8;
  const unsigned char* src = reinterpret_cast<const unsigned char*>(T.k_data) + static_cast<int64_t>(bh) * D * row_bytes +
                             static_cast<int64_t>(tile_t0) * BITS / 8;
  const int valid_bytes = ntok * BITS / 8;  // per row: a multiple of 8 (of 4 at 1 bit)
  if constexpr (BITS == 1) {
    // 16 bytes per row at 4-byte alignment: four 4-byte pieces; a copy instruction moves 8 rows
#pragma unroll
    for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = quarter * 32 + i * 8 + (lane >> 2), c4 = 4 * (lane & 3);
        if (c4 < valid_bytes) cp_async_4(ws.u.codes + row * 16 + c4, src + row * row_bytes + c4);
      }
      cp_async_commit();
    }
    return;
  }
  // a copy instruction moves 8 rows x 64 bytes (16 rows x 32 bytes at 2 bits)
  constexpr int LPR = BITS == 2 ? 2 : 4;    // lanes per row
  constexpr int RPI = 32 / LPR;             // rows per instruction
  const int c = lane % LPR, r0 = lane / LPR;
#pragma unroll
  for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
    for (int i = 0; i < 32 / RPI; ++i) {
      const int row = quarter * 32 + i * RPI + r0;
      const unsigned char* s = src + row * row_bytes + 16 * c;
      unsigned char* d = ws.u.codes + TL::offset(row, c);
      if constexpr (BITS == 2) {  // rows of 2-bit codes are only 8-byte aligned in memory
        if (16 * c < valid_bytes) cp_async_8(d, s);
        if (16 * c + 8 < valid_bytes) cp_async_8(d + 8, s + 8);
      } else {
        if (16 * c < valid_bytes) cp_async_16(d, s);
      }
    }
    cp_async_commit();
  }
}

// 16-bit halves of two words -> one half2 register (low half from a)
__device__ __forceinline__ uint32_t pack_lo16(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x5410); }

// Zq[group][head] of the tile for half hh of the heads: rows of the A operand are the tile's groups
// (at most four; rows 4-7 repeat them, rows 8-15 are zero).  zrow: this lane's two staged zero rows
// (channels 2*tig and 2*tig+1) at the half of the tile's first group.
// Gaussian-codebook tier (s_even / s_odd non-null: the std rows at the same halves): a value is
// std * C * (2 code - 1) + mean, so the term that does not depend on the code is sum_c (mean - C std) q.
__device__ __forceinline__ void k_tile_zq(KShared& sh, KWarpShared& ws, int hh, const __half* z_even, const __half* z_odd,
                                          const __half* s_even = nullptr, const __half* s_odd = nullptr) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int gam = g & 3;
  float zacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
  for (int kt = 0; kt < 8; ++kt) {
    const int o = (16 * kt) * K_RAW_HALFS + gam;
    const uint32_t a0 = pack_lo16(__half_as_ushort(z_even[o]), __half_as_ushort(z_odd[o]));
    const uint32_t a2 = pack_lo16(__half_as_ushort(z_even[o + 8 * K_RAW_HALFS]), __half_as_ushort(z_odd[o + 8 * K_RAW_HALFS]));
    const uint2 bq = sh.qb[hh][kt][lane];
    mma16816(zacc, a0, 0u, a2, 0u, bq.x, bq.y);
  }
  if (s_even) {
    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
    for (int kt = 0; kt < 8; ++kt) {
      const int o = (16 * kt) * K_RAW_HALFS + gam;
      const uint32_t a0 = pack_lo16(__half_as_ushort(s_even[o]), __half_as_ushort(s_odd[o]));
      const uint32_t a2 = pack_lo16(__half_as_ushort(s_even[o + 8 * K_RAW_HALFS]), __half_as_ushort(s_odd[o + 8 * K_RAW_HALFS]));
      const uint2 bq = sh.qb[hh][kt][lane];
      mma16816(sacc, a0, 0u, a2, 0u, bq.x, bq.y);
    }
    zacc[0] = fmaf(-HQKV_NORMAL1_CENTER, sacc[0], zacc[0]);
    zacc[1] = fmaf(-HQKV_NORMAL1_CENTER, sacc[1], zacc[1]);
  }
  __syncwarp();  // readers of the previous half are done
  if (g < 4 && tig < 2) {  // columns 0-3 are the four heads of this half; 4-7 repeat them
    ws.zq[g][2 * tig] = zacc[0];
    ws.zq[g][2 * tig + 1] = zacc[1];
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

// One tile of a quantised tier, already requested: all heads of this kv head.
// g0c = first scale group of the CTA's chunk.  m/l: this lane's running softmax pairs, [hh][e] for
// head 4*hh + 2*(tig&1) + e.
template <int BITS>
__device__ __forceinline__ void k_tile_compute(const DecodeParams& P, const TierDev& T, KShared& sh, KWarpShared& ws,
                                               int tile_t0, int ntok, int g0c, int nh, float* row0, const __half* mask0,
                                               float (&m)[2][2], float (&l)[2][2]) {
  using TL = KTile<BITS>;
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int G = T.n_k >> P.gk_shift;
  // staged scale / zero rows of this lane's channels 2*tig (even) and 2*tig+1 (odd) of step 0, at the
  // half of the chunk's first group; a step adds 16 rows, the +8 channels add 8 rows
  const int sh_even = static_cast<int>((static_cast<int64_t>(2 * tig) * G + g0c) & 7);
  const int sh_odd = static_cast<int>((static_cast<int64_t>(2 * tig + 1) * G + g0c) & 7);
  const int gt0 = (tile_t0 >> P.gk_shift) - g0c;  // first group of the tile within the chunk
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
  const float pscale = normal ? P.scale * (2.f * HQKV_NORMAL1_CENTER) : P.scale;

  for (int hh = 0; hh < nh; ++hh) {
    if (normal)
      k_tile_zq(sh, ws, hh, &sh.z[2 * tig][sh_even + gt0], &sh.z[2 * tig + 1][sh_odd + gt0], &sh.s[2 * tig][sh_even + gt0],
                &sh.s[2 * tig + 1][sh_odd + gt0]);
    else
      k_tile_zq(sh, ws, hh, &sh.z[2 * tig][sh_even + gt0], &sh.z[2 * tig + 1][sh_odd + gt0]);
    const uint2* qb = &sh.qb[hh][0][lane];
#pragma unroll 1
    for (int j = 0; j < TL::NSUB; ++j) {
      // as a B column this lane is n = g: columns 0-3 carry the scale group of tokens 0-31 of the
      // sub-span, columns 4-7 that of tokens 32-63
      const int gam = ((tile_t0 + j * K_SPAN + 32 * (g >> 2)) >> P.gk_shift) - g0c;
      const __half* s_even = &sh.s[2 * tig][sh_even + gam];
      const __half* s_odd = &sh.s[2 * tig + 1][sh_odd + gam];
      const unsigned char* kb = ws.u.codes + (BITS == 1 ? lm_off + j * 8 : (lm_off ^ (j * TL::CPS * 16)));
      const uint2* qk = qb;
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
      // two 16-channel steps per iteration (short loop body: the instruction cache is cold in every CTA
      // when the whole cache is one wave of CTAs)
#pragma unroll 1
      for (int kk = 0; kk < 4; ++kk) {
        if (hh == 0 && j == 0) {  // the codes arrive two steps at a time
          if (kk == 0) cp_async_wait<3>();
          else if (kk == 1) cp_async_wait<2>();
          else if (kk == 2) cp_async_wait<1>();
          else cp_async_wait<0>();
          __syncwarp();
        }
        uint32_t R2[4];  // 2 bits: one ldmatrix feeds both steps
        if constexpr (BITS == 2) ldmatrix_x4_trans(R2, kb);
        (void)R2;
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
          // A fragments: lo/hi of octet 0 -> registers 0/1 (channels 2tig, 2tig+1), of octet 1 -> 2/3 (+8)
          uint32_t a[4][4];  // [register][M-tile]
          if constexpr (BITS == 8) {
            uint32_t R[4];
            ldmatrix_x4_trans(R, kb + k2 * 16 * TL::PITCH);
            octet_frags<8>(R, a[0], a[1]);
            ldmatrix_x4_trans(R, kb + k2 * 16 * TL::PITCH + 8 * TL::PITCH);
            octet_frags<8>(R, a[2], a[3]);
          } else if constexpr (BITS == 4) {
            uint32_t R[4];
            ldmatrix_x4_trans(R, kb + k2 * 16 * TL::PITCH);
            octet_frags<4>(R, a[0], a[1]);
            octet_frags<4>(R + 2, a[2], a[3]);
          } else if constexpr (BITS == 2) {
            octet_frags<2>(R2 + 2 * k2, a[0], a[1]);
            octet_frags<2>(R2 + 2 * k2 + 1, a[2], a[3]);
          } else {
#pragma unroll
            for (int o = 0; o < 2; ++o) {  // channels 2tig, 2tig+1 (o = 0) and +8, +9 (o = 1)
              const unsigned char* cb = kb + (k2 * 16 + o * 8) * 16;
              const uint32_t t = pack_lo16(*reinterpret_cast<const uint16_t*>(cb), *reinterpret_cast<const uint16_t*>(cb + 16));
              const uint32_t lo = t >> (4 * (g >> 2)), hi = lo >> 8;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                a[2 * o][i] = lo & (0x00010001u << i);
                a[2 * o + 1][i] = hi & (0x00010001u << i);
              }
            }
          }
          const int o = (16 * k2) * K_RAW_HALFS;
          const __half2 s0 = u32_as_h2(pack_lo16(__half_as_ushort(s_even[o]), __half_as_ushort(s_odd[o])));
          const __half2 s1 = u32_as_h2(pack_lo16(__half_as_ushort(s_even[o + 8 * K_RAW_HALFS]),
                                                 __half_as_ushort(s_odd[o + 8 * K_RAW_HALFS])));
          const uint2 qv = qk[k2 * 32];
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
        kb += 32 * TL::PITCH;
        s_even += 32 * K_RAW_HALFS;
        s_odd += 32 * K_RAW_HALFS;
        qk += 64;
      }
      // Epilogue from registers: a lane keeps the accumulator columns whose scale group is its row's, and
      // every lane ends up with four tokens x two heads (heads 2*(tig&1), +1).
      //  8 / 4 bits: rows 0-7 are tokens 0-31, rows 8-15 tokens 32-63: lanes tig 0,1 own row g, lanes
      //              tig 2,3 own row g+8.
      //  2 bits:     rows g and g+8 are the eight tokens of block g, valid in the lanes with
      //              (g < 4) == (tig < 2); such a lane keeps the row of its tig half and hands the
      //              other row to lane tig ^ 2, whose own accumulators belong to the wrong scale group.
      //  1 bit:      the same with block g & 3: valid where ((g & 3) < 2) == (tig < 2).
      const int sub_t0 = j * K_SPAN;
      const int r = tig >> 1;
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
      // first of this lane's tokens (8 bits: tokens my_tok, +1, +16, +17; 4 and 2 bits: my_tok .. my_tok+3)
      const int my_tok = sub_t0 + (BITS == 8 ? 32 * r + 2 * g : BITS == 4 ? 32 * r + 4 * g : BITS == 2 ? 8 * g + 4 * r
                                                                : 16 * (g & 3) + 4 * (g >> 2) + 8 * r);
      const bool live = my_tok < ntok;
      const int my_gam = ((tile_t0 + my_tok) >> P.gk_shift) - g0c - gt0;
      uint32_t pos[4];
      if constexpr (BITS == 8) {
        const int4 pa = *reinterpret_cast<const int4*>(&ws.idx[my_tok]);  // low words of int64 positions: .x and .z
        const int4 pb = *reinterpret_cast<const int4*>(&ws.idx[my_tok + 16]);
        pos[0] = static_cast<uint32_t>(pa.x), pos[1] = static_cast<uint32_t>(pa.z);
        pos[2] = static_cast<uint32_t>(pb.x), pos[3] = static_cast<uint32_t>(pb.z);
      } else {
        const int4* ip = reinterpret_cast<const int4*>(&ws.idx[my_tok]);
        const int4 p01 = ip[0], p23 = ip[1];
        pos[0] = static_cast<uint32_t>(p01.x), pos[1] = static_cast<uint32_t>(p01.z);
        pos[2] = static_cast<uint32_t>(p23.x), pos[3] = static_cast<uint32_t>(p23.z);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int head = 4 * hh + 2 * hp + e;
        const bool on = live && head < P.rep;
        const float zqs = ws.zq[my_gam & 3][2 * hp + e] * P.scale;
        float* row = row0 + static_cast<int64_t>(head) * P.L;
        const __half* mrow = mask0 ? mask0 + head * P.mask_hstride : nullptr;
        float x[4];
        bool ok[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float unscale = static_cast<float>(1 << (24 - KField<BITS>::shift(i)));
          ok[i] = on && HQKV_INDEX_OK(pos[i], P.L);
          x[i] = ok[i] ? fmaf(val[i][e], pscale * unscale, zqs) : -INFINITY;
        }
        if (mrow) {  // one branch for the calls without a mask
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (ok[i]) x[i] += __half2float(mrow[pos[i]]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (ok[i]) row[pos[i]] = x[i];
        softmax_push4(m[hh][e], l[hh][e], x);
      }
    }
  }
}
// Write out a warp's logit tile [ntok][K_TROW] (already scaled) at the tokens' logical positions and
// leave the warp's (max, sum-exp) per head in red_m / red_l.  Element = (token, head) with the head
// fastest across lanes, so every lane owns ONE head for the whole call (rep divides 32): its running
// max and sum are scalars, and index loads and stores are spread over all 32 lanes.
// (fp16 tier and residual window only; the quantised tiers write from registers.)
__device__ __forceinline__ void k_write_tile(const DecodeParams& P, float* tile, int ntok, const int64_t* idx,
                                             int64_t first_pos, int b, int kvh, float* red_m, float* red_l) {
  const int lane = threadIdx.x & 31;
  const int rep = P.rep, rshift = P.rep_shift;
  const int h = lane & (rep - 1);
  float* row = P.logits + (static_cast<int64_t>(b) * P.nh_q + kvh * rep + h) * P.L;
  const __half* mrow = P.mask ? P.mask + b * P.mask_bstride + static_cast<int64_t>(kvh * rep + h) * P.mask_hstride : nullptr;
  const int tpr = 32 >> rshift;  // tokens per round
  float mx = -INFINITY;
#pragma unroll 2
  for (int t = lane >> rshift; t < ntok; t += tpr) {
    const int64_t pos = idx ? idx[t] : first_pos + t;
    float x = -INFINITY;
    if (HQKV_INDEX_OK(pos, P.L)) {
      x = tile[t * K_TROW + h];
      if (mrow) x += __half2float(mrow[pos]);
      row[pos] = x;
    }
    tile[t * K_TROW + h] = x;  // the masked value is what the sum below sees
    mx = fmaxf(mx, x);
  }
  for (int off = rep; off < 32; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  const float ref = mx == -INFINITY ? 0.f : mx;  // every position masked out: the sum is 0, not NaN
  float sum = 0.f;
#pragma unroll 2
  for (int t = lane >> rshift; t < ntok; t += tpr) sum += fast_exp2((tile[t * K_TROW + h] - ref) * LOG2E);
  for (int off = rep; off < 32; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (lane < rep) {
    red_m[lane] = mx;
    red_l[lane] = sum;
  }
}


// One tile per warp: request everything that depends only on the cache, wait for the kernels before
// this one, fetch q, agree that q and the scale rows are in shared memory, compute.
template <int BITS, typename LoadQ>
__device__ __forceinline__ void k_chunk(const DecodeParams& P, const TierDev& T, KShared& sh, int bh, int b, int kvh,
                                        int chunk_t0, int nh, LoadQ load_q) {
  using TL = KTile<BITS>;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  KWarpShared& ws = sh.w[warp];
  const int chunk_end = min(chunk_t0 + KWARPS * TL::TOKENS, T.n_k);
  const int g0c = chunk_t0 >> P.gk_shift;
  const int ngc = ((chunk_end - 1) >> P.gk_shift) - g0c + 1;
  k_scales_request(P, T, sh, bh, g0c, ngc);
  cp_async_commit();  // oldest group: the scale / zero rows
  const int tile_t0 = chunk_t0 + warp * TL::TOKENS;
  const int ntok = min(TL::TOKENS, T.n_k - tile_t0);  // <= 0: this warp has no tile
  if (ntok > 0) k_tile_request<BITS>(T, ws, bh, tile_t0, ntok);
  // Everything above reads only the cache.  From here on this grid reads q and writes the scratch that
  // the previous decode call of the stream may still be using: wait for the kernels before it.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  load_q();
  if (ntok > 0) {
    cp_async_wait<4>();
  } else {
    cp_async_wait<0>();
  }
  __syncthreads();
  float m[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, l[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  if (ntok > 0) {
    float* row0 = P.logits + (static_cast<int64_t>(b) * P.nh_q + kvh * P.rep) * P.L;
    // additive mask rows of this kv head's query heads (null: none)
    const __half* mask0 = P.mask ? P.mask + b * P.mask_bstride + static_cast<int64_t>(kvh * P.rep) * P.mask_hstride : nullptr;
    k_tile_compute<BITS>(P, T, sh, ws, tile_t0, ntok, g0c, nh, row0, mask0, m, l);
  }
  // the warp's (max, sum-exp) per head: lanes that share tig & 1 hold pairs of the same two heads
  for (int hh = 0; hh < nh; ++hh)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float mx = m[hh][e];
#pragma unroll
      for (int o = 2; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = l[hh][e] * fast_exp2((m[hh][e] - (mx == -INFINITY ? 0.f : mx)) * LOG2E);
#pragma unroll
      for (int o = 2; o < 32; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane < 2) {
        sh.red_m[warp][4 * hh + 2 * lane + e] = mx;
        sh.red_l[warp][4 * hh + 2 * lane + e] = sum;
      }
    }
}

// fp16 tier, channel-major rows [D][n]: four tokens per 8-byte slot, no scales; B = q exactly.
__device__ __forceinline__ void k_f16_span(const DecodeParams& P, const TierDev& T, KShared& sh, int bh, int b, int kvh,
                                           int span_t0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tig = lane & 3;
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
    const uint2 bq = sh.qb[0][kt][lane];
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
#pragma unroll
    for (int i = 0; i < K_SLOT; ++i) mma16816(acc[i], a[i][0], a[i][1], a[i][2], a[i][3], bq.x, bq.y);
  }
  float* tile = sh.w[warp].u.tile;
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int e = 0; e < 2; ++e)
#pragma unroll
      for (int i = 0; i < K_SLOT; ++i)
        tile[((r * 8 + g) * K_SLOT + i) * K_TROW + 2 * tig + e] = acc[i][r * 2 + e] * P.scale;
  __syncwarp();
  k_write_tile(P, tile, min(K_SPAN, n - span_t0), T.k_idx + span_t0, 0, b, kvh, sh.red_m[warp], sh.red_l[warp]);
}

// fp16 residual window, token-major [r][D]: A fragments are read directly; one 16-token tile per warp.
__device__ __forceinline__ void k_residual_tile(const DecodeParams& P, const TierDev& T, KShared& sh, int bh, int b,
                                                int kvh, int tile_t0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tig = lane & 3;
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
    const uint2 bq = sh.qb[0][kt][lane];
    mma16816(acc, a[kt][0], a[kt][1], a[kt][2], a[kt][3], bq.x, bq.y);
  }
  float* tile = sh.w[warp].u.tile;
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int e = 0; e < 2; ++e) tile[(r * 8 + g) * K_TROW + 2 * tig + e] = acc[r * 2 + e] * P.scale;
  __syncwarp();
  k_write_tile(P, tile, min(16, n - tile_t0), nullptr, static_cast<int64_t>(P.L) - n + tile_t0, b, kvh, sh.red_m[warp],
               sh.red_l[warp]);
}

__global__ void __launch_bounds__(KTHREADS, K_MIN_CTAS) k_pass_kernel(const __grid_constant__ DecodeParams P) {
  extern __shared__ __align__(128) unsigned char k_smem[];
  KShared& sh = *reinterpret_cast<KShared*>(k_smem);
  const int chunk = blockIdx.y, bh = blockIdx.x;  // (batch, head) fastest: neighbouring CTAs run the same tier code
  const int b = bh / P.H, kvh = bh - b * P.H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;

  // Let the V pass of this call (launched with programmatic stream serialisation) start its own
  // prologue - V words, index lists, scale/zero tiles - as soon as SM resources free up; it waits for
  // this grid to finish (griddepcontrol.wait) before it touches the logits or the softmax pairs.
  asm volatile("griddepcontrol.launch_dependents;");
  if (tid < KWARPS * MAX_REP) {
    (&sh.red_m[0][0])[tid] = -INFINITY;
    (&sh.red_l[0][0])[tid] = 0.f;
  }

  int ti = HQKV_NUM_TIERS;
#pragma unroll
  for (int t = 0; t < HQKV_NUM_TIERS; ++t)
    if (chunk >= P.tier[t].k_chunk0 && chunk < P.tier[t + 1].k_chunk0) ti = t;
  const TierDev& T = P.tier[ti];
  const int chunk_t0 = (chunk - T.k_chunk0) * T.k_chunk_tokens;
  const bool plain = ti == HQKV_NUM_TIERS || T.bits == 16;

  // B fragments of q: rows are channels 16*kt + 2*tig + (0,1 | 8,9), column n = g is a query head of
  // this kv head (see KShared::qb); warp hh stores its half.  q is the only input that an earlier
  // kernel of the stream may still be writing, so it is read after griddepcontrol.wait.
  const int nh = (!plain && P.rep > 4) ? 2 : 1;
  auto load_q = [&]() {
    if (warp < nh) {
      const int head = plain ? g : 4 * warp + (g & 3);
      const __half* qh = P.q + (static_cast<int64_t>(b) * P.nh_q + kvh * P.rep + head) * D + 2 * tig;
      uint2 qf[8];
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
        qf[kt] = make_uint2(0u, 0u);
        if (head < P.rep) {
          qf[kt].x = *reinterpret_cast<const uint32_t*>(qh + 16 * kt);
          qf[kt].y = *reinterpret_cast<const uint32_t*>(qh + 16 * kt + 8);
        }
      }
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) sh.qb[warp][kt][lane] = qf[kt];
    }
  };

  if (plain) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    load_q();
    __syncthreads();
    const int chunk_end = min(chunk_t0 + T.k_chunk_tokens, T.n_k);
    if (ti == HQKV_NUM_TIERS) {
      const int t0 = chunk_t0 + warp * 16;  // residual chunks are KWARPS * 16 tokens
      if (t0 < chunk_end) k_residual_tile(P, T, sh, bh, b, kvh, t0);
    } else {
      const int t0 = chunk_t0 + warp * K_SPAN;
      if (t0 < chunk_end) k_f16_span(P, T, sh, bh, b, kvh, t0);
    }
  } else if (T.bits == 8) {
    k_chunk<8>(P, T, sh, bh, b, kvh, chunk_t0, nh, load_q);
  } else if (T.bits == 4) {
    k_chunk<4>(P, T, sh, bh, b, kvh, chunk_t0, nh, load_q);
  } else if (T.bits == 2) {
    k_chunk<2>(P, T, sh, bh, b, kvh, chunk_t0, nh, load_q);
  } else {
    k_chunk<1>(P, T, sh, bh, b, kvh, chunk_t0, nh, load_q);
  }

  // the output accumulators of this (batch, kv head) start from zero in every call (the V pass, which
  // adds into them, starts after this grid has finished); both branches above have passed their
  // griddepcontrol.wait, so the previous call is done with them
  if (chunk == 0) {
    double* accum = P.v_acc + static_cast<int64_t>(bh) * P.rep * D;
    for (int i = tid; i < P.rep * D; i += KTHREADS) accum[i] = 0.0;
  }
  // (max, sum) of this CTA per head from the warps' pairs
  __syncthreads();
  if (tid < MAX_REP) {
    float m = sh.red_m[0][tid], l = sh.red_l[0][tid];
    for (int w = 1; w < KWARPS; ++w) softmax_merge(m, l, sh.red_m[w][tid], sh.red_l[w][tid]);
    P.k_part[(static_cast<int64_t>(bh) * P.nk_chunks + chunk) * MAX_REP + tid] = make_float2(m, l);
  }
}

// ------------------------------------------------------------------------------------------------
// v_pass
// ------------------------------------------------------------------------------------------------
// V tier, token-major rows of 128 channels.  Every warp of a CTA owns one TILE of consecutive tokens
// (8 KB of codes at 8 / 4 bits = 64 / 128 tokens, 4 KB at 2 bits = 128 tokens) with their scales,
// zeros and logical positions, all copied global -> shared with cp.async before anything else.
// The contraction runs over tokens, 16 per step.  ldmatrix.trans over 8 token rows x 16 bytes hands
// lane (g, tig) the 16-bit block g (2 / 4 / 8 channels) of tokens 2*tig and 2*tig+1 in one register:
// the two K-neighbours of an m16n8k16 A fragment.  As in the K pass the codes enter the tensor pipe
// as fp16 subnormals (one AND per pair of codes) and the scale - here per token and 32-channel
// group - is folded into the B operand: out[h][c] = sum_t (p_t * scale_t,G) * code_t,c + sum_t p_t *
// zero_t,G, with p*scale carried exactly as hi + lo and B columns 0-3 / 4-7 holding the two channel
// groups of a 64-channel half.  The zero term is one small MMA per step (rows = groups).
constexpr int V_MIN_CTAS = 4;  // CTAs per SM the V pass is compiled for
constexpr int VWARPS = 4;
constexpr int VTHREADS = VWARPS * 32;
constexpr int V_MAX_TT = 128;                 // tokens per tile at most
constexpr int V_PROW = V_MAX_TT + 8;          // halfs per staged probability row (pitch 68 words: rows 4 banks apart)

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

struct VWarpShared {
  union {
    unsigned char codes[8192];
    float red[4][D];            // partial output of the last walk over the tile (heads of that half)
  } u;
  union {
    struct {
      int64_t pos[V_MAX_TT];    // logical positions of the tile's tokens
      __half p[4][V_PROW];      // exp(logit - max) of heads 0-3
    } a;
    float red0[4][D];           // eight query heads per kv head: partial output of the first walk
  } v;
  __half p_hi[4][V_PROW];       // heads 4-7
  __half s[V_MAX_TT * 4];       // scales as in memory: [token][group]
  __half z[V_MAX_TT * 4];
  float zt[4][MAX_REP];         // sum_t p*zero per channel group and head
};
static_assert(sizeof(float) * 4 * D <= sizeof(int64_t) * V_MAX_TT + sizeof(__half) * 4 * V_PROW, "red0 fits its union");

// importance row emitted by the V pass: staging limits (positions + per-head halfs live in the warps' tile buffers)
constexpr int HS_TOKENS = 512;   // tokens of the largest chunk
constexpr int HS_HEADS = 32;     // query heads it is built for (beyond that a separate launch sums the heads)
struct VShared {
  float gm[MAX_REP], gl[MAX_REP];          // global max / sum of this kv head's query heads
  float wm[VWARPS][MAX_REP], wl[VWARPS][MAX_REP];
  unsigned is_last;
  unsigned pad_[3 + 12];
  VWarpShared w[VWARPS];
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

// Request a tile: positions, scales, zeros in the oldest commit group, then the codes in four groups
// of a quarter of the steps each.  ntok = valid tokens (a multiple of 32), ng = channel groups.
template <int BITS>
__device__ __forceinline__ void v_tile_request(const TierDev& T, VWarpShared& ws, int bh, int tile_t0, int ntok, int ng) {
  using TL = VTile<BITS>;
  const int lane = threadIdx.x & 31;
  const int64_t tok0 = static_cast<int64_t>(bh) * T.n_v + tile_t0;
#pragma unroll
  for (int j = 0; j < TL::TOKENS / 32; ++j) {
    const int t = lane + 32 * j;
    if (t < ntok) cp_async_8(&ws.v.a.pos[t], T.v_idx + tile_t0 + t);
  }
  // scale / zero rows are ng halfs per token, contiguous over the tile: 8-byte pieces
  {
    const int bytes = ntok * ng * 2;
    const unsigned char* s = reinterpret_cast<const unsigned char*>(T.v_scale + tok0 * ng);
    const unsigned char* z = reinterpret_cast<const unsigned char*>(T.v_zero + tok0 * ng);
#pragma unroll
    for (int j = 0; j < V_MAX_TT * 4 * 2 / (32 * 8); ++j) {
      const int o = (lane + 32 * j) * 8;
      if (o < bytes) {
        cp_async_8(reinterpret_cast<unsigned char*>(ws.s) + o, s + o);
        cp_async_8(reinterpret_cast<unsigned char*>(ws.z) + o, z + o);
      }
    }
  }
  cp_async_commit();
  const unsigned char* src = reinterpret_cast<const unsigned char*>(T.v_data) + tok0 * TL::PITCH;
  constexpr int PIECES = TL::TOKENS * TL::NPIECE;  // 512 (256 at 2 bits, 128 at 1 bit)
  constexpr int PER_Q = PIECES / 4 / 32;           // copies per lane and quarter: 4 (2, 1)
#pragma unroll
  for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
    for (int i = 0; i < PER_Q; ++i) {
      const int id = (quarter * PER_Q + i) * 32 + lane;
      const int row = id / TL::NPIECE, c = id % TL::NPIECE;
      if (row < ntok) cp_async_16(ws.u.codes + TL::offset(row, c), src + static_cast<int64_t>(id) * 16);
    }
    cp_async_commit();
  }
}

// exp(logit - max) of the tile's tokens for heads h0..h0+3 into prow[0..3][token], and the
// normalised probabilities into the output row; the gathers of four heads are in flight together.
template <int TOKENS>
__device__ __forceinline__ void v_tile_probs(const DecodeParams& P, const VShared& sh, const int64_t* pos_s, __half (*prow)[V_PROW],
                                             int b, int kvh, int h0, int ntok, int64_t first_pos) {
  const int lane = threadIdx.x & 31;
  const int rep = P.rep;
  constexpr int PER = TOKENS / 32;
  uint32_t pos[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int t = lane + 32 * j;
    pos[j] = t < ntok ? (pos_s ? static_cast<uint32_t>(pos_s[t]) : static_cast<uint32_t>(first_pos + t)) : 0u;
  }
  bool ok[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) ok[j] = lane + 32 * j < ntok && HQKV_INDEX_OK(pos[j], P.L);
  if (P.probs_in) {
    // caller-supplied weights: staged as they are, nothing is written back
#pragma unroll 1
    for (int hh = 0; hh < 4; ++hh) {
      const int h = h0 + hh;
      const unsigned short* row = reinterpret_cast<const unsigned short*>(P.probs_in) +
                                  (static_cast<int64_t>(b) * P.nh_q + kvh * rep + min(h, rep - 1)) * P.L;
#pragma unroll
      for (int j = 0; j < PER; ++j)
        prow[hh][lane + 32 * j] = __ushort_as_half((h < rep && ok[j]) ? __ldcg(row + pos[j]) : static_cast<unsigned short>(0));
    }
    return;
  }
  float x[4][PER];
#pragma unroll
  for (int hh = 0; hh < 4; ++hh) {
    const int h = min(h0 + hh, rep - 1);
    const float* row = P.logits + (static_cast<int64_t>(b) * P.nh_q + kvh * rep + h) * P.L;
#pragma unroll
    for (int j = 0; j < PER; ++j) x[hh][j] = ok[j] ? __ldcg(row + pos[j]) : -INFINITY;
  }
#pragma unroll
  for (int hh = 0; hh < 4; ++hh) {
    const int h = h0 + hh;
    const bool on = h < rep;
    const float mh = on ? sh.gm[h] * LOG2E : 0.f, inv = on ? 1.f / sh.gl[h] : 0.f;
    __half* wrow = P.weights + (static_cast<int64_t>(b) * P.nh_q + kvh * rep + min(h, rep - 1)) * P.L;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int t = lane + 32 * j;
      const float e = on ? fast_exp2(fmaf(x[hh][j], LOG2E, -mh)) : 0.f;  // exp2(-inf) = 0 beyond the tile
      prow[hh][t] = __float2half_rn(e);
      if (on && ok[j]) wrow[pos[j]] = __float2half_rn(e * inv);
    }
  }
}

// One tile of a quantised V tier for half hh of the heads: acc[mt] = M-tile mt of the output
// (channels x heads, see the channel map in v_tile_store), zacc = zero term rows.
template <int BITS>
__device__ __forceinline__ void v_tile_walk(const DecodeParams& P, VWarpShared& ws, const __half (*prow)[V_PROW], int ntok,
                                            float (&acc)[8][4], float (&zacc)[4], bool normal) {
  using TL = VTile<BITS>;
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int ng_shift = 7 - P.gv_shift;  // log2(groups per token): 2, 1, 0
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
  for (int q = 0; q < 2; ++q) gq[q] = (64 * q + 32 * (g >> 2)) >> P.gv_shift;
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
    const __half* sb = ws.s + ((t0 + 2 * tig) << ng_shift);
    const __half* zb = ws.z + ((t0 + 2 * tig) << ng_shift);
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
    const unsigned char* rowp = ws.u.codes;
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
  }
  if (BITS == 1 && normal) {  // value = std * C * (2 code - 1) + mean: the code-free term is sum_t p (mean - C std)
#pragma unroll
    for (int i = 0; i < 4; ++i) zacc[i] = fmaf(-HQKV_NORMAL1_CENTER, sacc[i], zacc[i]);
  }
}

// Accumulators of one walk -> red[head of this half][channel] (every element has exactly one owner).
//   8 / 4 bits: rows 0-7 and 8-15 of an M-tile are two different channel groups: lanes tig 0,1 own row g
//               (columns 0-3), lanes tig 2,3 own row g+8 (columns 4-7).
//   2 bits:     rows g and g+8 are channels of the same block: lanes with (g < 4) == (tig < 2) own both.
// M-tile -> channels:  8 bits  mt = 4q + 2u + f : row g = 64q + 16u + 2g + f,  row g+8 = +32
//                      4 bits  mt = 4pp + f     : row g = 64pp + 4g + f,        row g+8 = +32
//                      2 bits  mt = 4c + f      : row g = 64c + 8g + f,         row g+8 = +4
//                      1 bit   mt = 4c + f      : row g = 64c + 16(g&3) + 4(g>>2) + f, row g+8 = +8
//                              (owned by the lanes with ((g & 3) < 2) == (tig < 2))
template <int BITS>
__device__ __forceinline__ void v_tile_store(float (*red)[D], const float (&acc)[8][4], float gain) {
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
          red[2 * hp + e][ch] = acc[mt][e] * unscale;
          red[2 * hp + e][ch + UP] = acc[mt][2 + e] * unscale;
        }
      }
    } else {
      const int ch = BITS == 8 ? 64 * (mt >> 2) + 16 * ((mt >> 1) & 1) + 2 * g + f + 32 * r
                               : 64 * (mt >> 2) + 4 * g + f + 32 * r;
#pragma unroll
      for (int e = 0; e < 2; ++e) red[2 * hp + e][ch] = (r ? acc[mt][2 + e] : acc[mt][e]) * unscale;
    }
  }
}

// Everything a warp does for its tile of a quantised V tier.
template <int BITS>
__device__ __forceinline__ void v_tile(const DecodeParams& P, const TierDev& T, VShared& sh, VWarpShared& ws, int b,
                                       int kvh, int ntok, int nh) {
  using TL = VTile<BITS>;
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  cp_async_wait<4>();  // positions, scales, zeros
  __syncwarp();
  for (int hh = 0; hh < nh; ++hh)
    v_tile_probs<TL::TOKENS>(P, sh, ws.v.a.pos, hh ? ws.p_hi : ws.v.a.p, b, kvh, 4 * hh, ntok, 0);
  cp_async_wait<0>();  // the gathers above took at least as long as the codes
  __syncwarp();
  for (int hh = 0; hh < nh; ++hh) {
    float acc[8][4], zacc[4];
    const bool normal = BITS == 1 && T.normal != 0;
    v_tile_walk<BITS>(P, ws, hh ? ws.p_hi : ws.v.a.p, ntok, acc, zacc, normal);
    __syncwarp();  // all lanes are done with the codes (last walk) or with p of heads 0-3 (first of two)
    v_tile_store<BITS>(hh + 1 < nh ? ws.v.red0 : ws.u.red, acc, normal ? 2.f * HQKV_NORMAL1_CENTER : 1.f);
    if (g < 4 && tig < 2) {
      ws.zt[g][4 * hh + 2 * tig] = zacc[0];
      ws.zt[g][4 * hh + 2 * tig + 1] = zacc[1];
    }
  }
}

// fp16 tier and residual window, token-major rows [n][D] halfs: one 16-token step per warp straight
// from global memory; B = p.  Writes the partial outputs of all (up to eight) heads.
__device__ __forceinline__ void v_plain_tile(const DecodeParams& P, const TierDev& T, VShared& sh, VWarpShared& ws, int bh,
                                             int b, int kvh, int t0, int ntok, bool is_res) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int rep = P.rep;
  const uint4* base = reinterpret_cast<const uint4*>(T.v_data) + static_cast<int64_t>(bh) * T.n_v * 16;
  uint4 w[4][2];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int tl = 2 * tig + (p & 1) + (p >> 1) * 8;
    const int64_t tok = t0 + min(tl, ntok - 1);
#pragma unroll
    for (int s = 0; s < 2; ++s) w[p][s] = ld_stream(base + tok * 16 + s * 8 + g);
  }
  const int64_t first_pos = static_cast<int64_t>(P.L) - T.n_v + t0;
  for (int hh = 0; hh < (rep > 4 ? 2 : 1); ++hh)
    v_tile_probs<32>(P, sh, is_res ? nullptr : T.v_idx + t0, hh ? ws.p_hi : ws.v.a.p, b, kvh, 4 * hh, ntok, first_pos);
  __syncwarp();
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  uint32_t b0 = 0u, b1 = 0u;
  if (g < rep) {
    const __half* pr = g < 4 ? ws.v.a.p[g] : ws.p_hi[g - 4];
    b0 = *reinterpret_cast<const uint32_t*>(pr + 2 * tig);
    b1 = *reinterpret_cast<const uint32_t*>(pr + 2 * tig + 8);
  }
  const __half2 none[2][2] = {};
  mma_words<16, 8>(acc, w, none, none, b0, b1);
  __syncwarp();
  // M-tile mt, slot s: channel 8*(8s + g) + mt; columns 2tig, 2tig+1 = heads
#pragma unroll
  for (int mt = 0; mt < 8; ++mt)
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int ch = 8 * (s * 8 + g) + mt;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int h = 2 * tig + e;  // heads 0-3 are the first of two halves when there are eight
        if (rep > 4) {
          (h < 4 ? ws.v.red0 : ws.u.red)[h & 3][ch] = acc[mt][s * 2 + e];
        } else if (h < 4) {
          ws.u.red[h][ch] = acc[mt][s * 2 + e];
        }
      }
    }
}

// Cross-GPU barrier of one call, run by up to `world` threads of one CTA: thread r tells peer r "my stores
// of call number n are done" by raising a counter in the peer's signal pad, then waits until peer r has
// told it the same.  The call number lives in device memory and is advanced here, so the launch can
// sit in a CUDA graph that is replayed.  Every wait is bounded: after max_spins polls the thread gives
// up, records which peer was missing in the status word and returns, so a rank that died cannot hang
// the others' GPUs (the step's gathered data is then incomplete; the host checks the status).
template <bool FENCE_FIRST>
__device__ __forceinline__ void peer_barrier_device(unsigned* const* pad, int rank, int world, unsigned* call_no,
                                                    int* status, long long max_spins, unsigned* shared_n) {
  const int r = threadIdx.x;
  if (r == 0) *shared_n = *call_no + 1u;
  __syncthreads();
  const unsigned n = *shared_n;
  if (r < world && r != rank) {
    if (FENCE_FIRST) __threadfence_system();  // this GPU's earlier peer stores first (the V pass has fenced them already)
    atomicAdd_system(pad[r] + rank, 1u);      // slot `rank` of peer r's pad counts my arrivals
    volatile unsigned* mine = pad[rank] + r;  // slot r of my pad counts peer r's arrivals
    long long spins = 0;
    while (static_cast<int>(*mine - n) < 0) {
      if (++spins > max_spins) {
        atomicExch(status, r + 1);  // gave up waiting for peer r
        break;
      }
      __nanosleep(20);
    }
    __threadfence_system();
  }
  __syncthreads();
  if (r == 0) *call_no = n;
}

static_assert(sizeof(VWarpShared) * VWARPS >= HS_TOKENS * 4 + HS_TOKENS * HS_HEADS * 2, "importance-row staging fits the tile buffers");
// Importance row of one chunk of tokens, run by the last CTA to finish it (not inlined: its registers are its own).
__device__ __noinline__ void head_sum_chunk(const DecodeParams& P, const TierDev& T, VShared& sh, int chunk, bool is_res) {
  const int tid = threadIdx.x;
  __threadfence();
  const int c0 = (chunk - T.v_chunk0) * T.v_chunk_tokens;
  const int n = min(T.v_chunk_tokens, T.n_v - c0);
  // The warps' tile buffers are free by now: they stage the chunk's positions and, per token and head, the sum
  // over the batch rounded to fp16.  Loads first, all of them independent: an item is (token, eight heads),
  // four items - 32 gathers per batch entry - are in flight per thread; then one thread per token adds the
  // heads in head order.
  uint32_t* pos_s = reinterpret_cast<uint32_t*>(sh.w);                       // [HS_TOKENS]
  __half* stage = reinterpret_cast<__half*>(pos_s + HS_TOKENS);              // [HS_TOKENS][HS_HEADS]
  for (int t = tid; t < n; t += VTHREADS)
    pos_s[t] = is_res ? static_cast<uint32_t>(P.L - T.n_v + c0 + t) : static_cast<uint32_t>(T.v_idx[c0 + t]);
  __syncthreads();
  const int nhq = P.nh_q, ngr = (nhq + 7) >> 3, items = n * ngr;
  const unsigned short* w = reinterpret_cast<const unsigned short*>(P.weights);
  for (int base = tid; base < items; base += 4 * VTHREADS) {
    float ob[4][8];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int j = 0; j < 8; ++j) ob[q][j] = 0.f;
    for (int bb = 0; bb < P.B; ++bb) {
      unsigned short v[4][8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int item = base + q * VTHREADS;
        const int gq = item / n, t = item - gq * n;  // token fastest: neighbouring threads read neighbouring positions
        const bool live = item < items && HQKV_INDEX_OK(pos_s[t], P.L);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int h = 8 * gq + j;
          v[q][j] = (live && h < nhq) ? __ldcg(w + (static_cast<int64_t>(bb) * nhq + h) * P.L + pos_s[t])
                                      : static_cast<unsigned short>(0);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[q][j] = __fadd_rn(ob[q][j], __half2float(__ushort_as_half(v[q][j])));
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int item = base + q * VTHREADS;
      if (item >= items) continue;
      const int gq = item / n, t = item - gq * n;
#pragma unroll
      for (int j = 0; j < 8; ++j) stage[t * HS_HEADS + 8 * gq + j] = __float2half_rn(ob[q][j]);
    }
  }
  __syncthreads();
  for (int t = tid; t < n; t += VTHREADS) {
    if (!HQKV_INDEX_OK(pos_s[t], P.L)) continue;
    float over_heads = 0.f;
    for (int h = 0; h < nhq; ++h) over_heads = __fadd_rn(over_heads, __half2float(stage[t * HS_HEADS + h]));
    P.head_sum[pos_s[t]] = __float2half_rn(over_heads);
  }
}

__global__ void __launch_bounds__(VTHREADS, V_MIN_CTAS) v_pass_kernel(const __grid_constant__ DecodeParams P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  VShared& sh = *reinterpret_cast<VShared*>(smem_raw);
  const int chunk = blockIdx.y, bh = blockIdx.x;
  const int b = bh / P.H, kvh = bh - b * P.H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rep = P.rep;
  const int nh = rep > 4 ? 2 : 1;

  int ti = HQKV_NUM_TIERS;
#pragma unroll
  for (int t = 0; t < HQKV_NUM_TIERS; ++t)
    if (chunk >= P.tier[t].v_chunk0 && chunk < P.tier[t + 1].v_chunk0) ti = t;
  const TierDev& T = P.tier[ti];
  const bool is_res = ti == HQKV_NUM_TIERS;
  const int vb = is_res ? 16 : T.bits;
  const int tile_tokens = T.v_chunk_tokens / VWARPS;
  const int tile_t0 = (chunk - T.v_chunk0) * T.v_chunk_tokens + warp * tile_tokens;
  const int ntok = min(tile_tokens, T.n_v - tile_t0);  // <= 0: this warp has no tile
  VWarpShared& ws = sh.w[warp];
  const int ng = D >> P.gv_shift;

  // The next kernel of the stream - the K pass of the next decode call, if it was launched with
  // programmatic stream serialisation - may start its cache-only prologue while this grid drains.
  asm volatile("griddepcontrol.launch_dependents;");
  // ---- requests that read only the cache go out before the K pass is known to be complete
  if (ntok > 0) {
    if (vb == 8) v_tile_request<8>(T, ws, bh, tile_t0, ntok, ng);
    else if (vb == 4) v_tile_request<4>(T, ws, bh, tile_t0, ntok, ng);
    else if (vb == 2) v_tile_request<2>(T, ws, bh, tile_t0, ntok, ng);
    else if (vb == 1) v_tile_request<1>(T, ws, bh, tile_t0, ntok, ng);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (P.probs_in) {  // weights are given: nothing to fold, nothing to normalise by
    if (tid < rep) {
      sh.gm[tid] = 0.f;
      sh.gl[tid] = 1.f;
    }
    __syncthreads();
  } else
  // ---- global (max, sum) of the heads from the k_pass pairs: thread = (head, slice of the chunks);
  //      only the heads that exist are read, up to four pairs per thread in flight (one round of loads
  //      up to 4 * 128 / rep chunks), then slices are folded by shuffles and across warps
  {
    const int rs = P.rep_shift;
    const int h = tid & (rep - 1), slice = tid >> rs, slices = VTHREADS >> rs;
    const float2* part = P.k_part + static_cast<int64_t>(bh) * P.nk_chunks * MAX_REP;
    float m = -INFINITY, l = 0.f;
    for (int c0 = slice; c0 < P.nk_chunks; c0 += 4 * slices) {
      float2 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + slices * j;
        v[j] = c < P.nk_chunks ? __ldcg(part + c * MAX_REP + h) : make_float2(-INFINITY, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) softmax_merge(m, l, v[j].x, v[j].y);
    }
    for (int off = rep; off < 32; off <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
      const float l2 = __shfl_xor_sync(0xffffffffu, l, off);
      softmax_merge(m, l, m2, l2);
    }
    if (lane < rep) {
      sh.wm[warp][lane] = m;
      sh.wl[warp][lane] = l;
    }
    __syncthreads();
    if (tid < rep) {
      float mm = sh.wm[0][tid], ll = sh.wl[0][tid];
      for (int w = 1; w < VWARPS; ++w) softmax_merge(mm, ll, sh.wm[w][tid], sh.wl[w][tid]);
      sh.gm[tid] = mm;
      sh.gl[tid] = ll;
    }
    __syncthreads();
  }
  // ---- the warp's tile: probabilities of its tokens, then sum_t p_t * V_t
  if (ntok > 0 && vb != 16) {
    if (vb == 8) v_tile<8>(P, T, sh, ws, b, kvh, ntok, nh);
    else if (vb == 4) v_tile<4>(P, T, sh, ws, b, kvh, ntok, nh);
    else if (vb == 2) v_tile<2>(P, T, sh, ws, b, kvh, ntok, nh);
    else v_tile<1>(P, T, sh, ws, b, kvh, ntok, nh);
  } else {
    if (ntok > 0) {
      v_plain_tile(P, T, sh, ws, bh, b, kvh, tile_t0, ntok, is_res);
    } else {
      for (int i = lane; i < 4 * D; i += 32) {
        (&ws.u.red[0][0])[i] = 0.f;
        if (nh == 2) (&ws.v.red0[0][0])[i] = 0.f;
      }
    }
    (&ws.zt[0][0])[lane] = 0.f;  // 4 x MAX_REP floats
  }
  __syncthreads();
  // ---- partial output of this chunk (warps added in index order) joins the accumulators of this
  //      (batch, kv head).  The adds are fire-and-forget fp64 reductions: the sum of the fp32 partials
  //      depends on their order only below 2^-53, far below the fp16 rounding of the output, and no
  //      CTA has to read other CTAs' partials back (a chain of dependent L2 round trips that used to
  //      be a quarter of the kernel at batch 1).
  {
    double* accum = P.v_acc + static_cast<int64_t>(bh) * rep * D;
    for (int i = tid; i < rep * D; i += VTHREADS) {
      const int h = i >> 7, ch = i & (D - 1);
      const bool first_of_two = (h >> 2) + 1 < nh;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < VWARPS; ++w) {
        const VWarpShared& o = sh.w[w];
        v += (first_of_two ? o.v.red0[h & 3][ch] : o.u.red[h & 3][ch]) + o.zt[ch >> P.gv_shift][h];
      }
      atomicAdd(accum + i, static_cast<double>(v));
    }
  }
  // ---- the last CTA of this (batch, kv head) normalises and writes the output
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(&P.counters[bh], 1u);
    sh.is_last = (prev == static_cast<unsigned>(P.nv_chunks) - 1u) ? 1u : 0u;
    if (sh.is_last) P.counters[bh] = 0u;  // ready for the next call
  }
  __syncthreads();
  if (sh.is_last) {
    __threadfence();
    double* accum = P.v_acc + static_cast<int64_t>(bh) * rep * D;
    for (int i = tid * 2; i < rep * D; i += VTHREADS * 2) {
      const double2 v = __ldcg(reinterpret_cast<const double2*>(accum + i));
      const float inv = 1.f / sh.gl[i >> 7];
      const __half2 o = __floats2half2_rn(static_cast<float>(v.x) * inv, static_cast<float>(v.y) * inv);
      const int64_t at = (static_cast<int64_t>(b) * P.nh_q + kvh * rep) * D + i;
      *reinterpret_cast<__half2*>(P.out + at) = o;
      // kv-head sharding: the same rows go straight into every peer's copy of the gathered output
      // (plain stores over NVLink; the callers' cross-GPU barrier makes them visible before use)
      if (P.peer_flagged) {
        // value and call number travel in ONE 8-byte store: the receiver needs no fence and no signal
        const uint2 e = make_uint2(h2_as_u32(o), P.peer_state[0] + 1u);
        for (int p = 0; p < P.n_peers; ++p) reinterpret_cast<uint2*>(P.peer_out[p])[at >> 1] = e;
      } else {
        for (int p = 0; p < P.n_peers; ++p) *reinterpret_cast<__half2*>(P.peer_out[p] + at) = o;
      }
    }
    if (P.world > 1) {
      // the CTA that finishes the last (batch, kv head) of this GPU runs the cross-GPU barrier: when this
      // kernel completes, every rank's rows are in this GPU's gathered buffer
      __threadfence_system();
      __syncthreads();
      if (tid == 0) {
        const unsigned done = atomicAdd(P.peer_state + 2, 1u);
        sh.is_last = (done == static_cast<unsigned>(P.B * P.H) - 1u) ? 1u : 0u;
        if (sh.is_last) P.peer_state[2] = 0u;
      }
      __syncthreads();
      if (sh.is_last) {
        __threadfence();
        // every CTA fenced its peer stores system-wide before it counted itself in, and this CTA saw the
        // full count: the signal may go out at once
        peer_barrier_device<false>(P.pad, P.rank, P.world, P.peer_state, reinterpret_cast<int*>(P.peer_state + 1),
                                   P.max_spins, &sh.pad_[0]);
      }
    }
  }
  // ---- importance row: sum of the probabilities over batch, then over heads, for the tokens of this chunk.
  //      The CTAs of all (batch, kv head) pairs that hold this chunk index wrote these tokens' probabilities; the
  //      last of them to arrive adds them in fixed order with the roundings of attn_weights.sum(0).sum(0) on fp16
  //      tensors (fp32 accumulation, one fp16 rounding per sum; model/public_func.py:253-254 of the reference).
  if (P.head_sum) {
    __threadfence();  // this CTA's probabilities
    __syncthreads();
    if (tid == 0) {
      const unsigned prev = atomicAdd(&P.hs_count[chunk], 1u);
      sh.is_last = (prev == static_cast<unsigned>(P.B * P.H) - 1u) ? 1u : 0u;
      if (sh.is_last) P.hs_count[chunk] = 0u;  // ready for the next call
    }
    __syncthreads();
    if (sh.is_last) head_sum_chunk(P, T, sh, chunk, is_res);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static int ilog2(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

struct Layout {
  size_t acc_off, logits_off, kpart_off, total;
};

// sides: 1 = only the K side of the descriptor is looked at, 2 = only the V side, 3 = both
static int build_params(const hqkv_cache_desc_t* c, DecodeParams& P, Layout& lay, int sides = 3) {
  HQKV_REQUIRE(c != nullptr, "decode: null cache descriptor");
  HQKV_REQUIRE(c->B > 0 && c->H > 0 && c->nh_q > 0, "decode: B, H and nh_q must be positive");
  HQKV_REQUIRE(c->D == D, "decode: head dim must be 128 (got %d)", c->D);
  HQKV_REQUIRE(c->nh_q % c->H == 0 && c->nh_q / c->H <= MAX_REP,
               "decode: nh_q (%d) must be a multiple of H (%d) with at most %d query heads per kv head", c->nh_q,
               c->H, MAX_REP);
  HQKV_REQUIRE(valid_group(c->group_k) && valid_group(c->group_v), "decode: group sizes must be 32, 64 or 128");
  HQKV_REQUIRE(static_cast<int64_t>(c->B) * c->H <= 1024, "decode: B*H must not exceed 1024");
  HQKV_REQUIRE(c->n_new >= 0, "decode: negative residual length");
  memset(&P, 0, sizeof(P));
  P.B = c->B;
  P.H = c->H;
  P.nh_q = c->nh_q;
  P.rep = c->nh_q / c->H;
  HQKV_REQUIRE((P.rep & (P.rep - 1)) == 0, "decode: nh_q / H must be 1, 2, 4 or 8 (got %d)", P.rep);
  P.rep_shift = ilog2(P.rep);
  P.gk_shift = ilog2(c->group_k);
  P.gv_shift = ilog2(c->group_v);
  P.scale = c->softmax_scale;
  static const int expect_bits[HQKV_NUM_TIERS] = {16, 8, 4, 2, 1};
  int64_t nk_total = 0, nv_total = 0;
  int kc = 0, vc = 0;
  for (int t = 0; t < HQKV_NUM_TIERS; ++t) {
    const hqkv_tier_t& s = c->tier[t];
    TierDev& d = P.tier[t];
    HQKV_REQUIRE(s.n_k >= 0 && s.n_v >= 0, "decode: negative tier size");
    d.bits = expect_bits[t];
    d.n_k = (sides & 1) ? s.n_k : 0;
    d.n_v = (sides & 2) ? s.n_v : 0;
    if (d.n_k > 0 || d.n_v > 0) {
      HQKV_REQUIRE(s.bits == expect_bits[t], "decode: tier %d must hold %d-bit data (got %d)", t, expect_bits[t], s.bits);
      HQKV_REQUIRE(s.codec == HQKV_CODEC_UNIFORM || (s.codec == HQKV_CODEC_NORMAL && s.bits == 1),
                   "decode: tier %d: codec %d is not valid at %d bits (the Gaussian codebook is built for the 1-bit tier)", t,
                   s.codec, s.bits);
      d.normal = s.codec == HQKV_CODEC_NORMAL ? 1 : 0;
    }
    if (d.n_k > 0) {
      HQKV_REQUIRE(s.k_data && s.k_idx && aligned(s.k_idx, 8), "decode: tier %d K pointers are null or the index list is misaligned", t);
      if (s.bits < 16) {
        HQKV_REQUIRE(s.k_scale && s.k_zero && aligned(s.k_scale, 16) && aligned(s.k_zero, 16),
                     "decode: tier %d K scale/zero pointers are null or not 16-byte aligned", t);
        HQKV_REQUIRE(s.n_k % c->group_k == 0, "decode: tier %d K holds %d tokens, not a multiple of the K group %d", t,
                     s.n_k, c->group_k);
        HQKV_REQUIRE(aligned(s.k_data, 16), "decode: tier %d K codes must be 16-byte aligned", t);
      } else {
        HQKV_REQUIRE(s.n_k % 8 == 0 && aligned(s.k_data, 16),
                     "decode: the fp16 K tier needs a token count that is a multiple of 8 and 16-byte alignment");
      }
    }
    if (d.n_v > 0) {
      HQKV_REQUIRE(s.v_data && s.v_idx && aligned(s.v_idx, 8), "decode: tier %d V pointers are null or the index list is misaligned", t);
      if (s.bits < 16)
        HQKV_REQUIRE(s.v_scale && s.v_zero && aligned(s.v_scale, 8) && aligned(s.v_zero, 8),
                     "decode: tier %d V scale/zero pointers are null or not 8-byte aligned", t);
      HQKV_REQUIRE(aligned(s.v_data, 16), "decode: tier %d V data must be 16-byte aligned", t);
    }
    d.k_data = s.k_data;
    d.k_scale = static_cast<const __half*>(s.k_scale);
    d.k_zero = static_cast<const __half*>(s.k_zero);
    d.k_idx = s.k_idx;
    d.v_data = s.v_data;
    d.v_scale = static_cast<const __half*>(s.v_scale);
    d.v_zero = static_cast<const __half*>(s.v_zero);
    d.v_idx = s.v_idx;
    // chunk sizes: about the same number of bytes per CTA whatever the width
    const int b = d.bits;
    d.k_chunk_tokens = KWARPS * (b == 8 || b == 16 ? 64 : 128);  // one tile per warp
    HQKV_REQUIRE(static_cast<int64_t>(s.n_k) * D * b / 8 < (1ll << 31), "decode: tier %d K plane of one head exceeds 2 GiB", t);
    d.v_chunk_tokens = VWARPS * (b == 8 ? 64 : b == 16 ? 16 : 128);  // one tile per warp
    d.k_chunk0 = kc;
    d.v_chunk0 = vc;
    kc += static_cast<int>(ceil_div(d.n_k, d.k_chunk_tokens));
    vc += static_cast<int>(ceil_div(d.n_v, d.v_chunk_tokens));
    nk_total += d.n_k;
    nv_total += d.n_v;
  }
  if (sides == 3)
    HQKV_REQUIRE(nk_total == nv_total, "decode: K side holds %lld quantised tokens, V side %lld", (long long)nk_total,
                 (long long)nv_total);
  TierDev& r = P.tier[HQKV_NUM_TIERS];
  r.bits = 16;
  r.n_k = r.n_v = c->n_new;
  if (c->n_new > 0) {
    if (sides & 1) HQKV_REQUIRE(c->new_k && aligned(c->new_k, 16), "decode: residual K is null or not 16-byte aligned");
    if (sides & 2) HQKV_REQUIRE(c->new_v && aligned(c->new_v, 16), "decode: residual V is null or not 16-byte aligned");
  }
  r.k_data = c->new_k;
  r.v_data = c->new_v;
  r.k_chunk_tokens = KWARPS * 16;
  r.v_chunk_tokens = VWARPS * 16;
  r.k_chunk0 = kc;
  r.v_chunk0 = vc;
  kc += static_cast<int>(ceil_div(r.n_k, r.k_chunk_tokens));
  vc += static_cast<int>(ceil_div(r.n_v, r.v_chunk_tokens));
  const int64_t L = ((sides & 1) ? nk_total : nv_total) + c->n_new;
  HQKV_REQUIRE(L > 0, "decode: the cache is empty");
  HQKV_REQUIRE(L < (1ll << 30), "decode: cache too long");
  P.L = static_cast<int>(L);
  P.nk_chunks = kc;
  P.nv_chunks = vc;
  const int64_t BH = static_cast<int64_t>(c->B) * c->H;
  lay.acc_off = HQKV_WS_HEADER_BYTES;
  lay.logits_off = (lay.acc_off + static_cast<size_t>(BH) * P.rep * D * sizeof(double) + 255) & ~static_cast<size_t>(255);
  size_t off = lay.logits_off + static_cast<size_t>(c->B) * c->nh_q * L * sizeof(float);
  off = (off + 255) & ~static_cast<size_t>(255);
  lay.kpart_off = off;
  off += static_cast<size_t>(BH) * kc * MAX_REP * sizeof(float2);
  lay.total = (off + 255) & ~static_cast<size_t>(255);
  return HQKV_OK;
}

}  // namespace hqkv

using namespace hqkv;

extern "C" size_t hqkv_decode_workspace_bytes(const hqkv_cache_desc_t* cache_host) {
  DecodeParams P;
  Layout lay;
  if (build_params(cache_host, P, lay) != HQKV_OK) return 0;
  return lay.total;
}

extern "C" size_t hqkv_decode_workspace_zero_bytes(const hqkv_cache_desc_t* cache_host) {
  DecodeParams P;
  Layout lay;
  if (build_params(cache_host, P, lay) != HQKV_OK) return 0;
  return HQKV_WS_HEADER_BYTES;
}

namespace hqkv {
struct PeerArgs {
  void* const* out = nullptr;   // where this rank's block starts in each peer's gathered buffer
  int n_peers = 0;
  bool flagged = false;         // peers take flagged 8-byte entries
  void* const* pads = nullptr;  // signal pads of all ranks (own one included); null: no barrier
  int rank = 0, world = 0;
  void* state = nullptr;
  long long max_spins = 0;
};
static int decode_launch(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights, void* attn_output,
                         void* workspace, size_t workspace_bytes, int phases, const PeerArgs& peers, void* stream,
                         const void* probs_in = nullptr, const void* mask = nullptr, long long mask_bstride = 0,
                         long long mask_hstride = 0, void* head_sum = nullptr);
// the V pass emits the importance row itself up to these sizes (a CTA reads B*nh_q probabilities per token)
constexpr int HEAD_SUM_MAX_ROWS = 64;
constexpr int HEAD_SUM_MAX_CHUNKS = (HQKV_WS_HEADER_BYTES - 4096) / 4;
}

extern "C" int hqkv_decode_attention_phases(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                            void* attn_output, void* workspace, size_t workspace_bytes, int phases,
                                            void* stream) {
  return decode_launch(cache_host, q, attn_weights, attn_output, workspace, workspace_bytes, phases, hqkv::PeerArgs(), stream);
}

extern "C" int hqkv_decode_attention_gather(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                            void* attn_output, void* workspace, size_t workspace_bytes,
                                            void* const* peer_outputs_host, int n_peers, void* const* peer_pads_host,
                                            int rank, int world, void* state, long long max_spins, void* stream) {
  HQKV_REQUIRE(n_peers >= 0 && n_peers <= HQKV_MAX_PEERS, "decode_gather: at most %d peers (got %d)", HQKV_MAX_PEERS, n_peers);
  HQKV_REQUIRE(n_peers == 0 || peer_outputs_host, "decode_gather: null peer list");
  for (int p = 0; p < n_peers; ++p)
    HQKV_REQUIRE(peer_outputs_host[p] && aligned(peer_outputs_host[p], 4), "decode_gather: peer output %d is null or misaligned", p);
  hqkv::PeerArgs pa;
  pa.out = peer_outputs_host;
  pa.n_peers = n_peers;
  if (peer_pads_host) {
    HQKV_REQUIRE(world >= 2 && world <= HQKV_MAX_PEERS + 1 && rank >= 0 && rank < world, "decode_gather: bad rank/world");
    HQKV_REQUIRE(state && aligned(state, 4) && max_spins > 0, "decode_gather: null state or non-positive spin limit");
    for (int r = 0; r < world; ++r)
      HQKV_REQUIRE(peer_pads_host[r] && aligned(peer_pads_host[r], 4), "decode_gather: pad %d is null or misaligned", r);
    pa.pads = peer_pads_host;
    pa.rank = rank;
    pa.world = world;
    pa.state = state;
    pa.max_spins = max_spins;
  }
  return decode_launch(cache_host, q, attn_weights, attn_output, workspace, workspace_bytes, 3, pa, stream);
}

static int hqkv::decode_launch(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights, void* attn_output,
                               void* workspace, size_t workspace_bytes, int phases, const PeerArgs& peers, void* stream,
                               const void* probs_in, const void* mask, long long mask_bstride, long long mask_hstride,
                               void* head_sum) {
  HQKV_REQUIRE(phases >= 1 && phases <= 3, "decode: phases must be 1 (K pass), 2 (V pass) or 3 (both)");
  DecodeParams P;
  Layout lay;
  // a K-only call whose logits are the result, and a V-only call on given weights, look at one side only
  const int sides = probs_in ? 2 : ((phases == 1 && !attn_output) ? 1 : 3);
  int rc = build_params(cache_host, P, lay, sides);
  if (rc) return rc;
  P.n_peers = peers.n_peers;
  P.peer_flagged = peers.flagged ? 1 : 0;
  if (peers.flagged) P.peer_state = static_cast<unsigned*>(peers.state);
  for (int p = 0; p < peers.n_peers; ++p) P.peer_out[p] = static_cast<__half*>(peers.out[p]);
  if (peers.pads) {
    P.rank = peers.rank;
    P.world = peers.world;
    for (int r = 0; r < peers.world; ++r) P.pad[r] = static_cast<unsigned*>(peers.pads[r]);
    P.peer_state = static_cast<unsigned*>(peers.state);
    P.max_spins = peers.max_spins;
  }
  HQKV_REQUIRE(workspace, "decode: null pointer");
  if (phases & 1) HQKV_REQUIRE(q && aligned(q, 4), "decode: q is null or not 4-byte aligned");
  if (phases & 2) HQKV_REQUIRE(attn_output && (attn_weights || probs_in), "decode: null pointer");
  HQKV_REQUIRE(!probs_in || phases == 2, "decode: given weights go with the V pass alone");
  P.probs_in = static_cast<const __half*>(probs_in);
  HQKV_REQUIRE(!mask || (aligned(mask, 2) && mask_bstride >= 0 && mask_hstride >= 0), "decode: misaligned mask or negative stride");
  P.mask = static_cast<const __half*>(mask);
  P.mask_bstride = mask_bstride;
  P.mask_hstride = mask_hstride;
  HQKV_REQUIRE(aligned(workspace, 256), "decode: workspace must be 256-byte aligned");
  if (workspace_bytes < lay.total)
    return fail(HQKV_E_WORKSPACE, "decode: workspace holds %zu bytes, %zu needed", workspace_bytes, lay.total);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  P.q = static_cast<const __half*>(q);
  P.weights = static_cast<__half*>(attn_weights);
  P.out = static_cast<__half*>(attn_output);
  P.counters = reinterpret_cast<unsigned*>(ws);
  P.hs_count = reinterpret_cast<unsigned*>(ws + 4096);
  P.head_sum = static_cast<__half*>(head_sum);
  P.logits = reinterpret_cast<float*>(ws + lay.logits_off);
  P.k_part = reinterpret_cast<float2*>(ws + lay.kpart_off);
  P.v_acc = reinterpret_cast<double*>(ws + lay.acc_off);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned BH = static_cast<unsigned>(P.B * P.H);
  HQKV_REQUIRE(P.nk_chunks <= 65535 && P.nv_chunks <= 65535, "decode: too many chunks");
  {
    // opt in to >48 KB of dynamic shared memory once per device
    static bool attr_set[64] = {};
    int dev = 0;
    HQKV_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
      HQKV_CUDA(cudaFuncSetAttribute(v_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(sizeof(VShared))));
      HQKV_CUDA(cudaFuncSetAttribute(k_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(sizeof(KShared))));
      if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
  }
  // Both launches use programmatic stream serialisation: a grid may place its CTAs while the kernel before it
  // drains (if that kernel allows it - both of these do), and everything it does before its
  // griddepcontrol.wait reads only the cache tiers.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if ((phases & 1) && P.nk_chunks > 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(BH, P.nk_chunks);
    cfg.blockDim = dim3(KTHREADS);
    cfg.dynamicSmemBytes = sizeof(KShared);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HQKV_CUDA(cudaLaunchKernelEx(&cfg, k_pass_kernel, P));
  }
  if ((phases & 2) && P.nv_chunks > 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(BH, P.nv_chunks);
    cfg.blockDim = dim3(VTHREADS);
    cfg.dynamicSmemBytes = sizeof(VShared);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HQKV_CUDA(cudaLaunchKernelEx(&cfg, v_pass_kernel, P));
  }
  return HQKV_OK;
}

extern "C" int hqkv_decode_attention(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                     void* attn_output, void* workspace, size_t workspace_bytes, void* stream) {
  return hqkv_decode_attention_phases(cache_host, q, attn_weights, attn_output, workspace, workspace_bytes, 3, stream);
}

extern "C" int hqkv_decode_attention_masked(const hqkv_cache_desc_t* cache_host, const void* q, const void* mask,
                                            int64_t mask_b_stride, int64_t mask_h_stride, void* attn_weights,
                                            void* attn_output, void* workspace, size_t workspace_bytes, void* stream) {
  HQKV_REQUIRE(mask != nullptr, "decode_masked: null mask");
  return decode_launch(cache_host, q, attn_weights, attn_output, workspace, workspace_bytes, 3, hqkv::PeerArgs(), stream,
                       nullptr, mask, mask_b_stride, mask_h_stride);
}

extern "C" int hqkv_decode_attention_headsum(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                             void* attn_output, void* head_sum_row, void* workspace,
                                             size_t workspace_bytes, void* stream) {
  HQKV_REQUIRE(head_sum_row && aligned(head_sum_row, 2), "decode_headsum: null or misaligned row");
  DecodeParams P;
  Layout lay;
  int rc = build_params(cache_host, P, lay);
  if (rc) return rc;
  const bool fused = P.B * P.nh_q <= HEAD_SUM_MAX_ROWS && P.nh_q <= HS_HEADS && P.nv_chunks <= HEAD_SUM_MAX_CHUNKS;
  rc = decode_launch(cache_host, q, attn_weights, attn_output, workspace, workspace_bytes, 3, hqkv::PeerArgs(), stream,
                     nullptr, nullptr, 0, 0, fused ? head_sum_row : nullptr);
  if (rc || fused) return rc;
  // larger batches: one more launch over the probabilities just written
  return hqkv_head_sum(attn_weights, P.B, P.nh_q, P.L, P.L, head_sum_row, stream);
}

// ------------------------------------------------------------------------------------------------
// The two passes as operators of their own: raw logits of every tier, and the product of given weights with V
// ------------------------------------------------------------------------------------------------
namespace hqkv {
// fp32 logits of the scratch -> fp16 rows
__global__ void __launch_bounds__(256) logits_out_kernel(const float* logits, __half* out, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = __float2half_rn(__ldcg(logits + i));
}
}  // namespace hqkv

extern "C" int hqkv_decode_logits(const hqkv_cache_desc_t* cache_host, const void* q, void* logits_f16, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  HQKV_REQUIRE(logits_f16 && aligned(logits_f16, 2), "decode_logits: null or misaligned output");
  int rc = decode_launch(cache_host, q, nullptr, nullptr, workspace, workspace_bytes, 1, hqkv::PeerArgs(), stream);
  if (rc) return rc;
  DecodeParams P;
  Layout lay;
  rc = build_params(cache_host, P, lay, 1);
  if (rc) return rc;
  const int64_t n = static_cast<int64_t>(P.B) * P.nh_q * P.L;
  const int blocks = static_cast<int>(n / 2048 > 592 ? 592 : (n / 2048 > 0 ? n / 2048 : 1));
  hqkv::logits_out_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float*>(static_cast<unsigned char*>(workspace) + lay.logits_off),
      static_cast<__half*>(logits_f16), n);
  HQKV_LAUNCH_CHECK("decode_logits");
  return HQKV_OK;
}

extern "C" int hqkv_decode_weighted_sum(const hqkv_cache_desc_t* cache_host, const void* weights_f16, void* out,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  HQKV_REQUIRE(weights_f16 && aligned(weights_f16, 2), "decode_weighted_sum: null or misaligned weights");
  {
    // no K pass runs in this call, so nobody clears the output accumulators: a stream-ordered memset does
    DecodeParams P;
    Layout lay;
    int rc = build_params(cache_host, P, lay, 2);
    if (rc) return rc;
    HQKV_REQUIRE(workspace && workspace_bytes >= lay.total, "decode_weighted_sum: workspace too small");
    HQKV_CUDA(cudaMemsetAsync(static_cast<unsigned char*>(workspace) + lay.acc_off, 0, lay.logits_off - lay.acc_off,
                              static_cast<cudaStream_t>(stream)));
  }
  return decode_launch(cache_host, nullptr, nullptr, out, workspace, workspace_bytes, 2, hqkv::PeerArgs(), stream, weights_f16);
}

namespace hqkv {
unsigned decode_check_failures(bool reset) {
#if HQKV_CHECKS_ENABLED
  unsigned v = 0, z = 0;
  if (cudaMemcpyFromSymbol(&v, g_check_failures, sizeof(v)) != cudaSuccess) return ~0u;
  if (reset) cudaMemcpyToSymbol(g_check_failures, &z, sizeof(z));
  return v;
#else
  (void)reset;
  return 0u;
#endif
}
}  // namespace hqkv

extern "C" int hqkv_checks_enabled(void) { return HQKV_CHECKS_ENABLED; }

extern "C" int hqkv_check_failures(int reset, unsigned* count_host) {
  HQKV_REQUIRE(count_host != nullptr, "check_failures: null pointer");
  HQKV_CUDA(cudaDeviceSynchronize());
  *count_host = hqkv::decode_check_failures(reset != 0) + hqkv::policy_check_failures(reset != 0);
  return HQKV_OK;
}

// ------------------------------------------------------------------------------------------------
// Decode attention for callers that may not allocate device memory
// ------------------------------------------------------------------------------------------------
// Some hosts of this library cannot obtain scratch at call time: a serving loop that has handed all
// of the GPU's memory to its own pool, a latency-critical loop whose rules forbid allocation after
// start-up (cudaMalloc may synchronise the device, and may fail late), or a binding whose language
// runtime owns no device allocator.  For them the scratch of the two decode kernels lives in this
// fixed array, which every GPU that loads the library holds until the process exits.
//
// g_static_scratch names the array in DEVICE code.  In host code the same identifier is only a
// stand-in for the symbol, not a device address, so the host asks the runtime for the address once
// per device (cudaGetSymbolAddress with that device current) and passes the pointer it gets.
static __device__ __align__(256) unsigned char g_static_scratch[HQKV_STATIC_SCRATCH_BYTES];

namespace hqkv {
static void* g_static_scratch_ptr[64] = {};  // device address of the array, per device ordinal

static int static_scratch_address(void** out) {
  int dev = 0;
  HQKV_CUDA(cudaGetDevice(&dev));
  HQKV_REQUIRE(dev >= 0 && dev < 64, "decode_static: device ordinal %d out of range", dev);
  void* p = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    HQKV_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    HQKV_REQUIRE(p != nullptr, "decode_static: the scratch symbol has no address on device %d", dev);
    __atomic_store_n(&g_static_scratch_ptr[dev], p, __ATOMIC_RELEASE);  // every thread would store the same address
  }
  *out = p;
  return HQKV_OK;
}
}  // namespace hqkv

extern "C" size_t hqkv_decode_static_scratch_bytes(void) { return HQKV_STATIC_SCRATCH_BYTES; }

extern "C" int hqkv_decode_attention_static(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                            void* attn_output, void* stream) {
  const size_t need = hqkv_decode_workspace_bytes(cache_host);
  if (need == 0)  // invalid descriptor: let the regular path produce the precise message
    return hqkv_decode_attention(cache_host, q, attn_weights, attn_output, nullptr, 0, stream);
  if (need > HQKV_STATIC_SCRATCH_BYTES)
    return fail(HQKV_E_WORKSPACE,
                "decode_static: this cache needs %zu bytes of scratch, the built-in array holds %zu "
                "(HQKV_STATIC_SCRATCH_BYTES); use hqkv_decode_attention with caller-provided scratch",
                need, static_cast<size_t>(HQKV_STATIC_SCRATCH_BYTES));
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  // The array keeps whatever the previous call left.  Only the arrival counters have to start at
  // zero; a finished call leaves them zero, an aborted one might not, so they are cleared every time
  // (a stream-ordered memset, not an allocation).
  HQKV_CUDA(cudaMemsetAsync(scratch, 0, HQKV_WS_HEADER_BYTES, static_cast<cudaStream_t>(stream)));
  return hqkv_decode_attention(cache_host, q, attn_weights, attn_output, scratch, HQKV_STATIC_SCRATCH_BYTES, stream);
}

// ------------------------------------------------------------------------------------------------
// Cross-GPU barrier for the kv-head-sharded decode (one process per GPU)
// ------------------------------------------------------------------------------------------------
// After hqkv_decode_attention_gather every rank has written its heads' output rows into every peer's
// gathered buffer.  This kernel, launched by every rank on the same stream right after, (1) tells every
// peer "my stores of call number n are done" by raising a counter in the peer's signal pad, and (2)
// waits until every peer has told it the same.  The call number lives in device memory and is advanced
// by the kernel itself, so the launch can sit in a CUDA graph that is replayed.  Every wait is bounded:
// after max_spins polls the kernel gives up, records which peer was missing in *status and returns, so
// a rank that died cannot hang the others' GPUs (the data of that step is then incomplete and the host
// must check *status before it trusts it).
namespace hqkv {
struct PeerPads {
  unsigned* pad[HQKV_MAX_PEERS + 1];  // the ranks' signal pads, own one included
};

__global__ void peer_barrier_kernel(const __grid_constant__ PeerPads pads, int rank, int world, unsigned* call_no,
                                    int* status, long long max_spins) {
  __shared__ unsigned n;
  peer_barrier_device<true>(pads.pad, rank, world, call_no, status, max_spins, &n);
}
}  // namespace hqkv

extern "C" int hqkv_peer_barrier(void* const* peer_pads_host, int rank, int world, void* state, long long max_spins,
                                 void* stream) {
  HQKV_REQUIRE(world >= 1 && world <= HQKV_MAX_PEERS + 1 && rank >= 0 && rank < world, "peer_barrier: bad rank/world");
  HQKV_REQUIRE(peer_pads_host && state && aligned(state, 8) && max_spins > 0,
               "peer_barrier: null or misaligned pointer, or non-positive spin limit");
  hqkv::PeerPads pads = {};
  for (int r = 0; r < world; ++r) {
    HQKV_REQUIRE(peer_pads_host[r] && aligned(peer_pads_host[r], 4), "peer_barrier: pad %d is null or misaligned", r);
    pads.pad[r] = static_cast<unsigned*>(peer_pads_host[r]);
  }
  // state (8 bytes of this GPU's memory, zero before the first call): call number, status
  unsigned* st = static_cast<unsigned*>(state);
  hqkv::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pads, rank, world, st,
                                                                             reinterpret_cast<int*>(st + 1), max_spins);
  HQKV_LAUNCH_CHECK("peer_barrier");
  return HQKV_OK;
}

// ------------------------------------------------------------------------------------------------
// Flagged exchange: the low-latency form of the kv-head-sharded gather
// ------------------------------------------------------------------------------------------------
// hqkv_decode_attention_gather_flagged makes the V pass store every pair of output values together with
// the call number as ONE 8-byte word into the peers' receive buffers: a word whose flag equals the
// call number is complete, so no fence, no signal and no round trip is needed - the exchange costs
// one NVLink store latency.  hqkv_peer_unpack, enqueued by every rank right after, polls its own
// receive buffer (bounded), strips the flags into the plain gathered buffer [world][entries] of fp16
// pairs and advances the call number (device memory: the pair of launches replays from a CUDA graph).
// A receive buffer must not be reused before the peers have unpacked it: callers rotate at least two.
namespace hqkv {
__global__ void __launch_bounds__(256) peer_unpack_kernel(const uint2* recv, uint32_t* plain, int rank, int world,
                                                          int entries, unsigned* state, long long max_spins) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // this GPU's own decode call has finished
  const unsigned n = state[0] + 1u;
  // Four words per thread are requested together, so that a pass over words that have already arrived costs one
  // round trip, not one per word; a word that is still old is polled on its own.
  const int total = world * entries;
  for (int base = threadIdx.x; base < total; base += 4 * 256) {
    uint2 e[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = base + j * 256;
      e[j] = make_uint2(0u, n);
      if (i < total && i / entries != rank)  // own rows were written in place by the decode kernel
        asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(e[j].x), "=r"(e[j].y) : "l"(recv + i));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = base + j * 256;
      if (i >= total || i / entries == rank) continue;
      long long spins = 0;
      while (e[j].y != n) {
        if (++spins > max_spins) {
          atomicExch(reinterpret_cast<int*>(state + 1), i / entries + 1);  // gave up waiting for that rank
          break;
        }
        __nanosleep(20);
        asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(e[j].x), "=r"(e[j].y) : "l"(recv + i));
      }
      plain[i] = e[j].x;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) state[0] = n;
}
}  // namespace hqkv

extern "C" int hqkv_decode_attention_gather_flagged(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                                    void* attn_output, void* workspace, size_t workspace_bytes,
                                                    void* const* peer_recv_host, int n_peers, void* state, void* stream) {
  HQKV_REQUIRE(n_peers >= 1 && n_peers <= HQKV_MAX_PEERS, "decode_gather_flagged: 1..%d peers (got %d)", HQKV_MAX_PEERS, n_peers);
  HQKV_REQUIRE(peer_recv_host && state && aligned(state, 4), "decode_gather_flagged: null pointer");
  for (int p = 0; p < n_peers; ++p)
    HQKV_REQUIRE(peer_recv_host[p] && aligned(peer_recv_host[p], 8), "decode_gather_flagged: peer buffer %d is null or misaligned", p);
  hqkv::PeerArgs pa;
  pa.out = peer_recv_host;
  pa.n_peers = n_peers;
  pa.flagged = true;
  pa.state = state;
  return decode_launch(cache_host, q, attn_weights, attn_output, workspace, workspace_bytes, 3, pa, stream);
}

extern "C" int hqkv_peer_unpack(const void* recv, void* gathered, int rank, int world, int entries_per_rank, void* state,
                                long long max_spins, void* stream) {
  HQKV_REQUIRE(world >= 2 && world <= HQKV_MAX_PEERS + 1 && rank >= 0 && rank < world, "peer_unpack: bad rank/world");
  HQKV_REQUIRE(recv && gathered && state && aligned(recv, 8) && aligned(gathered, 4) && aligned(state, 4),
               "peer_unpack: null or misaligned pointer");
  HQKV_REQUIRE(entries_per_rank > 0 && max_spins > 0, "peer_unpack: sizes and the spin limit must be positive");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(256);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // polls may start while the decode call drains
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  HQKV_CUDA(cudaLaunchKernelEx(&cfg, hqkv::peer_unpack_kernel, static_cast<const uint2*>(recv),
                               static_cast<uint32_t*>(gathered), rank, world, entries_per_rank,
                               static_cast<unsigned*>(state), max_spins));
  return HQKV_OK;
}
