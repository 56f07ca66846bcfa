// Importance bookkeeping, block ranking and the flush (evict + tier-assign + re-quantise) on the
// device (sm_100a).  Integer / fp16 elementwise work on at most a few hundred thousand tokens; the
// quantity that matters is bit-exact agreement with the reference's torch op sequence, so every
// floating-point reduction here runs in a fixed order with one fp32 accumulator.
#include <string.h>

#include <cooperative_groups.h>

#include "common.cuh"

namespace hqkv {

HQKV_DEFINE_CHECK_COUNTER
unsigned policy_check_failures(bool reset) {
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

constexpr int D = 128;

// ------------------------------------------------------------------------------------------------
// importance ring
// ------------------------------------------------------------------------------------------------
// 32 positions per CTA, four warps.  The adds run in the reference's order (batch first with one fp32
// accumulator per head, rounded to fp16; then the heads, one fp32 accumulator), but a position's B * nh
// values lie a whole row apart, so a single chain of loads is all latency: warp w sums the batch for heads
// 8w .. 8w+7 of a pass of 32 heads (eight loads in flight per thread, every load a coalesced 64-byte row
// piece), the per-head results meet in shared memory, and warp 0 adds them in head order.
constexpr int HEAD_SUM_THREADS = 128;
__global__ void __launch_bounds__(HEAD_SUM_THREADS) head_sum_kernel(const __half* __restrict__ w, int B, int nh, int64_t L,
                                                                    int64_t bh_stride, __half* __restrict__ out) {
  __shared__ float per_head[32][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t l = static_cast<int64_t>(blockIdx.x) * 32 + lane;
  const bool live = l < L;
  float over_heads = 0.f;
  for (int h0 = 0; h0 < nh; h0 += 32) {
    const int hw = h0 + 8 * warp;
    float over_batch[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) over_batch[j] = 0.f;
#pragma unroll 2
    for (int b = 0; b < B; ++b) {
      __half v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        v[j] = live && hw + j < nh ? w[(static_cast<int64_t>(b) * nh + hw + j) * bh_stride + l] : __float2half_rn(0.f);
#pragma unroll
      for (int j = 0; j < 8; ++j) over_batch[j] = __fadd_rn(over_batch[j], __half2float(v[j]));
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) per_head[8 * warp + j][lane] = __half2float(__float2half_rn(over_batch[j]));
    __syncthreads();
    if (warp == 0) {
      const int n = nh - h0 < 32 ? nh - h0 : 32;
      for (int h = 0; h < n; ++h) over_heads = __fadd_rn(over_heads, per_head[h][lane]);
    }
    __syncthreads();
  }
  if (warp == 0 && live) out[l] = __float2half_rn(over_heads);
}

__global__ void __launch_bounds__(256) token_importance_kernel(const __half* __restrict__ ring, int rows,
                                                               int64_t stride, int64_t L, __half* __restrict__ out) {
  const int64_t l = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (l >= L) return;
  float acc = 0.f;
  for (int r0 = 0; r0 < rows; r0 += 4) {  // four loads in flight, adds in row order
    __half v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = r0 + j < rows ? ring[(r0 + j) * stride + l] : __float2half_rn(0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (r0 + j < rows) acc = __fadd_rn(acc, __half2float(v[j]));
  }
  const int64_t age = L - l;
  const float count = static_cast<float>(age < rows ? age : rows);
  out[l] = h_divf(__float2half_rn(acc), count);
}

// one warp per token: range over D channels per (b,h), summed over b then h
__global__ void __launch_bounds__(128) token_range_kernel(const __half* __restrict__ v, int B, int H, int64_t T,
                                                          int Dd, int64_t b_stride, int64_t h_stride,
                                                          __half* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  float over_heads = 0.f;
  for (int h = 0; h < H; ++h) {
    float over_batch = 0.f;
    for (int b = 0; b < B; ++b) {
      const __half* row = v + b * b_stride + h * h_stride + t * Dd;
      __half lo = row[lane], hi = row[lane];
      for (int d = lane + 32; d < Dd; d += 32) {
        lo = h_min(lo, row[d]);
        hi = h_max(hi, row[d]);
      }
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        lo = h_min(lo, __shfl_xor_sync(0xffffffffu, lo, off));
        hi = h_max(hi, __shfl_xor_sync(0xffffffffu, hi, off));
      }
      over_batch = __fadd_rn(over_batch, __half2float(h_sub(hi, lo)));
    }
    over_heads = __fadd_rn(over_heads, __half2float(__float2half_rn(over_batch)));
  }
  if (lane == 0) out[t] = __float2half_rn(over_heads);
}

// head_dim 128, 8-byte aligned rows: one 8-byte load per lane and row, eight rows in flight, half2 min / max.
// Same additions in the same order as above.
__global__ void __launch_bounds__(128) token_range128_kernel(const __half* __restrict__ v, int B, int H, int64_t T,
                                                             int64_t b_stride, int64_t h_stride,
                                                             __half* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int n = B * H;  // rows of this token, head-major: r = h * B + b
  float over_heads = 0.f, over_batch = 0.f;
  for (int r0 = 0; r0 < n; r0 += 8) {
    uint2 w[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = min(r0 + u, n - 1), h = r / B, b = r - h * B;
      w[u] = *reinterpret_cast<const uint2*>(v + b * b_stride + h * h_stride + t * 128 + 4 * lane);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (r0 + u >= n) break;
      const __half2 a = *reinterpret_cast<const __half2*>(&w[u].x), c = *reinterpret_cast<const __half2*>(&w[u].y);
      __half2 lo = __hmin2_nan(a, c), hi = __hmax2_nan(a, c);
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        lo = __hmin2_nan(lo, __shfl_xor_sync(0xffffffffu, lo, off));
        hi = __hmax2_nan(hi, __shfl_xor_sync(0xffffffffu, hi, off));
      }
      const __half l1 = __hmin_nan(__low2half(lo), __high2half(lo)), h1 = __hmax_nan(__low2half(hi), __high2half(hi));
      over_batch = __fadd_rn(over_batch, __half2float(h_sub(h1, l1)));
      if ((r0 + u) % B == B - 1) {  // last batch entry of this head
        over_heads = __fadd_rn(over_heads, __half2float(__float2half_rn(over_batch)));
        over_batch = 0.f;
      }
    }
  }
  if (lane == 0) out[t] = __float2half_rn(over_heads);
}

// ------------------------------------------------------------------------------------------------
// block ranking: one thread-block cluster; bitonic sort of (inverted key, block id) in the shared memory of its
// first CTA
// ------------------------------------------------------------------------------------------------
// The elementwise pass, the block keys and the final expansion to token ids are spread over the CTAs of the
// cluster (one launch of one CTA spent most of its time walking 32 k tokens with 1024 threads); the keys meet in
// the first CTA's shared memory (distributed shared memory stores), which sorts them alone, and all CTAs read the
// sorted keys back from there.  Cluster barriers separate the passes and order the in-place update of
// `importance` between the CTAs.
constexpr int RANK_THREADS = 1024;
constexpr int RANK_CLUSTER = 8;
constexpr int RANK_MAX_BLOCKS = 8192;

__global__ void __launch_bounds__(RANK_THREADS) block_rank_kernel(__half* __restrict__ importance,
                                                                  const __half* __restrict__ range, int block,
                                                                  int nblocks, int npow2,
                                                                  int64_t* __restrict__ sorted_ids) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ uint32_t keys[];  // npow2 entries; only the first CTA's copy is used
  uint32_t* keys0 = cluster.map_shared_rank(keys, 0);
  const int crank = static_cast<int>(cluster.block_rank());
  const int64_t gtid = static_cast<int64_t>(crank) * RANK_THREADS + threadIdx.x;
  constexpr int64_t GTHREADS = static_cast<int64_t>(RANK_THREADS) * RANK_CLUSTER;
  const int64_t total = static_cast<int64_t>(nblocks) * block;
  const float fblock = static_cast<float>(block);
  // elementwise: optional product with the range, then the in-place divide
  for (int64_t i = gtid; i < total; i += GTHREADS) {
    __half x = importance[i];
    if (range) x = h_mul(x, range[i]);
    importance[i] = h_divf(x, fblock);
  }
  cluster.sync();
  for (int64_t k = gtid; k < npow2; k += GTHREADS) {
    uint32_t composite = 0xFFFFFFFFu;
    if (k < nblocks) {
      float acc = 0.f;
      const __half* p = importance + k * block;
      for (int i = 0; i < block; ++i) acc = __fadd_rn(acc, __half2float(p[i]));
      const __half key = __float2half_rn(acc);
      uint16_t bits = __half_as_ushort(key);
      if ((bits & 0x7FFFu) == 0) bits = 0;                                  // -0 sorts like +0
      const uint16_t asc = (bits & 0x8000u) ? static_cast<uint16_t>(~bits) : static_cast<uint16_t>(bits | 0x8000u);
      const uint16_t desc = static_cast<uint16_t>(0xFFFFu - asc);           // larger key first
      composite = (static_cast<uint32_t>(desc) << 16) | static_cast<uint32_t>(k);  // ties: lower id first
    }
    keys0[k] = composite;
  }
  cluster.sync();
  if (crank == 0) {
    for (int size = 2; size <= npow2; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int i = threadIdx.x; i < (npow2 >> 1); i += RANK_THREADS) {
          const int lo = 2 * i - (i & (stride - 1));  // index with the `stride` bit clear
          const int hi = lo + stride;
          const bool up = (lo & size) == 0;
          const uint32_t a = keys[lo], b = keys[hi];
          if ((a > b) == up) {
            keys[lo] = b;
            keys[hi] = a;
          }
        }
        __syncthreads();
      }
    }
  }
  cluster.sync();
  for (int64_t i = gtid; i < total; i += GTHREADS) {
    const int j = static_cast<int>(i / block);
    const int64_t blk = keys0[j] & 0xFFFFu;
    sorted_ids[i] = blk * block + (i - static_cast<int64_t>(j) * block);
  }
  cluster.sync();  // the first CTA's shared memory stays until every CTA has read the sorted keys
}

// ------------------------------------------------------------------------------------------------
// flush plan: one thread-block cluster
// ------------------------------------------------------------------------------------------------
constexpr int PLAN_THREADS = 1024;
constexpr int PLAN_CLUSTER = 8;   // CTAs of the cluster (the portable maximum)

struct PlanArgs {
  const int64_t* tier_idx[HQKV_NUM_TIERS];
  int32_t tier_n[HQKV_NUM_TIERS];
  int64_t hist, compress;
  int64_t cum[6];
  const int64_t* sorted_ids;
  int32_t* plan_src;   // [5][total]
  int64_t* plan_ids;   // [5][total]
  int64_t* survivors;  // [total]
  int32_t* counts;     // [8]
  // scratch, each [total]
  int8_t* tgt;         // by token id
  int8_t* fin;         // by enumeration slot
  int32_t* rank;       // by token id: rank among survivors
  int32_t* gcnt;       // [PLAN_CATS][PLAN_CLUSTER * PLAN_WARPS] per-warp category counts of the whole cluster
  int32_t* flags;      // [0] = something is evicted
};

// Enumeration order of every cached token: residual (ascending id), then the 16-, 8-, 4-, 2-, 1-bit
// tier in storage order.  Slot -> (source tier, position, token id).
__device__ __forceinline__ void enum_slot(const PlanArgs& A, int64_t slot, int& src, int64_t& pos, int64_t& id) {
  if (slot < A.compress) {
    src = -1;
    pos = slot;
    id = A.hist + slot;
    return;
  }
  int64_t s = slot - A.compress;
  for (int t = 0; t < HQKV_NUM_TIERS; ++t) {
    if (s < A.tier_n[t]) {
      src = t;
      pos = s;
      id = A.tier_idx[t][s];
      return;
    }
    s -= A.tier_n[t];
  }
  src = -2;
  pos = 0;
  id = 0;
}

// One cluster of PLAN_CLUSTER CTAs of 32 warps.  Every pass walks the enumeration (or the token ids) in
// warp-contiguous ranges - warp w of CTA r is range r * 32 + w - PLAN_BATCH iterations at a time so that the
// dependent loads of a batch (index list -> target -> rank) are in flight together; ordered positions come from
// per-warp counts (left in global memory for the other CTAs), one scan over all warps of the cluster, and ballot /
// match prefixes inside a warp.  The passes are separated by cluster barriers, which also order the global-memory
// scratch between the CTAs.  Categories: 2*t = kept member of tier t, 2*t + 1 = arrival in tier t (destination
// order: kept members first, then arrivals, both in enumeration order); 10 = surviving token id.
constexpr int PLAN_WARPS = PLAN_THREADS / 32;
constexpr int PLAN_GWARPS = PLAN_WARPS * PLAN_CLUSTER;
constexpr int PLAN_BATCH = 8;
constexpr int PLAN_CATS = 2 * HQKV_NUM_TIERS + 1;

__global__ void __launch_bounds__(PLAN_THREADS) flush_plan_kernel(const __grid_constant__ PlanArgs A) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ int cnt[PLAN_CATS][PLAN_WARPS];  // this CTA's per-warp totals, then their exclusive offsets over the cluster
  __shared__ int tot[PLAN_CATS];
  const int64_t total = A.hist + A.compress;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int crank = static_cast<int>(cluster.block_rank());
  const int gwarp = crank * PLAN_WARPS + warp;
  const int64_t gtid = static_cast<int64_t>(crank) * PLAN_THREADS + tid;
  constexpr int64_t GTHREADS = static_cast<int64_t>(PLAN_THREADS) * PLAN_CLUSTER;
  const unsigned lt = (1u << lane) - 1u;
  // warp gw owns elements [gw * span, (gw + 1) * span), span a multiple of 32
  const int64_t iters = (total + GTHREADS - 1) / GTHREADS;
  const int64_t span = iters * 32, first = gwarp * span;
  if (gtid == 0) A.flags[0] = 0;
  if (tid < PLAN_CATS * PLAN_WARPS) (&cnt[0][0])[tid] = 0;
  // 1. targets by token id
  for (int64_t i = gtid; i < total; i += GTHREADS) A.tgt[i] = -1;
  cluster.sync();
  for (int64_t j = gtid; j < total; j += GTHREADS) {
    int t = -1;
#pragma unroll
    for (int k = 5; k >= 0; --k)
      if (j < A.cum[k] && j >= (k ? A.cum[k - 1] : 0)) t = k;
    if (t >= 0) {
      if (HQKV_INDEX_OK(A.sorted_ids[j], total)) A.tgt[A.sorted_ids[j]] = static_cast<int8_t>(t);
      if (t == 5) A.flags[0] = 1;
    }
  }
  cluster.sync();
  // 2. final tier of every enumeration slot (0..4 tier, 5 evicted, 6 dropped: residual without target),
  //    survival by token id, and the per-warp category counts
  for (int64_t j0 = 0; j0 < iters; j0 += PLAN_BATCH) {
    int src[PLAN_BATCH];
    int64_t id[PLAN_BATCH];
    int tg[PLAN_BATCH];
#pragma unroll
    for (int u = 0; u < PLAN_BATCH; ++u) {
      const int64_t s = first + (j0 + u) * 32 + lane;
      int64_t pos;
      src[u] = -2;
      id[u] = 0;
      if (j0 + u < iters && s < total) enum_slot(A, s, src[u], pos, id[u]);
    }
#pragma unroll
    for (int u = 0; u < PLAN_BATCH; ++u) tg[u] = (src[u] != -2 && HQKV_INDEX_OK(id[u], total)) ? A.tgt[id[u]] : -1;
#pragma unroll
    for (int u = 0; u < PLAN_BATCH; ++u) {
      if (src[u] == -2) continue;
      const int64_t s = first + (j0 + u) * 32 + lane;
      int f;
      if (tg[u] == 5) f = 5;
      else if (src[u] < 0) f = tg[u] < 0 ? 6 : tg[u];
      else f = tg[u] > src[u] ? tg[u] : src[u];  // only moves to fewer bits (larger index); tg == -1 stays
      A.fin[s] = static_cast<int8_t>(f);
      A.rank[id[u]] = (tg[u] != 5) ? 1 : 0;  // token ids are a permutation of 0..total-1 over the enumeration
      if (f < HQKV_NUM_TIERS) atomicAdd(&cnt[2 * f + (src[u] == f ? 0 : 1)][warp], 1);
    }
  }
  cluster.sync();
  // 3. survivor counts per warp range of token ids
  {
    int mine = 0;
    for (int64_t j0 = 0; j0 < iters; j0 += PLAN_BATCH) {
      int fl[PLAN_BATCH];
#pragma unroll
      for (int u = 0; u < PLAN_BATCH; ++u) {
        const int64_t i = first + (j0 + u) * 32 + lane;
        fl[u] = (j0 + u < iters && i < total) ? A.rank[i] : 0;
      }
#pragma unroll
      for (int u = 0; u < PLAN_BATCH; ++u) mine += fl[u];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) cnt[PLAN_CATS - 1][warp] = mine;
  }
  __syncthreads();
  // this CTA's per-warp totals -> global memory, for the scan over all warps of the cluster
  if (tid < PLAN_CATS * PLAN_WARPS) {
    const int c = tid / PLAN_WARPS, w = tid - c * PLAN_WARPS;
    A.gcnt[c * PLAN_GWARPS + crank * PLAN_WARPS + w] = cnt[c][w];
  }
  cluster.sync();
  // exclusive offsets of every category over the warps of the cluster (every CTA scans for its own warps)
  if (tid < PLAN_CATS) {
    int acc = 0;
    for (int w = 0; w < PLAN_GWARPS; ++w) {
      const int c = A.gcnt[tid * PLAN_GWARPS + w];
      if (w >= crank * PLAN_WARPS && w < (crank + 1) * PLAN_WARPS) cnt[tid][w - crank * PLAN_WARPS] = acc;
      acc += c;
    }
    tot[tid] = acc;
  }
  __syncthreads();
  const int any_evict = A.flags[0];
  // 4. survivor ranks by token id: rank[i] = survivors with a smaller id; survivors[rank] = id
  {
    int running = cnt[PLAN_CATS - 1][warp];
    for (int64_t j0 = 0; j0 < iters; j0 += PLAN_BATCH) {
      int fl[PLAN_BATCH];
#pragma unroll
      for (int u = 0; u < PLAN_BATCH; ++u) {
        const int64_t i = first + (j0 + u) * 32 + lane;
        fl[u] = (j0 + u < iters && i < total) ? A.rank[i] : -1;
      }
#pragma unroll
      for (int u = 0; u < PLAN_BATCH; ++u) {
        const unsigned ballot = __ballot_sync(0xffffffffu, fl[u] > 0);
        const int64_t i = first + (j0 + u) * 32 + lane;
        const int r = running + __popc(ballot & lt);
        if (fl[u] >= 0) A.rank[i] = r;
        if (fl[u] > 0) A.survivors[r] = i;
        running += __popc(ballot);
      }
    }
  }
  cluster.sync();
  // 5. destination lists
  {
    for (int64_t j0 = 0; j0 < iters; j0 += PLAN_BATCH) {
      int src[PLAN_BATCH], f[PLAN_BATCH];
      int64_t pos[PLAN_BATCH], id[PLAN_BATCH];
#pragma unroll
      for (int u = 0; u < PLAN_BATCH; ++u) {
        const int64_t s = first + (j0 + u) * 32 + lane;
        src[u] = -2;
        pos[u] = id[u] = 0;
        f[u] = 6;
        if (j0 + u < iters && s < total) {
          enum_slot(A, s, src[u], pos[u], id[u]);
          f[u] = A.fin[s];
        }
      }
      int64_t outid[PLAN_BATCH];
#pragma unroll
      for (int u = 0; u < PLAN_BATCH; ++u)
        outid[u] = (any_evict && f[u] < HQKV_NUM_TIERS) ? static_cast<int64_t>(A.rank[id[u]]) : id[u];
#pragma unroll
      for (int u = 0; u < PLAN_BATCH; ++u) {
        const bool on = f[u] < HQKV_NUM_TIERS;
        const int cat = on ? 2 * f[u] + (src[u] == f[u] ? 0 : 1) : PLAN_CATS;  // PLAN_CATS: no destination
        const unsigned same = __match_any_sync(0xffffffffu, cat);
        if (on) {
          const int base = cnt[cat][warp];  // this warp's running offset of the category (only this warp touches it)
          const int64_t j = (cat & 1 ? tot[cat - 1] : 0) + base + __popc(same & lt);
          A.plan_src[f[u] * total + j] = ((src[u] + 1) << 28) | static_cast<int32_t>(pos[u]);
          A.plan_ids[f[u] * total + j] = outid[u];
        }
        __syncwarp();
        if (on && (same & lt) == 0) cnt[cat][warp] += __popc(same);
        __syncwarp();
      }
    }
  }
  if (crank == 0) {
    if (tid < HQKV_NUM_TIERS) A.counts[tid] = tot[2 * tid] + tot[2 * tid + 1];
    if (tid == 0) {
      A.counts[5] = tot[PLAN_CATS - 1];
      A.counts[6] = any_evict;
      A.counts[7] = 0;
    }
  }
  cluster.sync();  // no CTA of the cluster exits while another may still read its shared memory - none does, but the
                   // barrier is cheap and keeps the exit orderly
}

// ------------------------------------------------------------------------------------------------
// flush build
// ------------------------------------------------------------------------------------------------
struct BuildArgs {
  const void* data[HQKV_NUM_TIERS];
  const __half* scale[HQKV_NUM_TIERS];
  const __half* zero[HQKV_NUM_TIERS];
  int32_t n[HQKV_NUM_TIERS];
  const __half* residual;
  int64_t res_b_stride, res_h_stride;
  int B, H, group, gshift, dst_tier, dst_bits;
  int normal_dst;  // the destination is the 1-bit tier in the Gaussian-codebook codec
  int per_warp;    // V side: destination tokens per warp
  const int32_t* plan;  // [n_dst]
  int64_t n_dst;
  void* out_data;
  __half* out_scale;
  __half* out_zero;
};

__device__ __forceinline__ int tier_bits(int t) { return 16 >> t; }  // 16, 8, 4, 2, 1

// K side: one CTA per (destination group of `group` tokens, batch*head); one thread per channel.
// The tokens of a destination group come from one source and are consecutive there (tiers are
// filled and emptied in whole blocks).
__device__ __forceinline__ __half k_src_value(const BuildArgs& A, int src, int64_t pos, int b, int h, int d) {
  const int64_t bh = static_cast<int64_t>(b) * A.H + h;
  if (src < 0) return A.residual[b * A.res_b_stride + h * A.res_h_stride + pos * D + d];
  const int64_t n = A.n[src];
  if (src == 0) return reinterpret_cast<const __half*>(A.data[0])[(bh * D + d) * n + pos];
  const int bits = tier_bits(src), fpi = 32 / bits;
  const uint32_t word = reinterpret_cast<const uint32_t*>(A.data[src])[(bh * D + d) * (n / fpi) + pos / fpi];
  const uint32_t code = (word >> ((pos % fpi) * bits)) & ((1u << bits) - 1u);
  const int64_t G = n >> A.gshift;
  const int64_t gi = (bh * D + d) * G + (pos >> A.gshift);
  return dequant_2r(code, A.scale[src][gi], A.zero[src][gi]);
}

constexpr int BUILD_V_TOKENS_MAX = 8;  // destination tokens per warp when the grid would be scheduling-bound

__device__ __forceinline__ void build_k_group(const BuildArgs& A, int64_t jg, int bh, int b, int h, int d) {
  const int32_t enc = A.plan[jg * A.group];
  const int src = (enc >> 28) - 1;
  const int64_t pos0 = enc & 0x0FFFFFFF;
  const int bits = A.dst_bits;
  const int64_t row = static_cast<int64_t>(bh) * D + d;
  if (bits == 16) {
    __half* dst = reinterpret_cast<__half*>(A.out_data) + row * A.n_dst + jg * A.group;
    for (int i = 0; i < A.group; ++i) dst[i] = k_src_value(A, src, pos0 + i, b, h, d);
    return;
  }
  const int fpi = 32 / bits, wpg = A.group / fpi;
  const int64_t Wd = A.n_dst / fpi, Gd = A.n_dst >> A.gshift;
  uint32_t* dst = reinterpret_cast<uint32_t*>(A.out_data) + row * Wd + jg * wpg;
  if (src == A.dst_tier) {  // kept block: copy words, scale, zero
    const int64_t n = A.n[src];
    const uint32_t* s = reinterpret_cast<const uint32_t*>(A.data[src]) + row * (n / fpi) + pos0 / fpi;
    for (int w = 0; w < wpg; ++w) dst[w] = s[w];
    const int64_t gi = row * (n >> A.gshift) + (pos0 >> A.gshift);
    A.out_scale[row * Gd + jg] = A.scale[src][gi];
    A.out_zero[row * Gd + jg] = A.zero[src][gi];
    return;
  }
  if (A.normal_dst) {  // group statistics in fp64, then one code per token
    double sum = 0.0;
    for (int i = 0; i < A.group; ++i) sum += static_cast<double>(__half2float(k_src_value(A, src, pos0 + i, b, h, d)));
    const double mean64 = sum / A.group;
    double ss = 0.0;
    for (int i = 0; i < A.group; ++i) {
      const double dv = static_cast<double>(__half2float(k_src_value(A, src, pos0 + i, b, h, d))) - mean64;
      ss += dv * dv;
    }
    const __half mean = __double2half(mean64), sd = normal1_sd(ss, A.group);
    for (int w = 0; w < wpg; ++w) {
      uint32_t word = 0;
      for (int i = 0; i < 32; ++i) word |= normal1_code(k_src_value(A, src, pos0 + w * 32 + i, b, h, d), mean, sd) << i;
      dst[w] = word;
    }
    A.out_scale[row * Gd + jg] = sd;
    A.out_zero[row * Gd + jg] = mean;
    return;
  }
  const float levels = static_cast<float>((1 << bits) - 1);
  __half lo = k_src_value(A, src, pos0, b, h, d), hi = lo;
  for (int i = 1; i < A.group; ++i) {
    const __half v = k_src_value(A, src, pos0 + i, b, h, d);
    lo = h_min(lo, v);
    hi = h_max(hi, v);
  }
  const __half sc = quant_scale(lo, hi, levels);
  const QuantGroup qg = quant_group(lo, sc, levels);
  for (int w = 0; w < wpg; ++w) {
    uint32_t word = 0;
    for (int i = 0; i < fpi; ++i)
      word |= quant_code_fast(k_src_value(A, src, pos0 + w * fpi + i, b, h, d), qg) << (i * bits);
    dst[w] = word;
  }
  A.out_scale[row * Gd + jg] = sc;
  A.out_zero[row * Gd + jg] = lo;
}

__global__ void __launch_bounds__(D) flush_build_k_kernel(const __grid_constant__ BuildArgs A) {
  const int bh = blockIdx.y, b = bh / A.H, h = bh - b * A.H;
  build_k_group(A, blockIdx.x, bh, b, h, threadIdx.x);  // one destination group per CTA
}

// V side: a warp per destination token of a (batch, head); a lane owns 4 consecutive channels.
__device__ __forceinline__ void build_v_token(const BuildArgs& A, int64_t j, int bh, int b, int h, int lane) {
  const int32_t enc = A.plan[j];
  const int src = (enc >> 28) - 1;
  const int64_t pos = enc & 0x0FFFFFFF;
  const int bits = A.dst_bits;
  const int ng = D >> A.gshift;
  const int c0 = lane * 4;
  // ---- source values of this lane's 4 channels
  __half v[4];
  if (src < 0) {
    const __half* r = A.residual + b * A.res_b_stride + h * A.res_h_stride + pos * D + c0;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = r[i];
  } else if (src == 0) {
    const __half* r = reinterpret_cast<const __half*>(A.data[0]) + (static_cast<int64_t>(bh) * A.n[0] + pos) * D + c0;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = r[i];
  } else {
    const int sb = tier_bits(src), fpi = 32 / sb;
    const int64_t trow = static_cast<int64_t>(bh) * A.n[src] + pos;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(A.data[src]) + trow * (D / fpi);
    if (src == A.dst_tier) {  // kept token: copy the row verbatim
      uint32_t* dw = reinterpret_cast<uint32_t*>(A.out_data) + (static_cast<int64_t>(bh) * A.n_dst + j) * (D / fpi);
      for (int w = lane; w < D / fpi; w += 32) dw[w] = words[w];
      if (lane < ng) {
        A.out_scale[(static_cast<int64_t>(bh) * A.n_dst + j) * ng + lane] = A.scale[src][trow * ng + lane];
        A.out_zero[(static_cast<int64_t>(bh) * A.n_dst + j) * ng + lane] = A.zero[src][trow * ng + lane];
      }
      return;
    }
    const __half sc = A.scale[src][trow * ng + (c0 >> A.gshift)];
    const __half z = A.zero[src][trow * ng + (c0 >> A.gshift)];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = c0 + i;
      const uint32_t code = (words[c / fpi] >> ((c % fpi) * sb)) & ((1u << sb) - 1u);
      v[i] = dequant_2r(code, sc, z);
    }
  }
  if (bits == 16) {
    __half* dst = reinterpret_cast<__half*>(A.out_data) + (static_cast<int64_t>(bh) * A.n_dst + j) * D + c0;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = v[i];
    return;
  }
  // ---- quantise groups of `group` channels = group/4 adjacent lanes
  __half lo, sc;  // zero and scale of the group (mean and std in the Gaussian-codebook codec)
  uint32_t part = 0;
  if (A.normal_dst) {
    double sum = 0.0;
#pragma unroll
    for (int i = 0; i < 4; ++i) sum += static_cast<double>(__half2float(v[i]));
    for (int off = 1; off < (A.group >> 2); off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const double mean64 = sum / A.group;
    double ss = 0.0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const double dv = static_cast<double>(__half2float(v[i])) - mean64;
      ss += dv * dv;
    }
    for (int off = 1; off < (A.group >> 2); off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    lo = __double2half(mean64);
    sc = normal1_sd(ss, A.group);
#pragma unroll
    for (int i = 0; i < 4; ++i) part |= normal1_code(v[i], lo, sc) << i;
  } else {
    const float levels = static_cast<float>((1 << bits) - 1);
    __half hi = v[0];
    lo = v[0];
#pragma unroll
    for (int i = 1; i < 4; ++i) {
      lo = h_min(lo, v[i]);
      hi = h_max(hi, v[i]);
    }
    for (int off = 1; off < (A.group >> 2); off <<= 1) {
      lo = h_min(lo, __shfl_xor_sync(0xffffffffu, lo, off));
      hi = h_max(hi, __shfl_xor_sync(0xffffffffu, hi, off));
    }
    sc = quant_scale(lo, hi, levels);
#pragma unroll
    for (int i = 0; i < 4; ++i) part |= quant_code_fast(v[i], quant_group(lo, sc, levels)) << (i * bits);
  }
  const int lpw = 32 / (4 * bits);  // lanes per word: 1, 2, 4, 8 for 8, 4, 2, 1 bits
  for (int off = 1; off < lpw; off <<= 1) {
    const uint32_t other = __shfl_down_sync(0xffffffffu, part, off);
    part |= other << (4 * bits * off);
  }
  const int fpi = 32 / bits;
  uint32_t* dw = reinterpret_cast<uint32_t*>(A.out_data) + (static_cast<int64_t>(bh) * A.n_dst + j) * (D / fpi);
  if (lane % lpw == 0) dw[lane / lpw] = part;
  if ((c0 & (A.group - 1)) == 0) {
    A.out_scale[(static_cast<int64_t>(bh) * A.n_dst + j) * ng + (c0 >> A.gshift)] = sc;
    A.out_zero[(static_cast<int64_t>(bh) * A.n_dst + j) * ng + (c0 >> A.gshift)] = lo;
  }
}

__global__ void __launch_bounds__(128) flush_build_v_kernel(const __grid_constant__ BuildArgs A) {
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / A.H, h = bh - b * A.H;
  const int64_t j0 = (static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5)) * A.per_warp;
  for (int i = 0; i < A.per_warp; ++i)
    if (j0 + i < A.n_dst) build_v_token(A, j0 + i, bh, b, h, lane);  // the whole warp takes the same branch
}

__global__ void __launch_bounds__(256) gather_columns_kernel(const __half* __restrict__ in, int64_t in_stride,
                                                             const int64_t* __restrict__ ids, int64_t n,
                                                             __half* __restrict__ out, int64_t out_stride) {
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const int r = blockIdx.y;
  out[r * out_stride + j] = in[r * in_stride + ids[j]];
}

static int ilog2(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

static int fill_build_args(BuildArgs& A, const hqkv_flush_src_t* src, int B, int H, int Dd, int group, int dst_tier,
                           const int32_t* plan, int64_t n_dst, void* out_data, void* out_scale, void* out_zero,
                           const char* who) {
  HQKV_REQUIRE(src != nullptr, "%s: null source descriptor", who);
  HQKV_REQUIRE(Dd == D, "%s: head dim must be 128", who);
  HQKV_REQUIRE(B > 0 && H > 0 && static_cast<int64_t>(B) * H <= 65535, "%s: bad B/H", who);
  HQKV_REQUIRE(valid_group(group), "%s: group must be 32, 64 or 128", who);
  HQKV_REQUIRE(dst_tier >= 0 && dst_tier < HQKV_NUM_TIERS, "%s: dst_tier out of range", who);
  HQKV_REQUIRE(n_dst >= 0, "%s: negative n_dst", who);
  memset(&A, 0, sizeof(A));
  for (int t = 0; t < HQKV_NUM_TIERS; ++t) {
    A.data[t] = src->data[t];
    A.scale[t] = static_cast<const __half*>(src->scale[t]);
    A.zero[t] = static_cast<const __half*>(src->zero[t]);
    A.n[t] = src->n[t];
  }
  A.residual = static_cast<const __half*>(src->residual);
  A.res_b_stride = src->residual_b_stride;
  A.res_h_stride = src->residual_h_stride;
  A.B = B;
  A.H = H;
  A.group = group;
  A.gshift = ilog2(group);
  A.dst_tier = dst_tier;
  A.dst_bits = 16 >> dst_tier;
  HQKV_REQUIRE(src->low_codec == HQKV_CODEC_UNIFORM || src->low_codec == HQKV_CODEC_NORMAL, "%s: unknown low_codec %d",
               who, src->low_codec);
  A.normal_dst = (A.dst_bits == 1 && src->low_codec == HQKV_CODEC_NORMAL) ? 1 : 0;
  A.plan = plan;
  A.n_dst = n_dst;
  A.out_data = out_data;
  A.out_scale = static_cast<__half*>(out_scale);
  A.out_zero = static_cast<__half*>(out_zero);
  if (n_dst > 0) {
    HQKV_REQUIRE(plan && out_data, "%s: null pointer", who);
    HQKV_REQUIRE(dst_tier == 0 || (out_scale && out_zero), "%s: null scale/zero output", who);
  }
  return HQKV_OK;
}

}  // namespace hqkv

using namespace hqkv;

extern "C" int hqkv_head_sum(const void* w, int B, int nh, int64_t L, int64_t bh_stride, void* out, void* stream) {
  HQKV_REQUIRE(B > 0 && nh > 0 && L >= 0 && bh_stride >= L, "head_sum: bad sizes");
  if (L == 0) return HQKV_OK;
  HQKV_REQUIRE(w && out, "head_sum: null pointer");
  head_sum_kernel<<<static_cast<unsigned>(ceil_div(L, 32)), HEAD_SUM_THREADS, 0,
                    static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(w), B, nh, L, bh_stride, static_cast<__half*>(out));
  HQKV_LAUNCH_CHECK("head_sum");
  return HQKV_OK;
}

extern "C" int hqkv_token_importance(const void* ring, int rows, int64_t ring_stride, int64_t L, void* out,
                                     void* stream) {
  HQKV_REQUIRE(rows > 0 && L >= 0 && ring_stride >= L, "token_importance: bad sizes");
  if (L == 0) return HQKV_OK;
  HQKV_REQUIRE(ring && out, "token_importance: null pointer");
  token_importance_kernel<<<static_cast<unsigned>(ceil_div(L, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(ring), rows, ring_stride, L, static_cast<__half*>(out));
  HQKV_LAUNCH_CHECK("token_importance");
  return HQKV_OK;
}

extern "C" int hqkv_token_range(const void* v, int B, int H, int64_t T, int Dd, int64_t b_stride, int64_t h_stride,
                                void* out, void* stream) {
  HQKV_REQUIRE(B > 0 && H > 0 && T >= 0 && Dd >= 32, "token_range: bad sizes");
  if (T == 0) return HQKV_OK;
  HQKV_REQUIRE(v && out, "token_range: null pointer");
  if (Dd == 128 && aligned(v, 8) && b_stride % 4 == 0 && h_stride % 4 == 0) {
    token_range128_kernel<<<static_cast<unsigned>(ceil_div(T, 4)), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(v), B, H, T, b_stride, h_stride, static_cast<__half*>(out));
  } else {
    token_range_kernel<<<static_cast<unsigned>(ceil_div(T, 4)), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(v), B, H, T, Dd, b_stride, h_stride, static_cast<__half*>(out));
  }
  HQKV_LAUNCH_CHECK("token_range");
  return HQKV_OK;
}

extern "C" int hqkv_block_rank(void* importance, const void* range_or_null, int block, int nblocks,
                               int64_t* sorted_ids, void* stream) {
  HQKV_REQUIRE(block > 0 && nblocks >= 0, "block_rank: bad sizes");
  HQKV_REQUIRE(nblocks <= RANK_MAX_BLOCKS, "block_rank: at most %d blocks (got %d)", RANK_MAX_BLOCKS, nblocks);
  if (nblocks == 0) return HQKV_OK;
  HQKV_REQUIRE(importance && sorted_ids, "block_rank: null pointer");
  int npow2 = 2;
  while (npow2 < nblocks) npow2 <<= 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(RANK_CLUSTER);
  cfg.blockDim = dim3(RANK_THREADS);
  cfg.dynamicSmemBytes = npow2 * sizeof(uint32_t);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = RANK_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  HQKV_CUDA(cudaLaunchKernelEx(&cfg, block_rank_kernel, static_cast<__half*>(importance),
                               static_cast<const __half*>(range_or_null), block, nblocks, npow2, sorted_ids));
  return HQKV_OK;
}

extern "C" size_t hqkv_flush_plan_workspace_bytes(int64_t total) {
  if (total < 0) return 0;
  const size_t t = static_cast<size_t>(total);
  // tgt (1 B) + fin (1 B) + rank (4 B) per token, each region rounded to 256 bytes; per-warp counts; flags
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  return up(t) + up(t) + up(4 * t) + up(sizeof(int32_t) * PLAN_CATS * PLAN_GWARPS) + 256;
}

extern "C" int hqkv_flush_plan(const int64_t* const* tier_idx_host, const int32_t* tier_n_host, int64_t hist,
                               int64_t compress, const int64_t* sorted_ids, const int64_t* cum_counts_host,
                               int32_t* plan_src, int64_t* plan_ids, int64_t* survivors, int32_t* counts,
                               void* workspace, size_t workspace_bytes, void* stream) {
  HQKV_REQUIRE(tier_idx_host && tier_n_host && cum_counts_host, "flush_plan: null host pointer");
  HQKV_REQUIRE(hist >= 0 && compress >= 0, "flush_plan: negative length");
  const int64_t total = hist + compress;
  HQKV_REQUIRE(total > 0 && total < (1ll << 28), "flush_plan: total length out of range");
  HQKV_REQUIRE(sorted_ids && plan_src && plan_ids && survivors && counts && workspace, "flush_plan: null pointer");
  int64_t in_tiers = 0;
  PlanArgs A;
  memset(&A, 0, sizeof(A));
  for (int t = 0; t < HQKV_NUM_TIERS; ++t) {
    HQKV_REQUIRE(tier_n_host[t] >= 0, "flush_plan: negative tier size");
    HQKV_REQUIRE(tier_n_host[t] == 0 || tier_idx_host[t], "flush_plan: tier %d has tokens but no id list", t);
    A.tier_idx[t] = tier_idx_host[t];
    A.tier_n[t] = tier_n_host[t];
    in_tiers += tier_n_host[t];
  }
  HQKV_REQUIRE(in_tiers == hist, "flush_plan: tiers hold %lld tokens but history_length is %lld", (long long)in_tiers,
               (long long)hist);
  int64_t prev = 0;
  for (int k = 0; k < 6; ++k) {
    HQKV_REQUIRE(cum_counts_host[k] >= prev && cum_counts_host[k] <= total,
                 "flush_plan: cumulative counts must be non-decreasing and at most hist+compress");
    A.cum[k] = cum_counts_host[k];
    prev = cum_counts_host[k];
  }
  const size_t need = hqkv_flush_plan_workspace_bytes(total);
  if (workspace_bytes < need)
    return fail(HQKV_E_WORKSPACE, "flush_plan: workspace holds %zu bytes, %zu needed", workspace_bytes, need);
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  A.tgt = reinterpret_cast<int8_t*>(ws);
  A.fin = reinterpret_cast<int8_t*>(ws + up(total));
  A.rank = reinterpret_cast<int32_t*>(ws + 2 * up(total));
  A.gcnt = reinterpret_cast<int32_t*>(ws + 2 * up(total) + up(4 * static_cast<size_t>(total)));
  A.flags = A.gcnt + ((up(sizeof(int32_t) * PLAN_CATS * PLAN_GWARPS)) / sizeof(int32_t));
  A.hist = hist;
  A.compress = compress;
  A.sorted_ids = sorted_ids;
  A.plan_src = plan_src;
  A.plan_ids = plan_ids;
  A.survivors = survivors;
  A.counts = counts;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(PLAN_CLUSTER);
  cfg.blockDim = dim3(PLAN_THREADS);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PLAN_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  HQKV_CUDA(cudaLaunchKernelEx(&cfg, flush_plan_kernel, A));
  return HQKV_OK;
}

extern "C" int hqkv_flush_build_k(const hqkv_flush_src_t* src_host, int B, int H, int Dd, int group, int dst_tier,
                                  const int32_t* plan_src_row, int64_t n_dst, void* out_data, void* out_scale,
                                  void* out_zero, void* stream) {
  BuildArgs A;
  int rc = fill_build_args(A, src_host, B, H, Dd, group, dst_tier, plan_src_row, n_dst, out_data, out_scale, out_zero,
                           "flush_build_k");
  if (rc) return rc;
  if (n_dst == 0) return HQKV_OK;
  HQKV_REQUIRE(n_dst % group == 0, "flush_build_k: n_dst (%lld) is not a multiple of the group %d", (long long)n_dst,
               group);
  flush_build_k_kernel<<<dim3(static_cast<unsigned>(n_dst / group), B * H), D, 0,
                         static_cast<cudaStream_t>(stream)>>>(A);
  HQKV_LAUNCH_CHECK("flush_build_k");
  return HQKV_OK;
}

extern "C" int hqkv_flush_build_v(const hqkv_flush_src_t* src_host, int B, int H, int Dd, int group, int dst_tier,
                                  const int32_t* plan_src_row, int64_t n_dst, void* out_data, void* out_scale,
                                  void* out_zero, void* stream) {
  BuildArgs A;
  int rc = fill_build_args(A, src_host, B, H, Dd, group, dst_tier, plan_src_row, n_dst, out_data, out_scale, out_zero,
                           "flush_build_v");
  if (rc) return rc;
  if (n_dst == 0) return HQKV_OK;
  // a token row is little work for a warp: beyond ~64k CTAs the launch is bound by CTA scheduling and warps
  // take several tokens each (222 -> 169 us at 200k CTAs); smaller launches are faster with one token per warp
  const int64_t ctas = ceil_div(n_dst, 4) * B * H;
  const int64_t per = ceil_div(ctas, 65536);
  A.per_warp = static_cast<int>(per < 1 ? 1 : per > BUILD_V_TOKENS_MAX ? BUILD_V_TOKENS_MAX : per);
  flush_build_v_kernel<<<dim3(static_cast<unsigned>(ceil_div(n_dst, 4 * A.per_warp)), B * H), 128, 0,
                         static_cast<cudaStream_t>(stream)>>>(A);
  HQKV_LAUNCH_CHECK("flush_build_v");
  return HQKV_OK;
}

extern "C" int hqkv_gather_columns_f16(const void* in, int64_t in_stride, int rows, const int64_t* ids, int64_t n,
                                       void* out, int64_t out_stride, void* stream) {
  HQKV_REQUIRE(rows >= 0 && n >= 0, "gather_columns: negative size");
  if (rows == 0 || n == 0) return HQKV_OK;
  HQKV_REQUIRE(in && ids && out, "gather_columns: null pointer");
  HQKV_REQUIRE(rows <= 65535, "gather_columns: too many rows");
  gather_columns_kernel<<<dim3(static_cast<unsigned>(ceil_div(n, 256)), rows), 256, 0,
                          static_cast<cudaStream_t>(stream)>>>(static_cast<const __half*>(in), in_stride, ids, n,
                                                               static_cast<__half*>(out), out_stride);
  HQKV_LAUNCH_CHECK("gather_columns");
  return HQKV_OK;
}
