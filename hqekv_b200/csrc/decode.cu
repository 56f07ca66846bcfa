// Fused mixed-precision decode attention over the tiered KV cache (sm_100a): ONE launch per call.
//
// The work of a (batch, kv head) pair is a list of K tiles (logits of 64 / 128 tokens of one tier) followed by a
// list of V tiles (exp, p.V of 64 / 128 tokens), see decode_tiles.cuh.  The grid is persistent: at most as many
// CTAs as fit on the GPU at once (two per SM), each of eight warps.  With fewer pairs than CTAs every pair is
// shared by a GROUP of m consecutive CTAs, each taking an equal slice of both lists (every warp an eighth of its
// CTA's slice); with more pairs than CTAs every CTA takes whole pairs, one after the other (a group of one).
//
//   K slice : logits written to an fp32 scratch row at the tokens' logical positions, a running (max, sum-exp)
//             per head.  A group of one folds its warps' pairs in shared memory.  A larger group publishes one
//             pair per head and CTA, counts itself in on the pair's arrival counter and
//   waits   - the first V tile has been requested before (V tiles do not depend on the logits) - until the K
//             side of its pair is complete, then folds the published pairs into the global (max, sum).  The wait
//             is bounded: a count that does not arrive within the spin limit is recorded in the status word and
//             the CTA goes on.
//   V slice : every warp writes the normalised probabilities of its tokens and adds sum_t exp(logit_t - max) *
//             V_t into its partial output in shared memory; the CTA's warps are added up.  A group of one
//             normalises and writes fp16 at once; in a larger group the sums join fp64 accumulators with
//             fire-and-forget reductions and the last CTA of the pair normalises and writes.
//
// Code size is a first-order cost here: with one tile per warp every instruction is executed about once per
// launch, so a launch walks through its code at instruction-fetch speed.  Hence one (batch, kv head) pair per
// CTA at a time (no tables, no divisions), request routines written once for all bit widths and not inlined,
// and step loops that are not unrolled.
//
// The launch is chained with programmatic dependent launch: what a CTA needs only from the cache (its
// first K tile) is requested before it waits for the kernels ahead of it in the stream, and the next
// kernel's CTAs may take the places of CTAs that have finished.
#include <string.h>

#include "decode_tiles.cuh"

namespace hqkv {

constexpr int NWARPS = 8;
constexpr int NTHREADS = NWARPS * 32;
constexpr int NUM_ITEM_TIERS = HQKV_NUM_TIERS + 1;  // [5] = fp16 residual window (token-major K and V)
constexpr int CTAS_PER_SM = 2;
constexpr int WS_KDONE_OFF = 0, WS_VDONE_OFF = 4096, WS_STATUS_OFF = 8192;  // inside the zeroed workspace header
constexpr int MAX_BH = 1024;
static_assert(HQKV_WS_HEADER_BYTES >= WS_STATUS_OFF + 64 && MAX_BH * 4 <= 4096, "workspace header layout");

struct DecodeParams {
  TierDev tier[NUM_ITEM_TIERS];
  int B, H, nh_q, rep, rep_shift, L;
  int gk_shift, gv_shift;
  int phases;     // bit 0: K slices, bit 1: V slices
  int kc_max;     // slots per (batch, kv head) in k_part
  int warp_smem;  // bytes of one warp's shared-memory region
  int cta_smem;   // bytes of the CTA-shared block ahead of the warps' regions
  int wk, wv;     // weight of all tiles of one (batch, kv head) on the K / V side
  int k_first, v_first;  // first tier that has tiles on that side
  // grouping: the first g_rem pairs have groups of g_m + 1 CTAs, the others of g_m; g_m == 0: whole pairs per CTA
  int g_m, g_rem;
  float g_inv[2];        // 1 / g_m, 1 / (g_m + 1)
  int kq[2], kr[2];      // wk / m and wk % m for m = g_m, g_m + 1: CTA i of m takes K weights [i*q + min(i, r), ...)
  int vq[2], vr[2];      // the same for wv
  float scale;
  const __half* q;
  const __half* mask;      // non-null: additive mask on the logits, fp16, element (b, head, pos) at b*mask_bstride + head*mask_hstride + pos
  long long mask_bstride, mask_hstride;
  const __half* probs_in;  // non-null: the V slices multiply these caller-supplied weights [B*nh_q][L] instead of exp(logit - max)
  __half* weights;
  __half* out;
  float* logits;   // [B*nh_q][L]
  float2* k_part;  // [B*H][kc_max][MAX_REP]
  double* v_acc;   // [B*H][rep][D] output accumulators: cleared by the K slices, summed into by the V slices
  unsigned* kdone;  // [B*H] CTAs whose K slice of this (batch, kv head) is complete
  unsigned* vdone;  // [B*H] the same for the V slices
  unsigned* status; // 0, or 1 + (batch, kv head) whose K side did not complete within the spin limit
  long long spin_limit;
  __half* peer_out[HQKV_MAX_PEERS];  // copies of `out` in other GPUs' memory (kv-head sharding), n_peers used
  int n_peers;
  int peer_flagged;  // 1: peer_out are flagged 8-byte entries {two fp16 values, call number}, see peer_unpack_kernel
  // cross-GPU barrier run by the CTA that finishes this GPU's last (batch, kv head) (world == 0: none)
  unsigned* pad[HQKV_MAX_PEERS + 1];  // the ranks' signal pads, own one included
  int rank, world;
  unsigned* peer_state;  // call number, status, finished (batch, kv head) count
  long long max_spins;
};

struct CtaShared {
  float gm[MAX_REP], gl[MAX_REP];  // global max / sum-exp of the pair's query heads
  unsigned is_last;
  unsigned bar_n;
  unsigned pad_[2];
};
constexpr int CTA_HEAD_BYTES = 128;
static_assert(sizeof(CtaShared) <= CTA_HEAD_BYTES, "CTA-shared block");
// after it: q of the CTA's current pair, 4 (8) rows of Q_PITCH halfs
__host__ __device__ constexpr int cta_shared_bytes(bool rep8) { return CTA_HEAD_BYTES + (rep8 ? 8 : 4) * Q_PITCH * 2; }
// two CTAs per SM: 2 x (dynamic + 1 KB reserved) must fit the 228 KB of an SM
static_assert(2 * (cta_shared_bytes(false) + NWARPS * ws_bytes(false) + 1024) <= 233472, "two CTAs per SM");

// ------------------------------------------------------------------------------------------------
// work lists
// ------------------------------------------------------------------------------------------------
// A pair's tiles of one side are ordered by tier, then tile; tile i of a tier starts at weight w0(tier) +
// i * w(tier).  A tile belongs to the warp whose weight range holds its start weight.
struct Cursor {
  int tier, tile;
  int s;  // start weight
};
template <bool K> __device__ __forceinline__ int t_tiles(const TierDev& T) { return K ? T.k_tiles : T.v_tiles; }
template <bool K> __device__ __forceinline__ int t_w(const TierDev& T) { return K ? T.k_w : T.v_w; }
template <bool K> __device__ __forceinline__ int t_w0(const TierDev& T) { return K ? T.k_w0 : T.v_w0; }

// first tile whose start weight is >= a (s = the side's total weight if there is none)
template <bool K>
__device__ __noinline__ Cursor cursor_at(const DecodeParams& P, int a) {
  Cursor c;
  c.tier = NUM_ITEM_TIERS;
  c.tile = 0;
  c.s = K ? P.wk : P.wv;
#pragma unroll 1
  for (int t = 0; t < NUM_ITEM_TIERS; ++t) {
    const TierDev& T = P.tier[t];
    const int n = t_tiles<K>(T), w = t_w<K>(T), w0 = t_w0<K>(T);
    if (n > 0 && c.tier == NUM_ITEM_TIERS) {
      const int d = a - w0;  // weights are 1, 3 or 4 in practice: no general integer division for those
      const int tile = d <= 0 ? 0 : (w == 4 ? (d + 3) >> 2 : w == 3 ? (d + 2) / 3 : w == 1 ? d : (d + w - 1) / w);
      if (tile < n) {
        c.tier = t;
        c.tile = tile;
        c.s = w0 + tile * w;
      }
    }
  }
  return c;
}
template <bool K>
__device__ __forceinline__ void cursor_next(const DecodeParams& P, Cursor& c) {
  if (++c.tile >= t_tiles<K>(P.tier[c.tier])) {
    c.tile = 0;
    do {
      ++c.tier;
    } while (c.tier < NUM_ITEM_TIERS && t_tiles<K>(P.tier[c.tier]) == 0);
  }
  c.s = c.tier < NUM_ITEM_TIERS ? t_w0<K>(P.tier[c.tier]) + c.tile * t_w<K>(P.tier[c.tier]) : (K ? P.wk : P.wv);
}

// (not inlined: called from several places, once per tile)
__device__ __noinline__ void k_request(const DecodeParams& P, const Cursor c, int bh, unsigned char* wsm) {
  if (c.tier >= HQKV_NUM_TIERS) return;
  const TierDev& T = P.tier[c.tier];
  if (T.bits == 16) return;  // fp16 tier: read straight from global memory
  const int t0 = c.tile * T.k_tile_tokens;
  k_tile_request(T, wsm, bh, t0, min(T.k_tile_tokens, T.n_k - t0), P.gk_shift);
}
__device__ __noinline__ uint4 v_request(const DecodeParams& P, const Cursor c, int bh, unsigned char* wsm) {
  uint32_t pos[4] = {0u, 0u, 0u, 0u};
  if (c.tier < HQKV_NUM_TIERS && P.tier[c.tier].bits < 16) {
    const TierDev& T = P.tier[c.tier];
    const int t0 = c.tile * T.v_tile_tokens, ntok = min(T.v_tile_tokens, T.n_v - t0);
    v_tile_positions(T, t0, ntok, pos);
    v_tile_request(T, wsm, bh, t0, ntok, D >> P.gv_shift);
  }
  return make_uint4(pos[0], pos[1], pos[2], pos[3]);
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
    if (FENCE_FIRST) __threadfence_system();  // this GPU's earlier peer stores first (the decode kernel has fenced them already)
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

__global__ void __launch_bounds__(NTHREADS, CTAS_PER_SM) decode_kernel(const __grid_constant__ DecodeParams P) {
  extern __shared__ __align__(128) unsigned char smem[];
  CtaShared& cs = *reinterpret_cast<CtaShared*>(smem);
  __half* qsm = reinterpret_cast<__half*>(smem + CTA_HEAD_BYTES);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* wsm = smem + P.cta_smem + warp * P.warp_smem;
  const bool rep8 = P.rep > 4;
  const int rep = P.rep;
  const int BH = P.B * P.H;
  const bool do_k = (P.phases & 1) != 0, do_v = (P.phases & 2) != 0;

  // The next kernel of the stream - the next decode call, if it was launched with programmatic stream
  // serialisation - may place its CTAs as soon as CTAs of this grid have finished; it requests its
  // first K tile and then waits for this grid to complete.
  asm volatile("griddepcontrol.launch_dependents;");

  // ---- this CTA's (batch, kv head) pair(s) and its place in the pair's group
  int bh, gi = 0, gm_ = 1, sel = 0, bh_step;
  if (P.g_m == 0) {  // more pairs than CTAs: whole pairs, one after the other
    bh = blockIdx.x;
    bh_step = gridDim.x;
  } else {
    const int c = blockIdx.x, big = P.g_rem * (P.g_m + 1);  // CTAs in the groups of g_m + 1
    if (c < big) {
      sel = 1;
      gm_ = P.g_m + 1;
      bh = static_cast<int>((c + 0.5f) * P.g_inv[1]);
      gi = c - bh * gm_;
    } else {
      gm_ = P.g_m;
      const int c2 = c - big, j = static_cast<int>((c2 + 0.5f) * P.g_inv[0]);
      bh = P.g_rem + j;
      gi = c2 - j * gm_;
    }
    bh_step = BH;  // one pair
  }
  const bool local = gm_ == 1 && P.phases == 3 && P.probs_in == nullptr;  // the CTA has the whole pair: no global hand-over
  float2* kstat = reinterpret_cast<float2*>(wsm + WS_KSTAT);  // this warp's (max, sum-exp) per head
  bool first_unit = true;
  unsigned finished = 0u;  // pairs this CTA wrote the output of (multi-GPU hand-over)

  for (; bh < BH; bh += bh_step) {
    const int b = bh / P.H, kvh = bh - b * P.H;
    const int64_t head0 = static_cast<int64_t>(b) * P.nh_q + kvh * rep;
    // weights of this CTA, then of this warp, on both sides
    const int ka0 = gi * P.kq[sel] + min(gi, P.kr[sel]), ka1 = ka0 + P.kq[sel] + (gi < P.kr[sel] ? 1 : 0);
    const int va0 = gi * P.vq[sel] + min(gi, P.vr[sel]), va1 = va0 + P.vq[sel] + (gi < P.vr[sel] ? 1 : 0);
    const int k_end = ka0 + (((ka1 - ka0) * (warp + 1)) >> 3), v_end = va0 + (((va1 - va0) * (warp + 1)) >> 3);
    Cursor cur, vcur;
    bool have = false, vhave = false;
    uint32_t vpos[4] = {0u, 0u, 0u, 0u};
    if (do_k) {
      cur = cursor_at<true>(P, ka0 + (((ka1 - ka0) * warp) >> 3));
      have = cur.s < k_end;
      if (have) k_request(P, cur, bh, wsm);  // reads only the cache
    }
    if (do_v) {
      vcur = cursor_at<false>(P, va0 + (((va1 - va0) * warp) >> 3));
      vhave = vcur.s < v_end;
      if (!do_k && vhave) {
        const uint4 r = v_request(P, vcur, bh, wsm);
        vpos[0] = r.x, vpos[1] = r.y, vpos[2] = r.z, vpos[3] = r.w;
      }
    }
    if (first_unit) {
      // Everything above reads only the cache.  From here on this grid reads q and writes the scratch that
      // the previous decode call of the stream may still be using: wait for the kernels before it.
      asm volatile("griddepcontrol.wait;" ::: "memory");
      first_unit = false;
    }

    // -------------------------------------------------------------------------------------------
    // K slice
    // -------------------------------------------------------------------------------------------
    if (do_k) {
      // q of the pair -> shared memory (rows of heads that do not exist are zero)
      {
        const int rows = rep8 ? 8 : 4;
        for (int i = tid; i < rows * (D / 2); i += NTHREADS) {
          const int c2 = i & (D / 2 - 1), row = i >> 6;
          uint32_t v = 0u;
          if (row < rep) v = __ldcg(reinterpret_cast<const uint32_t*>(P.q + (head0 + row) * D) + c2);
          *reinterpret_cast<uint32_t*>(qsm + row * Q_PITCH + 2 * c2) = v;
        }
      }
      // The first CTA of a group clears the pair's output accumulators: the V slices add into them only after
      // the K side of the pair is complete, and this CTA is part of it.
      if (!local && gi == 0) {
        double* accum = P.v_acc + static_cast<int64_t>(bh) * rep * D;
        for (int e = tid; e < rep * D; e += NTHREADS) accum[e] = 0.0;
      }
      __syncthreads();
      KWarpState st;
      st.pm = -INFINITY;
      st.pl = 0.f;
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          st.m[i][e] = -INFINITY;
          st.l[i][e] = 0.f;
        }
      st.mask0 = P.mask ? P.mask + b * P.mask_bstride + static_cast<int64_t>(kvh * rep) * P.mask_hstride : nullptr;
      st.mask_hstride = P.mask_hstride;
      float* row0 = P.logits + head0 * P.L;
      bool streamed = false;  // the current tile was requested while the previous one was computed
      while (have) {
        const TierDev& T = P.tier[cur.tier];
        const int t0 = cur.tile * T.k_tile_tokens, ntok = min(T.k_tile_tokens, T.n_k - t0);
        Cursor nxt = cur;
        cursor_next<true>(P, nxt);
        const bool have_next = nxt.s < k_end;
        // the next tile streams into this tile's buffer if it continues the same tier
        const bool quant = cur.tier < HQKV_NUM_TIERS && T.bits < 16;
        const bool stream = quant && have_next && nxt.tier == cur.tier;
        const int nt0 = t0 + T.k_tile_tokens, nntok = stream ? min(T.k_tile_tokens, T.n_k - nt0) : 0;
        if (cur.tier == HQKV_NUM_TIERS) {
          k_residual_tile(T, wsm, st, qsm, bh, rep, P.rep_shift, P.L, P.scale, t0, row0);
        } else if (T.bits == 16) {
          k_f16_span(T, wsm, st, qsm, bh, rep, P.rep_shift, P.L, P.scale, t0, row0);
        } else if (T.bits == 8) {
          k_tile_compute<8>(T, wsm, st, qsm, bh, rep, P.L, P.gk_shift, P.scale, t0, ntok, row0, streamed, nt0, nntok);
        } else if (T.bits == 4) {
          k_tile_compute<4>(T, wsm, st, qsm, bh, rep, P.L, P.gk_shift, P.scale, t0, ntok, row0, streamed, nt0, nntok);
        } else if (T.bits == 2) {
          k_tile_compute<2>(T, wsm, st, qsm, bh, rep, P.L, P.gk_shift, P.scale, t0, ntok, row0, streamed, nt0, nntok);
        } else {
          k_tile_compute<1>(T, wsm, st, qsm, bh, rep, P.L, P.gk_shift, P.scale, t0, ntok, row0, streamed, nt0, nntok);
        }
        cur = nxt;
        have = have_next;
        streamed = stream;
        __syncwarp();  // every lane is done with the tile in shared memory
        if (have && !streamed) k_request(P, cur, bh, wsm);
      }
      k_emit_stats(st, kstat, reinterpret_cast<float2*>(wsm + WS_K_ZQ), rep);
      // the first V tile does not depend on the logits: request it before the hand-over
      if (do_v && vhave) {
        const uint4 r = v_request(P, vcur, bh, wsm);
        vpos[0] = r.x, vpos[1] = r.y, vpos[2] = r.z, vpos[3] = r.w;
      }
      __syncthreads();
      // ---- one (max, sum-exp) per head for the CTA's slice
      if (tid < MAX_REP) {
        float m = -INFINITY, l = 0.f;
#pragma unroll 1
        for (int w = 0; w < NWARPS; ++w) {
          const float2 v = reinterpret_cast<const float2*>(smem + P.cta_smem + w * P.warp_smem + WS_KSTAT)[tid];
          softmax_merge(m, l, v.x, v.y);
        }
        if (local) {
          cs.gm[tid] = m;
          cs.gl[tid] = l;
        } else {
          P.k_part[(static_cast<int64_t>(bh) * P.kc_max + gi) * MAX_REP + tid] = make_float2(m, l);
        }
      }
      if (!local) {
        __threadfence();  // this thread's logits (and pair) before the count below
        __syncthreads();
        if (tid == 0) atomicAdd(&P.kdone[bh], 1u);
      } else {
        __syncthreads();
      }
    }
    if (!do_v) continue;

    // -------------------------------------------------------------------------------------------
    // wait for the K side of the pair; fold the published pairs
    // -------------------------------------------------------------------------------------------
    if (P.probs_in) {  // weights are given: nothing to wait for, nothing to normalise by
      if (tid < MAX_REP) {
        cs.gm[tid] = 0.f;
        cs.gl[tid] = 1.f;
      }
      __syncthreads();
    } else if (!local) {
      if (warp == 0) {
        if (lane == 0) {
          const volatile unsigned* c = P.kdone + bh;
          long long spins = 0;
          while (*c < static_cast<unsigned>(gm_)) {
            if (++spins > P.spin_limit) {
              atomicExch(P.status, static_cast<unsigned>(bh) + 1u);  // gave up: the result of this call is not valid
              break;
            }
            __nanosleep(40);
          }
          __threadfence();
        }
        __syncwarp();
        const int head = lane & 7, slice = lane >> 3;
        const float2* part = P.k_part + static_cast<int64_t>(bh) * P.kc_max * MAX_REP;
        float m = -INFINITY, l = 0.f;
#pragma unroll 1
        for (int c0 = slice; c0 < gm_; c0 += 16) {
          float2 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + 4 * j;
            v[j] = (c < gm_ && head < rep) ? __ldcg(part + c * MAX_REP + head) : make_float2(-INFINITY, 0.f);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) softmax_merge(m, l, v[j].x, v[j].y);
        }
#pragma unroll
        for (int off = 8; off < 32; off <<= 1) {
          const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
          const float l2 = __shfl_xor_sync(0xffffffffu, l, off);
          softmax_merge(m, l, m2, l2);
        }
        if (lane < MAX_REP) {
          cs.gm[lane] = m;
          cs.gl[lane] = l;
        }
      }
      __syncthreads();
    }

    // -------------------------------------------------------------------------------------------
    // V slice
    // -------------------------------------------------------------------------------------------
    float(*out)[D] = reinterpret_cast<float(*)[D]>(wsm + ws_v_out(rep8));
    float* zt = reinterpret_cast<float*>(wsm + ws_v_zt(rep8));
    {
      const int out_elems = (rep8 ? 8 : 4) * D;
      for (int i = lane * 4; i < out_elems; i += 128) *reinterpret_cast<float4*>(&out[0][0] + i) = make_float4(0.f, 0.f, 0.f, 0.f);
      zt[lane] = 0.f;  // 4 x MAX_REP floats
      __syncwarp();
    }
    const float* logit0 = P.logits + head0 * P.L;
    __half* w0 = P.weights + head0 * P.L;
    const __half* pin0 = P.probs_in ? P.probs_in + head0 * P.L : nullptr;
    while (vhave) {
      const TierDev& T = P.tier[vcur.tier];
      const int t0 = vcur.tile * T.v_tile_tokens, ntok = min(T.v_tile_tokens, T.n_v - t0);
      Cursor nxt = vcur;
      cursor_next<false>(P, nxt);
      const bool have_next = nxt.s < v_end;
      // the next tile streams into this tile's buffer if this one is full and the next continues the same tier;
      // its positions are fetched now, its rows during the walk over this tile
      const bool quant = vcur.tier < HQKV_NUM_TIERS && T.bits < 16;
      const bool stream = quant && have_next && nxt.tier == vcur.tier && ntok == T.v_tile_tokens;
      const int nt0 = t0 + T.v_tile_tokens, nntok = stream ? min(T.v_tile_tokens, T.n_v - nt0) : 0;
      uint32_t npos[4] = {0u, 0u, 0u, 0u};
      if (stream) v_tile_positions(T, nt0, nntok, npos);
      if (vcur.tier == HQKV_NUM_TIERS || T.bits == 16) {
        v_plain_tile(T, wsm, rep8, rep, P.L, cs.gm, cs.gl, bh, logit0, w0, pin0, t0, ntok, vcur.tier == HQKV_NUM_TIERS);
      } else if (T.bits == 8) {
        v_tile<8>(T, wsm, rep8, rep, P.L, P.gv_shift, cs.gm, cs.gl, vpos, logit0, w0, pin0, ntok, bh, nt0, nntok);
      } else if (T.bits == 4) {
        v_tile<4>(T, wsm, rep8, rep, P.L, P.gv_shift, cs.gm, cs.gl, vpos, logit0, w0, pin0, ntok, bh, nt0, nntok);
      } else if (T.bits == 2) {
        v_tile<2>(T, wsm, rep8, rep, P.L, P.gv_shift, cs.gm, cs.gl, vpos, logit0, w0, pin0, ntok, bh, nt0, nntok);
      } else {
        v_tile<1>(T, wsm, rep8, rep, P.L, P.gv_shift, cs.gm, cs.gl, vpos, logit0, w0, pin0, ntok, bh, nt0, nntok);
      }
      vcur = nxt;
      vhave = have_next;
      if (stream) {
#pragma unroll
        for (int j = 0; j < 4; ++j) vpos[j] = npos[j];
      } else if (vhave) {
        const uint4 r = v_request(P, vcur, bh, wsm);
        vpos[0] = r.x, vpos[1] = r.y, vpos[2] = r.z, vpos[3] = r.w;
      }
    }

    // ---- the warps' partial outputs are added up in warp order.  A group of one has the pair's whole sum:
    //      it normalises and writes.  In a larger group the sums join the pair's fp64 accumulators with
    //      fire-and-forget reductions (the sum of the fp32 partials depends on their order only below 2^-53, far
    //      below the fp16 rounding of the output, and no CTA has to read other CTAs' partials back), and the last
    //      CTA of the pair to arrive normalises and writes.
    __syncthreads();
    bool writes = local;
    if (!local) {
      for (int e = tid; e < rep * D; e += NTHREADS) {
        const int h = e >> 7, ch = e & (D - 1);
        float v = 0.f;
#pragma unroll 1
        for (int w = 0; w < NWARPS; ++w) {
          const unsigned char* o = smem + P.cta_smem + w * P.warp_smem;
          v += reinterpret_cast<const float*>(o + ws_v_out(rep8))[e] +
               reinterpret_cast<const float*>(o + ws_v_zt(rep8))[(ch >> P.gv_shift) * MAX_REP + h];
        }
        atomicAdd(P.v_acc + static_cast<int64_t>(bh) * rep * D + e, static_cast<double>(v));
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const unsigned prev = atomicAdd(&P.vdone[bh], 1u);
        cs.is_last = (prev == static_cast<unsigned>(gm_) - 1u) ? 1u : 0u;
      }
      __syncthreads();
      writes = cs.is_last != 0u;
      if (writes) __threadfence();
    }
    if (writes) {
      ++finished;
      const double* accum = P.v_acc + static_cast<int64_t>(bh) * rep * D;
      for (int e = tid * 2; e < rep * D; e += NTHREADS * 2) {
        float vx, vy;
        if (local) {
          const int h = e >> 7, ch = e & (D - 1);
          vx = vy = 0.f;
#pragma unroll 1
          for (int w = 0; w < NWARPS; ++w) {
            const unsigned char* o = smem + P.cta_smem + w * P.warp_smem;
            const float2 a = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(o + ws_v_out(rep8)) + e);
            const float z = reinterpret_cast<const float*>(o + ws_v_zt(rep8))[(ch >> P.gv_shift) * MAX_REP + h];
            vx += a.x + z;
            vy += a.y + z;
          }
        } else {
          const double2 v = __ldcg(reinterpret_cast<const double2*>(accum + e));
          vx = static_cast<float>(v.x);
          vy = static_cast<float>(v.y);
        }
        const float inv = 1.f / cs.gl[e >> 7];
        const __half2 o = __floats2half2_rn(vx * inv, vy * inv);
        const int64_t at = head0 * D + e;
        *reinterpret_cast<__half2*>(P.out + at) = o;
        // kv-head sharding: the same rows go straight into every peer's copy of the gathered output
        // (plain stores over NVLink; the callers' cross-GPU barrier makes them visible before use)
        if (P.peer_flagged) {
          // value and call number travel in ONE 8-byte store: the receiver needs no fence and no signal
          const uint2 w = make_uint2(h2_as_u32(o), P.peer_state[0] + 1u);
          for (int p = 0; p < P.n_peers; ++p) reinterpret_cast<uint2*>(P.peer_out[p])[at >> 1] = w;
        } else {
          for (int p = 0; p < P.n_peers; ++p) *reinterpret_cast<__half2*>(P.peer_out[p] + at) = o;
        }
      }
      if (!local && tid == 0) {  // every CTA of this pair has passed its wait and counted itself in
        P.kdone[bh] = 0u;
        P.vdone[bh] = 0u;
      }
    }
    __syncthreads();  // the shared memory of this pair is free for the next one
  }

  if (P.world > 1 && finished != 0u) {
    // the CTA that finishes the last (batch, kv head) of this GPU runs the cross-GPU barrier: when this
    // kernel completes, every rank's rows are in this GPU's gathered buffer
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
      const unsigned done = atomicAdd(P.peer_state + 2, finished);
      cs.bar_n = (done + finished == static_cast<unsigned>(BH)) ? 1u : 0u;
      if (cs.bar_n) P.peer_state[2] = 0u;
    }
    __syncthreads();
    if (cs.bar_n) {
      __threadfence();
      // every CTA fenced its peer stores system-wide before it counted itself in, and this CTA saw the
      // full count: the signal may go out at once
      peer_barrier_device<false>(P.pad, P.rank, P.world, P.peer_state, reinterpret_cast<int*>(P.peer_state + 1),
                                 P.max_spins, &cs.pad_[0]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static int sm_count() {
  static int cached[64] = {};
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return 148;  // B200
  }
  if (cached[dev] == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) {
      cached[dev] = n;
    } else {
      (void)cudaGetLastError();
      cached[dev] = 148;
    }
  }
  return cached[dev];
}

static int ilog2(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

struct Layout {
  size_t acc_off, logits_off, kpart_off, total;
  int smem_bytes;
  int ctas_per_sm;
  int grid;
};

// sides: bit 0 = the K side of the descriptor is used, bit 1 = the V side (a one-sided call ignores the other side's fields)
static int build_params(const hqkv_cache_desc_t* c, DecodeParams& P, Layout& lay, int sides = 3) {
  HQKV_REQUIRE(c != nullptr, "decode: null cache descriptor");
  HQKV_REQUIRE(c->B > 0 && c->H > 0 && c->nh_q > 0, "decode: B, H and nh_q must be positive");
  HQKV_REQUIRE(c->D == D, "decode: head dim must be 128 (got %d)", c->D);
  HQKV_REQUIRE(c->nh_q % c->H == 0 && c->nh_q / c->H <= MAX_REP,
               "decode: nh_q (%d) must be a multiple of H (%d) with at most %d query heads per kv head", c->nh_q,
               c->H, MAX_REP);
  HQKV_REQUIRE(valid_group(c->group_k) && valid_group(c->group_v), "decode: group sizes must be 32, 64 or 128");
  HQKV_REQUIRE(static_cast<int64_t>(c->B) * c->H <= MAX_BH, "decode: B*H must not exceed %d", MAX_BH);
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
  int64_t wk = 0, wv = 0;
  P.k_first = P.v_first = -1;
  for (int t = 0; t < HQKV_NUM_TIERS; ++t) {
    const hqkv_tier_t& s = c->tier[t];
    TierDev& d = P.tier[t];
    HQKV_REQUIRE(s.n_k >= 0 && s.n_v >= 0, "decode: negative tier size");
    d.bits = expect_bits[t];
    d.n_k = (sides & 1) ? s.n_k : 0;
    d.n_v = (sides & 2) ? s.n_v : 0;
    if (s.n_k > 0 || s.n_v > 0) {
      HQKV_REQUIRE(s.bits == expect_bits[t], "decode: tier %d must hold %d-bit data (got %d)", t, expect_bits[t], s.bits);
      HQKV_REQUIRE(s.codec == HQKV_CODEC_UNIFORM || (s.codec == HQKV_CODEC_NORMAL && s.bits == 1),
                   "decode: tier %d: codec %d is not valid at %d bits (the Gaussian codebook is built for the 1-bit tier)", t,
                   s.codec, s.bits);
      d.normal = s.codec == HQKV_CODEC_NORMAL ? 1 : 0;
    }
    if (d.n_k > 0) {
      HQKV_REQUIRE(s.k_data && s.k_idx, "decode: tier %d K pointers are null", t);
      HQKV_REQUIRE(aligned(s.k_idx, 8), "decode: tier %d K index list must be 8-byte aligned", t);
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
      HQKV_REQUIRE(s.v_data && s.v_idx, "decode: tier %d V pointers are null", t);
      HQKV_REQUIRE(aligned(s.v_idx, 8), "decode: tier %d V index list must be 8-byte aligned", t);
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
    // tiles: about the same number of bytes whatever the width
    const int b = d.bits;
    HQKV_REQUIRE(static_cast<int64_t>(s.n_k) * D * b / 8 < (1ll << 31), "decode: tier %d K plane of one head exceeds 2 GiB", t);
    d.k_tile_tokens = (b == 8 || b == 16) ? 64 : 128;
    d.v_tile_tokens = b == 8 ? 64 : b == 16 ? 16 : 128;
    d.k_tiles = static_cast<int>(ceil_div(d.n_k, d.k_tile_tokens));
    d.v_tiles = static_cast<int>(ceil_div(d.n_v, d.v_tile_tokens));
    // weights: a tile is first of all one load latency and one pass of per-tile work, so a 64-token tile or a tile
    // of the fp16 tier (read straight from global memory) counts three quarters of a 128-token tile
    d.k_w = d.k_tile_tokens == 64 ? 3 : 4;
    d.v_w = (b == 16 || d.v_tile_tokens == 64) ? 3 : 4;
    if (d.k_tiles > 0 && P.k_first < 0) P.k_first = t;
    if (d.v_tiles > 0 && P.v_first < 0) P.v_first = t;
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
  r.k_tile_tokens = r.v_tile_tokens = 16;
  r.k_tiles = r.v_tiles = static_cast<int>(ceil_div(c->n_new, 16));
  r.k_w = r.v_w = 3;
  if (r.k_tiles > 0 && P.k_first < 0) P.k_first = HQKV_NUM_TIERS;
  if (r.v_tiles > 0 && P.v_first < 0) P.v_first = HQKV_NUM_TIERS;
  const int64_t L = ((sides & 1) ? nk_total : nv_total) + c->n_new;
  HQKV_REQUIRE(L > 0, "decode: the cache is empty");
  HQKV_REQUIRE(L < (1ll << 30), "decode: cache too long");
  P.L = static_cast<int>(L);
  const bool rep8 = P.rep > 4;
  const int64_t BH = static_cast<int64_t>(c->B) * c->H;
  const int ctas_per_sm = rep8 ? 1 : CTAS_PER_SM;
#ifdef HQKV_X_GRID_PER_SM
  const int max_cta = HQKV_X_GRID_PER_SM * sm_count();
#else
  const int max_cta = ctas_per_sm * sm_count();
#endif
  {
    // Grouping.  Fewer pairs than CTAs: every pair gets a group of m CTAs, m chosen so that a warp holds about one
    // tile of the longer side (and all groups fit the GPU at once: the wait between the K slices and the V slices
    // relies on it).  When a warp holds at most one tile of a side, what a tile costs is its chain of latencies
    // whatever its size: all tiles weigh the same; otherwise the weights above.
    int64_t tk = 0, tv = 0;
    for (int t = 0; t < NUM_ITEM_TIERS; ++t) {
      tk += P.tier[t].k_tiles;
      tv += P.tier[t].v_tiles;
    }
    const int64_t tmax = tk > tv ? tk : tv;
    const int m_cap = static_cast<int>(max_cta / BH);  // 0: more pairs than CTAs
    const bool one_tile_per_warp = m_cap >= 1 && tmax <= static_cast<int64_t>(NWARPS) * m_cap;
    for (int t = 0; t < NUM_ITEM_TIERS; ++t) {
      TierDev& d = P.tier[t];
      if (one_tile_per_warp) d.k_w = d.v_w = 1;
      d.k_w0 = static_cast<int>(wk);
      d.v_w0 = static_cast<int>(wv);
      wk += static_cast<int64_t>(d.k_tiles) * d.k_w;
      wv += static_cast<int64_t>(d.v_tiles) * d.v_w;
    }
    HQKV_REQUIRE(wk < (1ll << 27) && wv < (1ll << 27), "decode: cache too long");
    P.wk = static_cast<int>(wk);
    P.wv = static_cast<int>(wv);
    const int64_t wmax = wk > wv ? wk : wv;
    if (m_cap == 0) {
      P.g_m = 0;
      P.g_rem = 0;
      lay.grid = max_cta;
    } else {
      const int64_t m_want = ceil_div(wmax, static_cast<int64_t>(NWARPS) * (one_tile_per_warp ? 1 : 3));
      if (m_want <= m_cap) {
        P.g_m = static_cast<int>(m_want < 1 ? 1 : m_want);
        P.g_rem = 0;
      } else {
        P.g_m = m_cap;
        P.g_rem = static_cast<int>(max_cta - BH * m_cap);  // that many pairs get one CTA more
      }
      lay.grid = static_cast<int>(BH * P.g_m + P.g_rem);
    }
    for (int j = 0; j < 2; ++j) {
      const int m = P.g_m + j < 1 ? 1 : P.g_m + j;
      P.g_inv[j] = 1.0f / static_cast<float>(m);
      P.kq[j] = P.wk / m;
      P.kr[j] = P.wk % m;
      P.vq[j] = P.wv / m;
      P.vr[j] = P.wv % m;
    }
  }
  P.warp_smem = ws_bytes(rep8);
  P.cta_smem = cta_shared_bytes(rep8);
  lay.smem_bytes = P.cta_smem + NWARPS * P.warp_smem;
  lay.ctas_per_sm = ctas_per_sm;
  P.kc_max = static_cast<int>((ctas_per_sm * sm_count()) / BH) + 2;  // a group has at most max_cta / BH + 1 CTAs
  lay.acc_off = HQKV_WS_HEADER_BYTES;
  lay.logits_off = (lay.acc_off + static_cast<size_t>(BH) * P.rep * D * sizeof(double) + 255) & ~static_cast<size_t>(255);
  size_t off = lay.logits_off + static_cast<size_t>(c->B) * c->nh_q * L * sizeof(float);
  off = (off + 255) & ~static_cast<size_t>(255);
  lay.kpart_off = off;
  off += static_cast<size_t>(BH) * P.kc_max * MAX_REP * sizeof(float2);
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
                         long long mask_hstride = 0);
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
                               const void* probs_in, const void* mask, long long mask_bstride, long long mask_hstride) {
  HQKV_REQUIRE(phases >= 1 && phases <= 3, "decode: phases must be 1 (K ranges), 2 (V ranges) or 3 (both)");
  DecodeParams P;
  Layout lay;
  // a K-only call whose logits are the result, and a V-only call on given weights, look at one side only
  const int sides = probs_in ? 2 : ((phases == 1 && !attn_output) ? 1 : 3);
  int rc = build_params(cache_host, P, lay, sides);
  if (rc) return rc;
  P.phases = phases;
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
  HQKV_REQUIRE(!probs_in || phases == 2, "decode: given weights go with the V ranges alone");
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
  P.kdone = reinterpret_cast<unsigned*>(ws + WS_KDONE_OFF);
  P.vdone = reinterpret_cast<unsigned*>(ws + WS_VDONE_OFF);
  P.status = reinterpret_cast<unsigned*>(ws + WS_STATUS_OFF);
  P.logits = reinterpret_cast<float*>(ws + lay.logits_off);
  P.k_part = reinterpret_cast<float2*>(ws + lay.kpart_off);
  P.v_acc = reinterpret_cast<double*>(ws + lay.acc_off);
  P.spin_limit = 1ll << 22;  // x ~0.1 us per poll: about half a second
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    // opt in to >48 KB of dynamic shared memory once per device
    static bool attr_set[64] = {};
    int dev = 0;
    HQKV_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
      HQKV_CUDA(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     cta_shared_bytes(true) + NWARPS * ws_bytes(true)));
      // two CTAs per SM need nearly all of the SM's shared memory: ask for the largest carve-out
      HQKV_CUDA(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     static_cast<int>(cudaSharedmemCarveoutMaxShared)));
      if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
  }
  // programmatic stream serialisation: the grid may start while the kernel before it drains, if that
  // kernel allows it (the previous decode call does); everything it does before its
  // griddepcontrol.wait reads only the cache tiers
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(lay.grid);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = lay.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  HQKV_CUDA(cudaLaunchKernelEx(&cfg, decode_kernel, P));
  return HQKV_OK;
}

extern "C" int hqkv_decode_attention(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                     void* attn_output, void* workspace, size_t workspace_bytes, void* stream) {
  return hqkv_decode_attention_phases(cache_host, q, attn_weights, attn_output, workspace, workspace_bytes, 3, stream);
}

// ------------------------------------------------------------------------------------------------
// The two halves as operators of their own: raw logits of every tier, and the product of given weights with V
// ------------------------------------------------------------------------------------------------
namespace hqkv {
// fp32 logits of the scratch -> fp16 rows; the arrival counters of the K ranges go back to zero
__global__ void __launch_bounds__(256) logits_out_kernel(const float* logits, __half* out, int64_t n, unsigned* kdone, int bh) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = __float2half_rn(__ldcg(logits + i));
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i < bh; i += blockDim.x) kdone[i] = 0u;
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
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  const int64_t n = static_cast<int64_t>(P.B) * P.nh_q * P.L;
  const int blocks = static_cast<int>(n / 2048 > 592 ? 592 : (n / 2048 > 0 ? n / 2048 : 1));
  hqkv::logits_out_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float*>(ws + lay.logits_off), static_cast<__half*>(logits_f16), n,
      reinterpret_cast<unsigned*>(ws + WS_KDONE_OFF), P.B * P.H);
  HQKV_LAUNCH_CHECK("decode_logits");
  return HQKV_OK;
}

extern "C" int hqkv_decode_weighted_sum(const hqkv_cache_desc_t* cache_host, const void* weights_f16, void* out,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  HQKV_REQUIRE(weights_f16 && aligned(weights_f16, 2), "decode_weighted_sum: null or misaligned weights");
  {
    // no K ranges run in this call, so nobody clears the output accumulators: a stream-ordered memset does
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

extern "C" int hqkv_decode_attention_masked(const hqkv_cache_desc_t* cache_host, const void* q, const void* mask,
                                            int64_t mask_b_stride, int64_t mask_h_stride, void* attn_weights,
                                            void* attn_output, void* workspace, size_t workspace_bytes, void* stream) {
  HQKV_REQUIRE(mask != nullptr, "decode_masked: null mask");
  return decode_launch(cache_host, q, attn_weights, attn_output, workspace, workspace_bytes, 3, hqkv::PeerArgs(), stream,
                       nullptr, mask, mask_b_stride, mask_h_stride);
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

extern "C" int hqkv_decode_status(const void* workspace, void* stream, int* status_host) {
  HQKV_REQUIRE(workspace && status_host, "decode_status: null pointer");
  unsigned v = 0;
  HQKV_CUDA(cudaMemcpyAsync(&v, static_cast<const unsigned char*>(workspace) + WS_STATUS_OFF, sizeof(v),
                            cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  HQKV_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  *status_host = static_cast<int>(v);
  return HQKV_OK;
}

// ------------------------------------------------------------------------------------------------
// Decode attention for callers that may not allocate device memory
// ------------------------------------------------------------------------------------------------
// Some hosts of this library cannot obtain scratch at call time: a serving loop that has handed all
// of the GPU's memory to its own pool, a latency-critical loop whose rules forbid allocation after
// start-up (cudaMalloc may synchronise the device, and may fail late), or a binding whose language
// runtime owns no device allocator.  For them the scratch of the decode kernel lives in this
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
  // The array keeps whatever the previous call left.  Only the arrival counters and the status word have
  // to start at zero; a finished call leaves them zero, an aborted one might not, so they are cleared
  // every time (a stream-ordered memset, not an allocation).
  HQKV_CUDA(cudaMemsetAsync(scratch, 0, hqkv_decode_workspace_zero_bytes(cache_host), static_cast<cudaStream_t>(stream)));
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
// hqkv_decode_attention_gather_flagged makes the decode kernel store every pair of output values together
// with the call number as ONE 8-byte word into the peers' receive buffers: a word whose flag equals the
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
  for (int i = threadIdx.x; i < world * entries; i += blockDim.x) {
    const int r = i / entries;
    if (r == rank) continue;  // own rows were written in place by the decode kernel
    long long spins = 0;
    uint2 e;
    for (;;) {
      asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(e.x), "=r"(e.y) : "l"(recv + i));
      if (e.y == n) break;
      if (++spins > max_spins) {
        atomicExch(reinterpret_cast<int*>(state + 1), r + 1);  // gave up waiting for rank r
        break;
      }
      __nanosleep(20);
    }
    plain[i] = e.x;
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
