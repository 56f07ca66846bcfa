/*
 * hqkv.h — C ABI of libhqkv, the sm_100a implementation of the hybrid mixed-precision
 * KV-cache decode path (evict / tier-assign, group quantise + bit-pack, fused decode
 * attention over the packed tiers, residual flush).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - fp16 data is IEEE binary16 (`__half`), packed codes are int32 words with element i of a
 *     word at bits [i*bits, (i+1)*bits), index lists are int64;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and no entry
 *     point synchronises unless its comment says so;
 *   - every function returns 0 on success or a negative HQKV_E_* code; the text of the last
 *     failure on the calling thread is available from hqkv_last_error();
 *   - nothing here allocates device memory unless its comment says so: scratch is passed in.
 *
 * Each entry point names the interface of the reference project (skywclouds/HqeKV, paths
 * relative to its root) that it stands in for.
 */
#ifndef HQKV_H
#define HQKV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HQKV_OK 0
#define HQKV_E_INVALID (-1)     /* bad argument (shape, bits, group size, alignment, null pointer) */
#define HQKV_E_UNSUPPORTED (-2) /* valid in the reference but not built here (e.g. Gaussian codebooks above 1 bit) */
#define HQKV_E_WORKSPACE (-3)   /* scratch buffer too small */
#define HQKV_E_CUDA (-4)        /* a CUDA runtime call failed */

/* Text of the last error raised on this thread ("" if none). Never NULL. */
const char* hqkv_last_error(void);

/* Library version: major*10000 + minor*100 + patch. */
int hqkv_version(void);

/* Which sources this binary was compiled from: the first 16 hex digits of the SHA-256 over the library's
 * source files (csrc, sorted by name) and this header, stamped at build time by hqekv_b200/build.py
 * ("unstamped" for a build made another way).  A host compares it with the hash of the sources it has. */
const char* hqkv_build_id(void);

/*
 * Bounds-check build.  A library compiled with -DHQKV_CHECKS (python -m hqekv_b200.build --checks writes
 * libhqkv_checked.so) range-checks every index it takes out of a caller-supplied list - the logical positions in
 * the tiers' index lists, the token ids of the flush plan - before it addresses memory with it; a violation is
 * counted and the access skipped, nothing traps.  hqkv_checks_enabled() tells which build is loaded;
 * hqkv_check_failures() synchronises the device and reports (optionally clears) the count, always 0 in the
 * regular build.  No counterpart in the reference (its kernels check nothing).
 */
int hqkv_checks_enabled(void);
int hqkv_check_failures(int reset, unsigned* count_host);

/* ---------------------------------------------------------------------------------------------
 * Codec
 * ------------------------------------------------------------------------------------------- */

/*
 * Asymmetric uniform group quantisation + bit-packing along the LAST logical axis of a
 * [rows, T] fp16 matrix.  Stands in for uniform_group_quantize_pack_last_dim
 * (quant/pack_unpack.py:156-193) together with the Triton kernel _pack_along_last_dim
 * (quant/pack_unpack.py:16-51).  Arithmetic: fp16 with a rounding after every step, exactly
 * as the torch op sequence there (min, max, sub, div, sub_, div_, clamp_, round_).
 *
 * The source element (row, t) lives at  x[(row / inner) * outer_stride + (row % inner) * inner_stride + t * t_stride]
 * (strides in elements).  Two access patterns are built:
 *   t_stride == 1                      rows contiguous along T (V: one row per token, T = head_dim);
 *   inner_stride == 1, t_stride >= inner  K: token-major source [outer, T, inner] read as [outer*inner, T]
 *                                       (the transposed view the reference quantises, without materialising it).
 * Outputs are dense: code int32 [rows, T*bits/32], scale and mn fp16 [rows, T/group].
 * bits in {8,4,2,1}; group in {32,64,128}; T a multiple of group.
 * The source is NOT modified (the reference overwrites it with intermediate values).
 */
int hqkv_quantize_pack(const void* x, int64_t rows, int64_t T, int64_t inner, int64_t outer_stride,
                       int64_t inner_stride, int64_t t_stride, int group, int bits, void* code, void* scale,
                       void* mn, void* stream);

/*
 * Inverse: unpack + dequantise, x = half(half(code * scale) + mn)   (two fp16 roundings).
 * Stands in for uniform_group_dequantize_unpack_last_dim (quant/pack_unpack.py:316-333) and the
 * Triton kernel _unpack_along_last_dim (:255-278).  code int32 [rows, T*bits/32] dense,
 * scale/mn fp16 [rows, T/group] dense, out fp16 [rows, T] dense.
 */
int hqkv_dequantize_unpack(const void* code, const void* scale, const void* mn, int64_t rows, int64_t T, int group,
                           int bits, void* out, void* stream);

/*
 * Gaussian-codebook codec at 1 bit: the quantiser of the 1-bit tier under quant_strategy
 * 'high_uniform_group_low_normal_group'.  Stands in for normal_group_quantize_pack_last_dim /
 * normal_group_dequantize_unpack_last_dim with bit = 1 (quant/pack_unpack.py:218-253, 356-376).
 * std / mean = unbiased torch.std_mean of each group (fp16); code = ((x - mean) / std > 0) with fp16
 * roundings after the subtract and the divide; x^ = half(half(c * std) + mean), c = +-fp16(0.67448974).
 * Same source addressing and output layout as hqkv_quantize_pack with bits = 1.
 */
int hqkv_normal1_quantize_pack(const void* x, int64_t rows, int64_t T, int64_t inner, int64_t outer_stride,
                               int64_t inner_stride, int64_t t_stride, int group, void* code, void* std_out,
                               void* mean_out, void* stream);
int hqkv_normal1_dequantize_unpack(const void* code, const void* std_in, const void* mean_in, int64_t rows, int64_t T,
                                   int group, void* out, void* stream);

/* pack_along_last_dim (quant/pack_unpack.py:53-70): int32 codes [rows, T] -> int32 words [rows, T*bits/32]. */
int hqkv_pack(const void* codes_i32, int64_t rows, int64_t T, int bits, void* words, void* stream);

/* unpack_along_last_dim (quant/pack_unpack.py:281-297): int32 words [rows, W] -> fp16 integers [rows, W*32/bits]. */
int hqkv_unpack(const void* words, int64_t rows, int64_t W, int bits, void* out_f16, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Decode attention over the tiered cache
 * ------------------------------------------------------------------------------------------- */

#define HQKV_NUM_TIERS 5 /* 16-, 8-, 4-, 2-, 1-bit, in the slot order of the reference's cache tuple */
#define HQKV_CODEC_UNIFORM 0 /* code * scale + zero (min/max groups) */
#define HQKV_CODEC_NORMAL 1  /* 1-bit tier only: center[code] * std + mean with the centres -+0.67448974, the
                                low tier of quant_strategy 'high_uniform_group_low_normal_group'
                                (quant/hqe_2.py:488-492, quant/pack_unpack.py:6-14, 218-253); the scale slots then
                                hold std and the zero slots hold mean */
#define HQKV_MAX_PEERS 7 /* other GPUs a kv-head-sharded decode can write its output rows to */

/* One precision tier of the cache (slots 0-35 of the 42-entry tuple, quant/hqe_matmul.py:364-368). */
typedef struct {
  int32_t bits; /* 16, 8, 4, 2 or 1 */
  int32_t n_k;  /* tokens held on the K side (0 = tier absent) */
  int32_t n_v;  /* tokens held on the V side */
  int32_t codec; /* HQKV_CODEC_UNIFORM, or HQKV_CODEC_NORMAL (bits == 1 only) */
  const void* k_data;   /* bits<16: int32 [B,H,D,n_k*bits/32]; bits==16: fp16 [B,H,D,n_k]  (channel-major) */
  const void* k_scale;  /* fp16 [B,H,D,n_k/group_k]   (NULL when bits==16) */
  const void* k_zero;   /* fp16 [B,H,D,n_k/group_k] */
  const int64_t* k_idx; /* [n_k] logical position of every K token */
  const void* v_data;   /* bits<16: int32 [B,H,n_v,D*bits/32]; bits==16: fp16 [B,H,n_v,D]  (token-major) */
  const void* v_scale;  /* fp16 [B,H,n_v,D/group_v] */
  const void* v_zero;   /* fp16 [B,H,n_v,D/group_v] */
  const int64_t* v_idx; /* [n_v] logical position of every V token */
} hqkv_tier_t;

typedef struct {
  int32_t B;        /* batch */
  int32_t H;        /* kv heads */
  int32_t nh_q;     /* query heads, a multiple of H with nh_q/H <= 8 */
  int32_t D;        /* head dim, must be 128 */
  int32_t group_k;  /* tokens per K group (the reference passes block_size): 32, 64 or 128 */
  int32_t group_v;  /* channels per V group: 32, 64 or 128 */
  int32_t n_new;    /* tokens in the fp16 residual window (may be 0) */
  float softmax_scale; /* multiplies q.k before the softmax: 1/sqrt(head_dim) */
  const void* new_k;   /* fp16 [B,H,n_new,D] token-major; logical positions are the last n_new */
  const void* new_v;   /* fp16 [B,H,n_new,D] */
  hqkv_tier_t tier[HQKV_NUM_TIERS];
} hqkv_cache_desc_t;

/* Bytes of scratch hqkv_decode_attention needs for this cache on the current device (0 on invalid input). */
size_t hqkv_decode_workspace_bytes(const hqkv_cache_desc_t* cache_host);
/* Leading part of that scratch (arrival counters) that must be zero before a call:
 * HQKV_WS_HEADER_BYTES whatever the cache; 0 on invalid input. */
size_t hqkv_decode_workspace_zero_bytes(const hqkv_cache_desc_t* cache_host);

/*
 * One decode step of attention over the whole tiered cache: q.K^T for every tier with the
 * packed codes dequantised in registers, softmax in fp32, p.V for every tier, plus the fp16
 * residual window and the fp16 tier.  Two launches chained by programmatic dependent launch: the K pass
 * (logits of every cached token at its logical position, one softmax pair per CTA) and the V pass (folds the
 * pairs, writes the probabilities, accumulates p.V; the last CTA of a (batch, kv head) normalises and
 * writes).  Stands in for qkv_matmul_hqe_2
 * (quant/hqe_matmul.py:354-451) and everything below it: the layout glue of
 * cuda_bmm_fA_qB_uniform_group (quant/matmul.py:263-299), gemv_forward_cuda_uniform_group and
 * bgemv_kernel_uniform_group_{8,4,2} (quant/csrc/gemv_cuda_uniform.cu:1533-1599, 411-733), the
 * torch.matmul calls on the fp16 tier and the residual, and the softmax block (:430-433).
 *
 *   q            fp16 [B, nh_q, 1, D]
 *   attn_weights fp16 [B, nh_q, 1, L]   L = sum_t n_k + n_new; normalised probabilities at logical positions
 *   attn_output  fp16 [B, nh_q, 1, D]
 *   workspace    at least hqkv_decode_workspace_bytes() bytes, 256-byte aligned.  Zero its first
 *                HQKV_WS_HEADER_BYTES bytes once after allocating it: they hold the arrival counters of the V
 *                pass, and every call that completes leaves them zero again, so one workspace
 *                serves calls on caches of any shape.  Calls that share a workspace must be ordered on
 *                one stream.
 * The K-side and V-side token counts of a tier may differ only in order, not in total
 * (sum n_k == sum n_v).  A 1-bit tier is read in the codec its `codec` field names.
 *
 * Ordering contract for callers that chain kernels with programmatic dependent launch: both kernels
 * read the cache tiers (codes, scales, zeros, index lists) BEFORE they wait for the kernels ahead of them
 * in the stream; q, the residual window and the scratch are read after that wait.  A kernel
 * that writes a tier must therefore have completed (not merely have triggered its dependents) before
 * a decode call on the same stream is launched; an ordinary launch always satisfies this.
 * Neither kernel waits on another CTA, so the call makes no demand on how many CTAs are resident.
 */
#define HQKV_WS_HEADER_BYTES 12288
int hqkv_decode_attention(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights, void* attn_output,
                          void* workspace, size_t workspace_bytes, void* stream);

/*
 * hqkv_decode_attention with an additive mask on the logits (after the softmax scale, before the softmax):
 * element (b, head, pos) of the mask is mask[b * mask_b_stride + head * mask_h_stride + pos] (fp16; a stride
 * of 0 broadcasts; -inf removes a position).  Stands in for ``attn_weights += attention_mask`` of the
 * no-eviction flavour (quant/quant_matmul_hq.py:101, :164).
 */
int hqkv_decode_attention_masked(const hqkv_cache_desc_t* cache_host, const void* q, const void* mask,
                                 int64_t mask_b_stride, int64_t mask_h_stride, void* attn_weights, void* attn_output,
                                 void* workspace, size_t workspace_bytes, void* stream);

/*
 * hqkv_decode_attention that also writes the importance row of the step: head_sum_row[pos] (fp16 [L]) =
 * attn_weights.sum(0).sum(0) with the roundings of fp16 tensors (fp32 accumulation over the batch, one fp16
 * rounding, fp32 accumulation over the heads in head order, one fp16 rounding) - bit-identical to hqkv_head_sum
 * on the probabilities.  Stands in for last_attn_weights.update on a decode step
 * (model/public_func.py:243-257; called at model/llama_hqe.py:199-200).  Up to B * nh_q = 64 and nh_q = 32 the V
 * pass emits the row itself (the last CTA to finish a chunk of tokens adds the probabilities the others have just
 * written); beyond that the call adds one hqkv_head_sum launch.  One launch less than hqkv_decode_attention +
 * hqkv_head_sum, but at batch 1 and 32 k context the pair is the faster of the two (26 against 37 us per layer on
 * a B200): a chunk's gathers run on one CTA here and over the whole GPU there.
 */
int hqkv_decode_attention_headsum(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                  void* attn_output, void* head_sum_row, void* workspace, size_t workspace_bytes,
                                  void* stream);

/*
 * The same call restricted to one of its launches: phases = 1 runs the K pass only (logits and
 * per-CTA softmax statistics into the workspace), 2 the V pass only (needs the workspace a K-only
 * call of the same cache left), 3 both.  Serves
 * cuda_bmm_forward_qk_group_hq / cuda_bmm_forward_wv_group_hq style callers and the timing of the two
 * halves; the split itself has no counterpart in the reference.
 */
int hqkv_decode_attention_phases(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                 void* attn_output, void* workspace, size_t workspace_bytes, int phases, void* stream);

/*
 * The K half as an operator of its own: out[b, h, 0, pos] = fp16(softmax_scale * q_h . K^_pos) for every cached
 * token at its logical position, all tiers and the residual window in one K pass plus a conversion of the
 * scratch row to fp16 (pass softmax_scale = 1 for the raw product).  Stands in for cuda_bmm_forward_qk_group_hq (quant/matmul.py:351-434) =
 * kvhq_gemv.gemv_forward_cuda_qk_group_hq (quant/csrc/gemv_cuda.h:78-109), and with identity index lists for
 * the _seq forms (quant/matmul.py:436-505, gemv_cuda.h:111-137).  logits_f16: fp16 [B, nh_q, 1, L].  Workspace as for
 * hqkv_decode_attention; the call leaves it ready for any other call.
 */
int hqkv_decode_logits(const hqkv_cache_desc_t* cache_host, const void* q, void* logits_f16, void* workspace,
                       size_t workspace_bytes, void* stream);

/*
 * The V half as an operator of its own: out[b, h, 0, :] = sum_pos w[b, h, 0, pos] * V^_pos over every tier and
 * the residual window, for caller-supplied weights w (fp16 [B, nh_q, 1, L], indexed by logical position).  Stands
 * in for cuda_bmm_forward_wv_group_hq (quant/matmul.py:507-579) = kvhq_gemv.gemv_forward_cuda_wv_group_hq
 * (quant/csrc/gemv_cuda.h:139-170) and the _seq forms (quant/matmul.py:581-649, gemv_cuda.h:172-198).
 * out: fp16 [B, nh_q, 1, D].
 */
int hqkv_decode_weighted_sum(const hqkv_cache_desc_t* cache_host, const void* weights_f16, void* out, void* workspace,
                             size_t workspace_bytes, void* stream);

/*
 * kv-head sharding over the GPUs of one node (one process per GPU; reference: none - the reference is
 * single-GPU; the head split follows its per-(batch*head) kernel indexing, quant/csrc/gemv_cuda_uniform.cu:415-428).
 * hqkv_decode_attention_gather is hqkv_decode_attention whose last step also stores this GPU's output
 * rows [B, nh_q_local, 1, D] into n_peers other GPUs' memory (peer_outputs_host[p] = where THIS rank's
 * block starts inside peer p's gathered buffer; peer-accessible device pointers, e.g. CUDA IPC or
 * torch symmetric memory).  The stores are plain NVLink writes.  With peer_pads_host != NULL the CTA
 * that finishes this GPU's last (batch, kv head) then runs a cross-GPU barrier before the kernel ends,
 * so that once the call has completed on a rank, every rank's rows are in that rank's gathered buffer;
 * with NULL the caller orders the GPUs itself (hqkv_peer_barrier, or any collective).
 *
 * Barrier arguments: peer_pads_host[r] = rank r's signal pad (>= 4*world bytes, zero before the first
 * call, written by the peers); state = 12 bytes of this GPU's memory, zero before the first call (call
 * number, status, finished-head count).  Waits are bounded by max_spins polls per peer; when a peer
 * does not arrive the kernel stores (peer + 1) in the status word (state + 4) and returns - no trap,
 * no endless loop.  hqkv_peer_barrier is the same barrier as a kernel of its own (state: 8 bytes).
 */
int hqkv_decode_attention_gather(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                 void* attn_output, void* workspace, size_t workspace_bytes,
                                 void* const* peer_outputs_host, int n_peers, void* const* peer_pads_host, int rank,
                                 int world, void* state, long long max_spins, void* stream);
int hqkv_peer_barrier(void* const* peer_pads_host, int rank, int world, void* state, long long max_spins, void* stream);

/*
 * Low-latency form of the same exchange (no counterpart in the reference).  The decode kernel stores each
 * pair of output values together with the call number as one 8-byte word into the peers' RECEIVE
 * buffers (peer_recv_host[p] = where THIS rank's entries start in peer p's receive buffer of
 * world * entries_per_rank 8-byte words, zero before the first call); hqkv_peer_unpack, enqueued by every
 * rank right after, polls its own receive buffer until every word carries the current call number
 * (bounded by max_spins per word; a missing rank is recorded as rank + 1 in the status word at
 * state + 4), writes the values into the plain gathered buffer [world][entries_per_rank] of fp16 pairs
 * and advances the call number at state + 0.  entries_per_rank = B * nh_q_local * D / 2.  A receive buffer
 * may be reused only after every peer has unpacked it: rotate at least two.  state: 8 bytes of this
 * GPU's memory, zero before the first call, shared by the two functions.
 */
int hqkv_decode_attention_gather_flagged(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                         void* attn_output, void* workspace, size_t workspace_bytes,
                                         void* const* peer_recv_host, int n_peers, void* state, void* stream);
int hqkv_peer_unpack(const void* recv, void* gathered, int rank, int world, int entries_per_rank, void* state,
                     long long max_spins, void* stream);

/*
 * hqkv_decode_attention for callers that cannot allocate device memory.  It has no counterpart in the
 * reference, whose wrappers allocate freely through torch.
 *
 * Who needs it: a host that has given the whole GPU to its own memory pool, a latency-critical loop
 * that may not allocate after start-up (cudaMalloc can synchronise the device and can fail late), or a
 * language binding with no device allocator of its own.  Inputs and outputs are still the caller's; only the scratch of the
 * decode kernel comes from a fixed array of HQKV_STATIC_SCRATCH_BYTES inside the library, resident on
 * every GPU that loads it for the life of the process.  The call allocates and frees nothing.
 *
 *  - Limit: caches whose hqkv_decode_workspace_bytes() exceeds HQKV_STATIC_SCRATCH_BYTES are refused
 *    with HQKV_E_WORKSPACE (16 MiB covers batch 1 up to ~100k cached tokens with 32 query heads; the
 *    need grows with B * nh_q * L * 4 bytes).
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress with
 *    that device current).  Make that first call outside any stream capture, and make it at start-up,
 *    before the host's own pool takes the remaining memory: with CUDA's lazy module loading that call
 *    may be the one that loads the library's module onto the device, which is when the array itself
 *    is placed (CUDA_MODULE_LOADING=EAGER moves that to context creation).
 *  - All calls on a device share the one array, which keeps the previous call's contents (the
 *    arrival counters are cleared by a stream-ordered
 *    memset at the start of every call; that memset sits between the previous kernel and this one, so
 *    this entry point gives up the overlap of consecutive decode kernels that the regular one has).
 *    Two calls that overlap on the GPU, e.g. on different streams, race on it: order them on one
 *    stream or with events.
 */
#define HQKV_STATIC_SCRATCH_BYTES (16u << 20)
size_t hqkv_decode_static_scratch_bytes(void);
int hqkv_decode_attention_static(const hqkv_cache_desc_t* cache_host, const void* q, void* attn_weights,
                                 void* attn_output, void* stream);

/*
 * Batched GEMV  C = fA x dequant(qB)  with the reference's un-transposed operand layout, fp32
 * accumulation, fp16 result.  Stands in for cuda_bmm_fA_qB_uniform_group (quant/matmul.py:263-299)
 * = transposes + kvhq_gemv.gemv_forward_cuda_uniform_group (quant/csrc/pybind.cpp:11,
 * quant/csrc/gemv_cuda_uniform.cu:1533-1599), without the transposed copies.
 *   fA fp16 [B, nh_q, 1, K];  qB int32 [B, nh_kv, K, N*bits/32];  scales/zeros fp16 [B, nh_kv, K, N/group]
 *   out fp16 [B, nh_q, 1, N].   bits in {8,4,2,1}; group in {32,64,128}; N a multiple of group.
 * Both uses of the reference are covered: K = head_dim, N = tokens (q.K^T of one tier) and
 * K = tokens, N = head_dim (p.V of one tier).
 */
int hqkv_gemv_uniform_group(const void* fA, const void* qB, const void* scales, const void* zeros, int B, int nh_q,
                            int nh_kv, int64_t K, int64_t N, int group, int bits, void* out, void* stream);
/* The same over a Gaussian-codebook tier: value = std * (code ? C : -C) + mean, C = 0.67448974 in float32.
 * Stands in for cuda_bmm_fA_qB_normal_group (quant/matmul.py:72-95) = transposes +
 * kvhq_gemv.gemv_forward_cuda_normalize_group (quant/csrc/gemv_cuda_normal.cu) at bits = 1, the width the
 * live strategy 'high_uniform_group_low_normal_group' uses; other widths return HQKV_E_INVALID. */
int hqkv_gemv_normal_group(const void* fA, const void* qB, const void* stds, const void* means, int B, int nh_q,
                           int nh_kv, int64_t K, int64_t N, int group, int bits, void* out, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Importance bookkeeping and block ranking
 * ------------------------------------------------------------------------------------------- */

/*
 * Row the importance ring stores for one query row: out[l] = half(sum_h half(sum_b w[b,h,l])),
 * fp32 accumulation in index order.  Stands in for ``attn_weights.sum(0).sum(0)`` in
 * last_attn_weights.update (model/public_func.py:243-257).  Row (b,h) of w starts at
 * w + (b*nh + h)*bh_stride (elements) and holds L fp16 values; out fp16 [L].  For a decode step
 * (w dense [B, nh, 1, L]) bh_stride = L; for one row r of a prefill block [B, nh, q_len, L] pass
 * w + r*L and bh_stride = q_len*L.
 */
int hqkv_head_sum(const void* w, int B, int nh, int64_t L, int64_t bh_stride, void* out, void* stream);

/*
 * importance[l] = half( half(sum_r ring[r,l]) / min(last_len, L - l) ) — calculate_token_importance
 * (model/public_func.py:217-221).  ring fp16 [rows, ring_stride]; out fp16 [L].
 */
int hqkv_token_importance(const void* ring, int rows, int64_t ring_stride, int64_t L, void* out, void* stream);

/*
 * Per-token value range summed over batch and heads: calculate_token_range (model/public_func.py:58-73).
 * v fp16 [B, H, T, D] with token stride D and the given batch/head strides (elements); out fp16 [T].
 */
int hqkv_token_range(const void* v, int B, int H, int64_t T, int D, int64_t b_stride, int64_t h_stride, void* out,
                     void* stream);

/*
 * Block ranking: get_block_token_idx (model/public_func.py:92-106).  Divides importance[0 .. nblocks*block)
 * by `block` IN PLACE (as the reference does to its argument), forms each block's fp16 key, orders blocks by
 * descending key with ties broken by ascending block id, and writes the expanded int64 token ids.
 * If range_or_null is given, importance is first multiplied by it elementwise in fp16 into `importance`
 * (the V-side key of quant/hqe_2.py:515).  nblocks <= 8192.
 */
int hqkv_block_rank(void* importance, const void* range_or_null, int block, int nblocks, int64_t* sorted_ids,
                    void* stream);

/* ---------------------------------------------------------------------------------------------
 * Flush: evict + tier-assign + re-quantise  (KV_cache_hqe_2, quant/hqe_2.py:456-843)
 * ------------------------------------------------------------------------------------------- */

/*
 * Phase 1 — plan one side (K or V) of a flush on the device.
 *
 * Inputs: the id list of every tier (tier_idx[t], length tier_n[t], NULL if empty), the ranked ids
 * (sorted_ids, hist+compress entries) and the six cumulative tier counts (cum_counts_host: 16,8,4,2,1-bit,
 * evict).  A token moves only to a tier of strictly fewer bits than it has now; residual tokens always take
 * their target (the ladder of quant/hqe_2.py:584-659 / :737-825).
 *
 * Outputs (device, sized for total = hist+compress tokens):
 *   plan_src   int32 [5][total]   for destination tier t, entry j: source of the j-th token, encoded as
 *                                 (source_tier+1)<<28 | position in that source (source_tier -1 = residual)
 *   plan_ids   int64 [5][total]   final idx list of every tier (already re-ranked if anything was evicted)
 *   survivors  int64 [total]      ascending ids of the tokens that are not evicted
 *   counts     int32 [8]          final size of the five tiers, number of survivors, 1 if any token was
 *                                 evicted else 0, 0
 * The caller reads `counts` back (one small copy) to size the new tier tensors.
 */
int hqkv_flush_plan(const int64_t* const* tier_idx_host, const int32_t* tier_n_host, int64_t hist, int64_t compress,
                    const int64_t* sorted_ids, const int64_t* cum_counts_host, int32_t* plan_src, int64_t* plan_ids,
                    int64_t* survivors, int32_t* counts, void* workspace, size_t workspace_bytes, void* stream);
size_t hqkv_flush_plan_workspace_bytes(int64_t total);

/* Source tensors of one side for phase 2 (same layouts as hqkv_tier_t; index 0..4 = 16,8,4,2,1-bit). */
typedef struct {
  const void* data[HQKV_NUM_TIERS];
  const void* scale[HQKV_NUM_TIERS];
  const void* zero[HQKV_NUM_TIERS];
  int32_t n[HQKV_NUM_TIERS];
  int32_t low_codec; /* codec the 1-bit DESTINATION tier is written in (and its kept blocks already are):
                        HQKV_CODEC_UNIFORM or HQKV_CODEC_NORMAL; the other tiers are always uniform */
  const void* residual; /* fp16 [B,H,r,D] token-major, first `compress` tokens are flushed */
  int64_t residual_b_stride, residual_h_stride; /* elements */
} hqkv_flush_src_t;

/*
 * Phase 2 — build destination tier `dst_tier` of the K side from the plan: kept blocks are copied,
 * arrivals are dequantised (two-rounding recipe) if they were quantised, then re-quantised at the
 * destination width in groups of `group` tokens per channel (K_high_2_low / quant_new_K,
 * quant/hqe_2.py:16-42, 88-130).  n_dst = counts[dst_tier] from phase 1; outputs dense
 * [B,H,D,n_dst*bits/32] / [B,H,D,n_dst/group] (fp16 [B,H,D,n_dst] for the 16-bit tier).
 */
int hqkv_flush_build_k(const hqkv_flush_src_t* src_host, int B, int H, int D, int group, int dst_tier,
                       const int32_t* plan_src_row, int64_t n_dst, void* out_data, void* out_scale, void* out_zero,
                       void* stream);
/* Same for the V side, groups of `group` channels per token (V_high_2_low, quant/hqe_2.py:132-170). */
int hqkv_flush_build_v(const hqkv_flush_src_t* src_host, int B, int H, int D, int group, int dst_tier,
                       const int32_t* plan_src_row, int64_t n_dst, void* out_data, void* out_scale, void* out_zero,
                       void* stream);

/* out[r, j] = in[r, ids[j]] for fp16 rows — compaction of V_token_norm and of the importance ring to the
 * survivors (quant/hqe_2.py:733-735, last_attn_weights.eviction model/public_func.py:228-231).
 * in/out may not overlap. */
int hqkv_gather_columns_f16(const void* in, int64_t in_stride, int rows, const int64_t* ids, int64_t n, void* out,
                            int64_t out_stride, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HQKV_H */
