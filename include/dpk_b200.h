/*
 * dpk_b200 -- C ABI of the B200 (sm_100a) routed dynamic-width operators.
 *
 * This is the native boundary a host binding calls in place of the reference's
 * TVM-FFI `Host::run(TensorView...)` functions.  Every entry point takes raw
 * device pointers, sizes, element strides and a CUDA stream, launches on that
 * stream without synchronising, allocates nothing and keeps no state besides
 * cached device properties -- with one exception: dpk_peer_alloc / dpk_peer_free
 * (tensor-parallel set-up, not on any per-step path) allocate and release the
 * device buffer that peers map through CUDA IPC.  All return 0 on success or one
 * of the DPK_ERR_* codes; dpk_last_error() then holds a message (thread local).
 *
 * Conventions
 *   - "half" tensors are fp16 or bf16 as selected by `dtype` (DPK_F16 / DPK_BF16),
 *     row-major, innermost dimension contiguous, 16-byte aligned rows.
 *   - M = B*T flattened tokens, NG = routed groups, G = group width.
 *   - masks are one byte per element, non-zero = active (a torch.bool tensor).
 *   - `stream` is a cudaStream_t passed as void*.
 *   - workspaces are caller-owned device buffers; their sizes come from the
 *     dpk_*_workspace_bytes() helpers.
 */
#ifndef DPK_B200_H_
#define DPK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DPK_OK 0
#define DPK_ERR_INVALID 1     /* bad argument: shape, stride, alignment, dtype  */
#define DPK_ERR_CUDA 2        /* a CUDA runtime / driver call failed              */
#define DPK_ERR_UNSUPPORTED 3 /* valid request this build has no kernel for       */
#define DPK_ERR_DEVICE 4      /* a kernel reported a problem in its status word   */

#define DPK_F16 0
#define DPK_BF16 1

#define DPK_ACT_IDENTITY 0
#define DPK_ACT_RELU 1
#define DPK_ACT_SILU 2

/* Library version (major*100 + minor). */
int dpk_version(void);

/*
 * The persistent GEMM kernels launch one CTA per SM.  A caller that runs a collective
 * (NCCL) concurrently with them can leave `sms` SMs free for it; 0 restores the default.
 * Process-wide setting, not thread safe against concurrent launches.  No counterpart in
 * the reference, which has no collective in its kernel library.
 */
int dpk_set_sm_margin(int sms);

/* Message of the last failing call made by this thread ("" if none). */
const char* dpk_last_error(void);

/*
 * Reads (and clears) the status word kernels write when a bounded wait ran out or a
 * routing index was out of range.  Synchronises `stream`.  *status == 0 means fine.
 * Otherwise *status = 1000 * kernel + code: code 101/102 a pipeline stage was never
 * filled / drained, 103/104 the same for an accumulator in tensor memory, 105 a routing
 * index outside the token range, 106 misaligned shared memory; kernel 1 gemm_mn, 2 gemm_mn
 * on CTA pairs, 3 gemm_k, 4 gemm_k on CTA pairs, 5 prefill attention, 6 decode attention,
 * 7 routing, 9 router + norm, 11 small-M FFN.  The first report wins until it is read.
 * The reference's device code has no counterpart: its waits are unbounded
 * (DynamicPruningKernels/include/attention_prefill/v3/sm12x_causal.cuh:401,535).
 */
int dpk_device_status(int* status, void* stream);

/* ------------------------------------------------------------------ routing ---- */

/*
 * Per-token top-k over fp32 router logits [M,NG] -> byte mask [M,NG]; ties go to the
 * lower group index.  The reference ships no top-k router (its kernels consume a
 * ready Boolean mask, DynamicPruningKernels/README.md:35; WIDE's evaluation routing is
 * a 2-way argmax, WIDE/wrapper/base_layer.py:204-207); this is the benchmark's way of
 * producing a mask with an exact keep count.
 */
int dpk_topk_mask(const float* logits, int64_t M, int NG, int keep, uint8_t* mask, void* stream);

/* Bytes of scratch dpk_route_compact needs for an [M,NG] mask. */
size_t dpk_route_workspace_bytes(int batches, int64_t M, int NG);

/*
 * Routing layout.  Replaces the reference hosts'
 *   torch.sort(Mask.flatten(0,1), dim=0, descending=True, stable=False)
 * (DynamicPruningKernels/python/gemm_mn/jit.py:410-415, gemm_k/jit.py:396-401) with
 * batches = 1, M = B*T, and the per-batch sort of prefill attention
 *   torch.sort(Mask, dim=1, descending=True, stable=False)
 * (attention_prefill/jit.py:259-263) with batches = B, M = Tq (indices then count
 * from 0 inside each batch, as the reference's do).
 *   mask            [batches,M,NG] bytes
 *   sorted_mask     [batches,M,NG] bytes: row r of column g is 1 iff r < counts[b,g]
 *   sorted_indices  [batches,M,NG] int64: column g lists the active rows ascending,
 *                   then the inactive rows ascending (the stable order)
 *   counts          [batches,NG] int32 active rows per group
 */
int dpk_route_compact(const uint8_t* mask, int batches, int64_t M, int NG, uint8_t* sorted_mask,
                      int64_t* sorted_indices, int32_t* counts, void* workspace,
                      size_t workspace_bytes, void* stream);

/*
 * Same result as dpk_route_compact, for callers that have no way to provide scratch
 * memory: code that runs where device allocation is off limits (inside a serving loop
 * whose memory pool is fixed up front, a plugin whose host only lends it the input and
 * output buffers, a latency path that must not touch the allocator).  The counters the
 * three kernels exchange live in a 256 KiB array built into the library image, which
 * every GPU that loads the library holds until the process exits.  This entry point has
 * no counterpart in the reference, whose hosts allocate their temporaries through
 * PyTorch on every call.
 *   - Limit: batches * ceil(M/256) * NG <= 65536 counters (256 KiB); larger problems
 *     are refused with DPK_ERR_INVALID and a message naming the limit.
 *   - The first call on each device looks up the array's device address (with that
 *     device current) and remembers it; make that first call outside any stream capture.
 *   - It calls no allocating routine: no cudaMalloc / cudaFree, nothing from a tensor
 *     library.
 *   - All calls on a device share the one array, which keeps whatever the previous call
 *     left; each call overwrites every counter it later reads, so nothing needs
 *     clearing.  Two calls whose kernels overlap on the GPU (different streams, or
 *     different host threads) race on it: serialise them or use dpk_route_compact.
 */
int dpk_route_compact_static(const uint8_t* mask, int batches, int64_t M, int NG,
                             uint8_t* sorted_mask, int64_t* sorted_indices, int32_t* counts,
                             void* stream);

/*
 * counts[b,g] = number of leading non-zero entries of column g of sorted_mask
 * [batches,M,NG] (every active row of a column precedes every inactive one).  Used
 * when the caller passes `sorted_mask` / `sorted_indices` from an earlier call
 * (metadata reuse, DynamicPruningKernels/tests/test_gpu_smoke.py:203-292).
 */
int dpk_route_counts(const uint8_t* sorted_mask, int batches, int64_t M, int NG, int32_t* counts,
                     void* stream);

/*
 * Packed routing bits for the reduction-width GEMM: row_bits [M, ceil(NG/32)] uint32
 * (bit g%32 of word g/32 = mask[r,g] != 0) and win_bits [ceil(M/128), ceil(NG/32)]
 * (OR over each 128-row window).  Plays the role of the reference kernel's per-tile
 * skip metadata (DynamicPruningKernels/include/gemm_k/v1/sm12x.cuh:258-358, 525).
 */
int dpk_mask_pack(const uint8_t* mask, int64_t M, int NG, uint32_t* row_bits, uint32_t* win_bits,
                  void* stream);

/*
 * dpk_route_compact (batches = 1) and dpk_mask_pack in one pass over the mask: everything
 * the fused FFN needs from the routing decision, in three launches.  Same outputs, same
 * workspace as dpk_route_compact.
 */
int dpk_route_plan(const uint8_t* mask, int64_t M, int NG, uint8_t* sorted_mask,
                   int64_t* sorted_indices, int32_t* counts, uint32_t* row_bits, uint32_t* win_bits,
                   void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------ routed GEMMs ---- */

/*
 * Output-width routed projection (reference: GEMM_MN_V1_Host::run,
 * DynamicPruningKernels/include/gemm_mn/v1/sm12x.cuh:766-860; host wrapper
 * python/gemm_mn/jit.py:357-440).
 *   D[t, g*G + j] = act( sum_k A[t,k] * W[g*G + j, k] )      for active (t,g)
 * Rows of inactive (t,g) blocks are not written: pass D zero-filled, as the reference
 * host does (jit.py:381).
 *   A [M,K] lda, W [N,K] ldw, D [M,N] ldd   (strides in elements)
 *   W2: optional second weight [N,K] (same ldw).  When non-NULL the kernel computes the
 *       SwiGLU combination D = silu(A W^T) * (A W2^T) in one pass (`act` ignored);
 *       this fuses the reference callers' gate GEMM, up GEMM and multiply
 *       (PruningInferSim/ops/mlp/m_pruning.py:76-105).
 *   sorted_indices [M,NG] int64 and counts [NG] int32 from dpk_route_compact.
 * Requirements: K % 8 == 0, G = N/NG a multiple of 16, 16-byte aligned rows.
 */
int dpk_gemm_mn(const void* A, int64_t lda, const void* W, const void* W2, int64_t ldw,
                const int64_t* sorted_indices, const int32_t* counts, void* D, int64_t ldd,
                int64_t M, int N, int K, int NG, int dtype, int act, void* stream);

/*
 * How the CTA-pair form of dpk_gemm_mn brings the gathered token rows into shared memory:
 * 0 = 16-byte cp.async issued by four warps (reference mechanism:
 * include/gemm_mn/v1/sm12x.cuh:541-573), 1 = TMA tile::gather4, one warp issuing 32 four-row
 * copies per 64-wide k-block.  Same results; process-wide, for measurements and tests.
 */
int dpk_set_gemm_mn_gather(int mode);

/*
 * Reduction-width routed projection (reference: GEMM_K_V1_Host::run,
 * DynamicPruningKernels/include/gemm_k/v1/sm12x.cuh:738-832; host wrapper
 * python/gemm_k/jit.py:345-425).
 *   D[t, n] = sum over active g, j of A[t, g*G + j] * W[n, g*G + j]
 * D is overwritten (the behaviour of the reference's PyTorch path,
 * python/references.py:21-26, 83-86), accumulated in fp32 without atomics.
 *   A [M,K] lda, W [N,K] ldw, D [M,N] ldd; row_bits / win_bits from dpk_mask_pack;
 *   residual: optional [M,N] ldr (NULL = none) added in fp32 before the single rounding --
 *   D = residual + projection, the sub-block's skip connection in the same pass; it may be D
 *   itself, which is the accumulate-onto-D behaviour of the reference's CuTe path
 *   (python/gemm_k/jit.py:368);
 *   workspace: see dpk_gemm_k_workspace_bytes (may be NULL).
 * Requirements: G = K/NG a multiple of 64, N % 8 == 0, 16-byte aligned rows.
 * Large shapes run on CTA pairs (one tile = 256 tokens x 256 outputs).  Where W is larger
 * than L2, their tiles are walked in groups of 8 weight chunks with the token windows inside, and the copy-issuing threads of all
 * CTAs line up at the start of every wave of tiles (a counter per wave in a per-device array,
 * zeroed on the stream before the launch; a bounded wait that is given up silently), so that
 * tiles sharing an operand find it in L2: 7.9 GB instead of 24.2 GB of DRAM reads for the
 * 16384 x 28672 x 8192 down projection.  dpk_set_gemm_k_wave_order(0) restores the plain order
 * without alignment (process-wide; for measurements and tests; same bits either way).
 */
int dpk_set_gemm_k_wave_order(int on);
int dpk_gemm_k(const void* A, int64_t lda, const void* W, int64_t ldw, const uint32_t* row_bits,
               const uint32_t* win_bits, void* D, int64_t ldd, int64_t M, int N, int K, int NG,
               int dtype, const void* residual, int64_t ldr, void* workspace, size_t workspace_bytes,
               void* stream);

/*
 * Optional scratch of dpk_gemm_k: with very few token windows (decode, M <= 512) the
 * group range is split over several CTAs which add fp32 partial sums into this buffer
 * (zero-filled by the call) before a final conversion.  Returns 0 when the shape never
 * uses it; passing NULL / 0 to dpk_gemm_k is always allowed and only costs decode speed.
 */
size_t dpk_gemm_k_workspace_bytes(int64_t M, int N);

/*
 * Small-batch / odd-shape routed projections on CUDA cores, reading the byte mask
 * directly (reference: GEMV_MN_V0_Host::run, include/gemv_mn/v0/sm8x.cuh:277-359 and
 * GEMV_K_V0_Host::run, include/gemv_k/v0/sm8x.cuh:216-295; dispatch rules
 * python/gemm_mn/jit.py:41,388 and python/gemm_k/jit.py:337-342).  `reduce_k` = 0 is
 * the gemm_mn semantics (inactive blocks left untouched), 1 the gemm_k semantics.
 * Requirement: K % 8 == 0.
 */
int dpk_gemv_routed(const void* A, int64_t lda, const void* W, int64_t ldw, const uint8_t* mask,
                    void* D, int64_t ldd, int64_t M, int N, int K, int NG, int dtype, int act,
                    int reduce_k, void* stream);

/* Bytes of scratch dpk_ffn_swiglu needs (routing layout, packed bits, intermediate). */
size_t dpk_ffn_workspace_bytes(int64_t M, int H, int I, int NG);

/*
 * Dynamic-width SwiGLU FFN in one call:
 *   y = down( mask * silu(gate(x)) * up(x) )
 * = routing layout + packed bits + fused gate/up GEMM + reduction-width down GEMM.
 * Replaces the caller-side composition gemm_mn(silu) / gemm_mn / multiply / gemm_k
 * (PruningInferSim/ops/mlp/m_pruning.py:76-105; WIDE/wrapper/attn_group_ffn_block.py:33-38).
 *   x [M,H], Wg,Wu [I,H], Wd [H,I], mask [M,NG] bytes, y [M,H]; all contiguous.
 */
int dpk_ffn_swiglu(const void* x, const void* Wg, const void* Wu, const void* Wd,
                   const uint8_t* mask, void* y, int64_t M, int H, int I, int NG, int dtype,
                   void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------- routed attention ---- */

/*
 * Prefill attention over the active query rows of each head group (reference:
 * Attention_Head_V3_Host::run, DynamicPruningKernels/include/attention_prefill/v3/
 * sm12x.cuh:25-169; host wrapper python/attention_prefill/jit.py:223-284).
 *   Q,O [B,Tq,Hq,D], K,V [B,Tk,Hk,D]; group g = query heads
 *   [g*Hq/NG, (g+1)*Hq/NG); query head h reads KV head h / (Hq/Hk).
 *   O is packed.  Q, K and V keep the heads of a token back to back but may be strided
 *   beyond that (a slice of a fused projection's output, a view of a KV cache with spare
 *   capacity): q_token_stride / q_batch_stride and kv_token_stride / kv_batch_stride (K and V
 *   alike) are in elements, multiples of 8, 0 = packed.  The reference takes DLPack views
 *   with strides {.., D, 1} the same way (sm12x.cuh:88-99).
 *   sorted_indices [B,Tq,NG] int64 (token index within the batch row), counts [B,NG].
 *   leftpad: optional [B] uint32 (keys k < leftpad[b] excluded) or NULL.
 *   causal: keys k <= q + causal_shift are visible (0 = top-left alignment).
 * Rows of inactive (token, group) pairs are not written: pass O zero-filled
 * (jit.py:250).  Requirements: D in {64,128}, Hq % NG == 0, Hq % Hk == 0.
 */
int dpk_attn_prefill(const void* Q, const void* K, const void* V, const int64_t* sorted_indices,
                     const int32_t* counts, const uint32_t* leftpad, void* O, int B, int Tq,
                     int Tk, int Hq, int Hk, int D, int NG, float scale, int causal,
                     int causal_shift, int dtype, int64_t q_token_stride, int64_t q_batch_stride,
                     int64_t kv_token_stride, int64_t kv_batch_stride, void* stream);

/*
 * Which prefill-attention kernel dpk_attn_prefill launches: 0 or 1 (default) = one query head
 * per CTA; 2 = two query heads per CTA sharing one K/V stream wherever heads 2i and 2i+1 share
 * their routing group and KV head (Hq/NG and Hq/Hk even), one head per CTA elsewhere.  Both give
 * the same bits; the one-head kernel measured faster.  Process-wide, for measurements and tests;
 * the reference selects kernel versions the same way through its kernel_version argument
 * (python/attention_prefill/jit.py:223-239).
 */
int dpk_set_attn_prefill_heads(int heads);

/* Bytes of scratch dpk_attn_decode needs. */
size_t dpk_attn_decode_workspace_bytes(int B, int Tk, int Hq, int Hk, int D, int NG);

/*
 * Decode attention, one query token per sequence, split over the KV length and
 * merged by log-sum-exp (reference: Attention_Head_V0_Host::run,
 * DynamicPruningKernels/include/attention_decode/v0/sm12x.cuh:23-198; host wrapper
 * python/attention_decode/jit.py:201-261).  KV heads none of whose query-head groups
 * are active for a sequence are never read.
 *   Q,O [B,1,Hq,D] packed, K,V [B,Tk,Hk,D], mask [B,NG] bytes, leftpad optional [B] uint32.
 *   kv_token_stride / kv_batch_stride (elements, multiples of 8, 0 = packed): K and V may be
 *   the first Tk rows of a [B,capacity,Hk,D] cache, read in place.
 * O is fully written (zeros for inactive groups).
 */
int dpk_attn_decode(const void* Q, const void* K, const void* V, const uint8_t* mask,
                    const uint32_t* leftpad, void* O, int B, int Tk, int Hq, int Hk, int D, int NG,
                    float scale, int dtype, int64_t kv_token_stride, int64_t kv_batch_stride,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same FFN for at most 128 tokens (decode steps), as two launches without any routing
 * layout: the weights are the M operand of the MMAs, all tokens the N operand, and the routing
 * mask is applied to the SwiGLU result (routed-out blocks are exact zeros, as in dpk_ffn_swiglu).
 * Same reference composition as dpk_ffn_swiglu.  mask [M,NG] bytes; H and I multiples of 128
 * (DPK_ERR_UNSUPPORTED otherwise: use dpk_ffn_swiglu).
 * Workspace: dpk_ffn_small_workspace_bytes(M,H,I) bytes, 256-byte aligned, ZERO-FILLED ONCE by
 * the caller before the first call; every call leaves it zero-filled again where it matters, so
 * it can be reused call after call (by one stream at a time) without a memset.
 */
size_t dpk_ffn_small_workspace_bytes(int64_t M, int H, int I);
int dpk_ffn_swiglu_small(const void* x, const void* Wg, const void* Wu, const void* Wd,
                         const uint8_t* mask, void* y, int64_t M, int H, int I, int NG, int dtype,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * Token router fused with the RMSNorm that reads the same hidden state (reference:
 * TokenRouter.forward, WIDE/wrapper/base_layer.py:89-114 -- the arithmetic of BottleneckRouter,
 * PruningInferSim/ops/router.py:85-126 --, the evaluation-time decision of
 * base_layer.py:204-207, and the norm modules called beside it,
 * WIDE/wrapper/attn_group_ffn_block.py:170-176, 195-200):
 *   c = x . w_down^T + b_down  [R];  logits = c . w_route^T + b_route  [NG,2];
 *   execute[m,g] = logits[m,g,0] >= logits[m,g,1]  (argmax of the pair, ties execute);
 *   xn = gamma * dtype(x * rsqrt(mean(x^2) + eps))  when gamma and xn are given.
 * x [M,ldx], w_down [R,H], w_route [2*NG,R] (contiguous), biases optional, execute [M,NG]
 * bytes, logits optional fp32 [M,NG,2].  R <= 16, H a multiple of 32 and at most ~14000.
 * round_like_module != 0 rounds c and the logits to `dtype` as a module running in that
 * dtype does; 0 keeps fp32.  x is read from device memory once.
 * Where H splits into 1, 2, 4 or 8 slices of at most 2048 columns (multiples of 32) a cluster
 * of that many CTAs works on 16 rows at a time, each CTA keeping its slice of w_down in shared
 * memory and streaming its columns of the rows through a ring of bulk copies; the partial
 * sums meet through distributed shared memory.  Other widths (up to ~14000 columns) take the
 * one-CTA-per-tile kernel, which re-reads w_down from L2 for every 8 rows.
 * dpk_set_router_norm_cluster(0) forces the latter everywhere (a measurement switch, process
 * wide; 1 = default).  No reference counterpart for the switch.
 */
int dpk_set_router_norm_cluster(int on);
int dpk_router_norm(const void* x, int64_t ldx, const void* gamma, float eps, const void* w_down,
                    const void* b_down, const void* w_route, const void* b_route, void* xn,
                    int64_t ldxn, uint8_t* execute, float* logits, int64_t M, int H, int R, int NG,
                    int dtype, int round_like_module, void* stream);

/*
 * Rotary embedding of q and k fused with the append of k and v to a preallocated
 * sequence-first KV cache (reference: apply_rotary_pos_emb, WIDE/wrapper/base_layer.py:18-44,
 * then past_key_values.update, WIDE/wrapper/attn_group_ffn_block.py:62-67, whose layer
 * concatenates [B,T,Hk,D] tensors, WIDE/wrapper/cache.py:24-46).
 *   q [B,T,Hq,D] rotated in place; k [B,T,Hk,D]; v [B,T,Hk,D]; cos, sin [T,D] (batch stride
 *   0) or [B,T,D]; k_cache, v_cache [B,capacity,Hk,D]: rows past_len .. past_len+T-1 receive
 *   the rotated k and v.  Without caches (both NULL) k is rotated in place.
 *   q_token_stride / kv_token_stride (elements, multiples of 8, 0 = packed): q, and k and v,
 *   may be column slices of one fused projection output [B*T, width].
 * fp32 arithmetic, one rounding.  D a multiple of 16.
 */
int dpk_rope_append(void* q, void* k, const void* v, const void* cos, const void* sin,
                    int64_t cs_batch_stride, void* k_cache, void* v_cache, int B, int T, int Hq,
                    int Hk, int D, int64_t capacity, int64_t past_len, int dtype,
                    int64_t q_token_stride, int64_t kv_token_stride, void* stream);

/* ---- tensor parallel: the row-parallel sum fused into the projection ---------------
 *
 * The reference runs one process on one GPU and has no collective; it only sketches the
 * split these calls serve (gate/up/q/k/v column parallel, down/o row parallel,
 * WIDE/transformer_fsdp_hook.py:44-54, switched off at WIDE/mainloop.py:602).  Rank r
 * holds the weights of its channel (or head) groups and computes a partial [M,N] sum.
 * Token rows [o*R, (o+1)*R), R = rows_per_owner (a multiple of 128), are owned by rank o.
 *
 *   1. dpk_gemm_k_scatter: dpk_gemm_k whose epilogue stores each token window into slab
 *      `rank` of the owner's staging buffer stage[o], laid out [world, R, ldd] -- stores
 *      into peer memory, overlapped with the tiles still being computed.
 *   2. the caller makes sure every rank has finished step 1 (any barrier between ranks
 *      that is ordered after the kernel on `stream`: dpk_peer_barrier, or a one-element
 *      all-reduce);
 *   3. dpk_reduce_gather on every rank: adds the `world` slabs of the rows it owns in
 *      fp32 (+ an optional residual [M,ld]), rounds once and stores the rows into every
 *      rank's out[j] ([M,ld]);
 *   4. a second barrier before anyone reads out[] or starts the next step 1.
 * No kernel of these waits on another GPU.  world <= 8.
 */

/* A device buffer other processes of the node can map.  handle: 64 bytes out, to be sent
 * to the peers by any host channel.  dpk_peer_open maps a peer's buffer into this
 * process (and enables peer access); close/free undo open/alloc. */
int dpk_peer_alloc(size_t bytes, void** ptr, void* handle);
int dpk_peer_open(const void* handle, void** ptr);
int dpk_peer_close(void* ptr);
int dpk_peer_free(void* ptr);

/*
 * Barrier between the ranks through flags in peer-mapped memory, as one small kernel on
 * `stream` (no counterpart in the reference).  Each rank owns `world` 32-bit slots, zero before
 * the first use; peer_flags: host array of `world` device pointers to every rank's slot array
 * (peer_flags[rank] == my_flags).  The kernel publishes this rank's arrival (epoch) to every
 * rank, ordered after everything earlier work of the stream wrote to peer memory, and waits
 * until every rank's arrival for the same epoch is visible here.  epoch has to grow by one per
 * barrier, identically on all ranks.  The wait gives up after timeout_ms: the status word is
 * set (code 107, kernel 8), the kernel returns, the context stays usable and the data of that
 * step must be discarded.  Every rank has to run on a GPU of its own.
 */
int dpk_peer_barrier(void* const* peer_flags, void* my_flags, int world, int rank, uint32_t epoch,
                     int timeout_ms, void* stream);

size_t dpk_gemm_k_scatter_workspace_bytes(int64_t M, int N, int64_t ldd);

/* Arguments as dpk_gemm_k, with the output replaced by the table of staging buffers
 * (host array of `world` device pointers, stage[rank] being this rank's own). */
int dpk_gemm_k_scatter(const void* A, int64_t lda, const void* W, int64_t ldw,
                       const uint32_t* row_bits, const uint32_t* win_bits, void* const* stage,
                       int world, int rank, int64_t rows_per_owner, int64_t ldd, int64_t M, int N,
                       int K, int NG, int dtype, void* workspace, size_t workspace_bytes,
                       void* stream);

/* stage: this rank's own staging buffer; out: host array of `world` device pointers;
 * residual: optional local [M,ld] added to the sum (NULL for none); max_blocks: upper bound
 * of the grid (0 = fill the GPU) -- a caller that runs this kernel beside a projection on
 * another stream passes about one block per SM so that both fit. */
int dpk_reduce_gather(const void* stage, void* const* out, const void* residual, int world,
                      int rank, int64_t rows_per_owner, int64_t M, int N, int64_t ld, int dtype,
                      int max_blocks, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DPK_B200_H_ */
