/*
 * b200nodes — C ABI of the B200 (sm_100a) decode / speculative-verify hot path.
 *
 * These entry points are what a host binding for the reference bundle's two ops
 * (`model.layers.*` -> qwen36_layer/layer.py, `logits_processor` -> qwen36_lmhead8/node.py,
 * manifest.toml:142-157 of snapshot qwen36_nodes_kb34) calls instead of the reference's pybind
 * units.  Conventions:
 *   - plain pointers and sizes only; every pointer is DEVICE memory unless its name ends in
 *     `_host`; the library allocates nothing and frees nothing, the caller owns all memory;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing synchronises;
 *   - bf16 tensors are passed as `const void*` / `void*` (2 bytes per element, row-major);
 *   - every function returns 0 on success, a negative B200_E_* code on an argument error or a
 *     positive cudaError_t value if a launch failed; nothing throws across the ABI;
 *     b200_last_error() returns a thread-local message for the last non-zero return;
 *   - kernels that wait on asynchronous copies bound every wait; when a wait gives up the kernel
 *     writes a B200_ST_* code into `status` (a device int32, may be NULL) and returns early.
 *     The caller reads it after synchronising the stream; 0 means no wait was abandoned.
 *   - there is no CPU fallback.
 */
#ifndef B200NODES_H
#define B200NODES_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1

#define B200_E_ARG (-1)      /* null pointer, bad size or unsupported shape */
#define B200_E_ALIGN (-2)    /* pointer not aligned as documented */
#define B200_E_WS (-3)       /* workspace too small */
#define B200_E_DRIVER (-4)   /* tensor-map encoder unavailable (no CUDA driver) */

#define B200_ST_WAIT_FULL 101
#define B200_ST_WAIT_EMPTY 102
#define B200_ST_WAIT_TMEM_FULL 103
#define B200_ST_WAIT_TMEM_EMPTY 104
#define B200_ST_WAIT_STATE 105
#define B200_ST_WAIT_STORE 106
#define B200_ST_WAIT_PEER 107   /* expert-parallel barrier: a peer rank's flag did not arrive in time */
#define B200_ST_BAD_LIST 110

int b200_abi_version(void);
const char* b200_last_error(void);

/* Budget of every device-side wait on an asynchronous copy or a tensor-core commit, in nanoseconds of
 * %globaltimer, for kernels launched on the CURRENT device after this call (0 restores the default of one
 * second).  The reference's waits spin without a limit (qk_gdn_verify.cu:140-144, qk_moe_up16.cu:656);
 * here a wait that runs out records a B200_ST_* code in the call's status word, and every role of the CTA
 * winds down (copies in flight are given a bounded time to land, TMEM is freed) and returns.
 * Not to be changed while kernels of the library are running on the device. */
int b200_set_wait_budget_ns(unsigned long long ns);
/* Self-test of that path: one CTA waits on a barrier that nothing arrives on and must come back with
 * B200_ST_WAIT_FULL in `status` after the budget.  The GPU stays usable. */
int b200_selftest_wait_expiry(int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Router.  Replaces qk_route.route / route48 / route16w (qk_route.cu:214,496,972) and the Triton
 * twins i8x_dec_gate / i8x_dec_topk (i8x_decode.py:226-262).
 *
 * logits[t,e] = sum_k x[t,k] * wr[e,k] (+ bias[e]) in fp32 with a fixed summation tree (one fma
 * chain from 0 per 128-deep k slice, ascending k; slices added in slice order; bias last), so
 * that expert ids are reproducible bit for bit.  Then softmax over E, top-k by largest logit with
 * ties to the smaller expert id (-0 == +0, NaN lowest), weights renormalised over the picks
 * (i8x_decode.py:99-117).
 *   x bf16 [T,H]; wr fp32 [E,H]; bias fp32 [E] or NULL; logits fp32 [T,E] (output) or NULL;
 *   ids int32 [T,K]; wts fp32 [T,K]; scratch: b200_router_scratch_bytes() bytes (slice partials),
 *   16-byte aligned.  H % 128 == 0, E % 64 == 0, E <= 1024, K <= 32.
 *   flags bit 0: round the logits to bf16 before the softmax / top-k (the reference's behaviour,
 *   i8x_decode.py:100).
 */
size_t b200_router_scratch_bytes(int T, int H, int E);
int b200_router(const void* x, const float* wr, const float* bias, int T, int H, int E, int K, int flags,
                float* logits, int32_t* ids, float* wts, void* scratch, size_t scratch_bytes, void* stream);

/* Router without a scratch argument, for hosts that cannot allocate device memory.
 * (No counterpart in the reference: its units allocate through torch.)
 *
 * A plugin slot that a serving engine calls per decode step gets its inputs and outputs from the
 * engine and nothing else; the engine owns the memory pool, and a cudaMalloc inside the step would
 * stall the device.  This entry point takes the same arguments as b200_router minus the scratch:
 * the slice partials go to a 2 MiB array built into the library (held by every GPU that loads the
 * library, until exit).  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - Limit: b200_router_scratch_bytes(T, H, E) must fit in b200_router_static_max_scratch_bytes()
 *     (2 MiB: 64 tokens x 512 experts at H = 2048 fit exactly); larger problems return B200_E_WS.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before any stream capture.
 *   - All calls share the array, and it keeps the last call's contents (nothing needs clearing:
 *     every partial that is read was written by the same call).  Calls that overlap on the GPU race.
 */
size_t b200_router_static_max_scratch_bytes(void);
int b200_router_static(const void* x, const float* wr, const float* bias, int T, int H, int E, int K, int flags,
                       float* logits, int32_t* ids, float* wts, void* stream);

/* ------------------------------------------------------------------------------------------
 * Routing lists.  Replaces i8x_dec_lists (i8x_decode.py:264-289) and the list-building tail of
 * route_kernel (qk_route.cu:297-357).
 *
 * Sorted-row layout used by the MoE kernels: routed pairs (slot p = t*K + j, i8x_decode.py:297)
 * are grouped by expert, in ascending slot order inside an expert, at rows [0, T*K); the shared
 * expert's rows are [T*K, T*K + T) (slot T*K + t, i8x_decode.py:442).  Only experts in
 * [e_lo, e_lo + E_local) are listed (expert-parallel shard); tokens with pos[t] == 0 are graph
 * padding and are skipped (qk_route.cu:229,307).  `block_rows` is the largest N tile of the
 * GEMM that will consume the lists (128 for int8, 32 for fp8).
 */
typedef struct b200_moe_lists {
  int32_t* counts;      /* [E_local + 1]   rows per local expert; entry E_local = shared expert */
  int32_t* offsets;     /* [E_local + 2]   first sorted row per expert (shared expert at T*K) */
  int32_t* row_of_pair; /* [T*K]           sorted row of routed slot p, or -1 */
  int32_t* slot_of_row; /* [T*(K+1)]       slot id of a sorted row, or -1 */
  float* wt_of_row;     /* [T*(K+1)]       routing weight of a sorted row (1 for the shared expert) */
  int32_t* blk_expert;  /* [max_blocks]    local expert of each GEMM block (E_local = shared) */
  int32_t* blk_row0;    /* [max_blocks]    first sorted row of the block */
  int32_t* blk_rows;    /* [max_blocks]    rows in the block, 1..block_rows */
  int32_t* nblocks;     /* [1] */
} b200_moe_lists;

/* Order of the block list: with block_rows = 128 the blocks come heaviest first (all full blocks, then the
 * partial ones by quarter of the block size, each class in expert order), which balances the int8 GEMMs'
 * round-robin tile deal; with smaller block_rows they come in expert order (the reference's order,
 * qk_route.cu:322-357).  Consumers must not assume either.
 * max_blocks the caller must provide for a given problem: */
int b200_moe_max_blocks(int T, int K, int E_local, int block_rows);

int b200_moe_build_lists(const int32_t* ids, const float* wts, const int64_t* pos, int T, int K, int e_lo,
                         int E_local, int block_rows, int with_shared, const b200_moe_lists* lists, void* stream);
/* The same with shared-expert rows for tokens [shared_lo, shared_lo + shared_n) only (0 <= shared_lo,
 * shared_lo + shared_n <= T; shared_n = 0: none).  Expert-parallel ranks see the gathered tokens of all
 * ranks but run the shared expert for their own tokens only.  (No counterpart in the reference.) */
int b200_moe_build_lists_range(const int32_t* ids, const float* wts, const int64_t* pos, int T, int K, int e_lo,
                               int E_local, int block_rows, int shared_lo, int shared_n,
                               const b200_moe_lists* lists, void* stream);

/* ------------------------------------------------------------------------------------------
 * MoE block, int8 W8A8.  Replaces i8x_decode.moe_row_batch (i8x_decode.py:528-576): up + SwiGLU
 * (i8x_dec_up, qk_moe_up16.cu:139), down (i8x_dec_down, qk_moe_dn16.cu:136) and, via
 * b200_moe_combine, the combine; the W8A8 arithmetic is the reference's w8_up / w8_dn lane
 * (qk_moe_prefill_i8.cu:3646-3655,4061-4071): int32 accumulation over the whole K, value =
 * (float(acc) * xs[row]) * ws[col], h rounded to bf16 and re-quantised per row.
 *
 *   x bf16 [T,H];  w13 int8 [E_local,2I,H] (rows 0..I-1 gate, I..2I-1 up), s13 fp32 [E_local,2I];
 *   w2 int8 [E_local,H,I], s2 fp32 [E_local,H];  shared expert sh13 [2I,H], shs13 [2I],
 *   sh2 [H,I], shs2 [H] (NULL sh13 = no shared expert);
 *   cache bf16 [T*(K+1),H] (output): row `slot` = bf16(down row * routing weight)
 *   (i8x_decode.py:420-422).  H % 256 == 0, I % 128 == 0.
 *   ws: workspace of b200_moe_w8a8_workspace_bytes() bytes, 1024-byte aligned.
 *   dbg_acc13 int32 [T*(K+1), 2I] or NULL: raw up accumulators per slot (parity checks).
 *   dbg_h bf16 [T*(K+1), I] or NULL: SwiGLU output per slot.
 *   stages: 0 runs the whole block; otherwise a mask of B200_MOE_STAGE_* runs only those launches
 *   on the data the earlier ones left in `ws` (used to time one kernel on its own).
 */
#define B200_MOE_STAGE_QUANT 1   /* quantise + permute activations */
#define B200_MOE_STAGE_UP 2      /* gate/up GEMM + SwiGLU */
#define B200_MOE_STAGE_HQUANT 4  /* re-quantise h */
#define B200_MOE_STAGE_DOWN 8    /* down GEMM + weighted unpermute */
#define B200_MOE_TEST_STARVE 16  /* self-test, OR-ed into `stages`: the GEMM producers leave out the token rows, so no
                                    pipeline stage ever completes, every bounded wait runs out and the kernels return
                                    with a B200_ST_WAIT_* status (set a short b200_set_wait_budget_ns first) */
typedef struct b200_moe_weights {
  const void* w13;
  const float* s13;
  const void* w2;
  const float* s2;
  const void* sh13;
  const float* shs13;
  const void* sh2;
  const float* shs2;
} b200_moe_weights;

size_t b200_moe_w8a8_workspace_bytes(int T, int H, int I, int K);
int b200_moe_w8a8(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                  const b200_moe_lists* lists, void* cache, void* ws, size_t ws_bytes, int32_t* dbg_acc13,
                  void* dbg_h, int stages, int32_t* status, void* stream);

/* Expert-parallel form of b200_moe_w8a8 with the combine-side exchange fused into the down GEMM.
 * (No counterpart in the reference, which is single-GPU: layer.py:396-402.)
 * x holds the gathered tokens of all ranks, T = ep_world * ep_tokens_per_rank, rank r's tokens at rows
 * [r * ep_tokens_per_rank, ...); `lists` were built for this rank's experts (e_lo, E_local), without the
 * shared expert or with shared rows for this rank's own tokens (b200_moe_build_lists_range with
 * shared_lo = ep_rank * ep_tokens_per_rank, shared_n = ep_tokens_per_rank).  The down epilogue stores bf16(y * routing weight) for global slot
 * s = t*K + j straight into the home rank's cache, peer_cache_host[s / (ep_tokens_per_rank*K)] +
 * (s % (ep_tokens_per_rank*K)) * H, with ordinary stores; shared-expert rows are kept only for this
 * rank's own tokens, at row ep_tokens_per_rank*K + local token of its own cache (the layout
 * b200_moe_combine reads).  peer_cache_host is a HOST array of ep_world DEVICE pointers, entry r being
 * rank r's cache [ep_tokens_per_rank*(K+1), H] bf16 as mapped into this process (its own buffer for
 * r == ep_rank, peer-mapped memory otherwise).  No TMA touches peer memory.  The caller synchronises the
 * ranks (any barrier that orders their streams) before the home ranks read their caches. */
int b200_moe_w8a8_ep(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                     const b200_moe_lists* lists, void* const* peer_cache_host, int ep_world, int ep_rank,
                     int ep_tokens_per_rank, void* ws, size_t ws_bytes, int32_t* status, void* stream);

/* Expert-parallel dispatch (no counterpart in the reference): this rank's T_local token rows and their routing
 * are stored into every rank's gathered buffers at row offset ep_rank * T_local, over NVLink with ordinary
 * stores: peer_*_host are HOST arrays of ep_world DEVICE pointers, entry r being rank r's x_all
 * [ep_world * T_local, H] bf16, ids_all / wts_all [ep_world * T_local, K] as mapped into this process.  The
 * caller runs a barrier among the ranks before any rank reads its gathered buffers. */
int b200_ep_push(const void* x, const int32_t* ids, const float* wts, int T_local, int H, int K, int ep_rank,
                 int ep_world, void* const* peer_x_host, void* const* peer_ids_host, void* const* peer_wts_host,
                 void* stream);

/* MoE block, fp8 e4m3 with 128x128 weight block scales and per-(token,128-channel) activation
 * scales.  The reference has no block-scaled fp8 MoE; the arithmetic is its scaled-GEMM recipe
 * applied per block: per 128-k block the MMA chain starts from zero and is promoted
 * acc = fma(partial, a_scale * w_scale, acc) in increasing k (qk_lt.cu:361-364,
 * qk_moe_prefill_i8.cu:3649-3651); activations are quantised scale = max(amax/448, 1e-12),
 * y = e4m3(x * (1/scale)) (fp8.py:21-34); SwiGLU rounding points as in the int8 block.
 * Same layouts with e4m3 bytes; s13 fp32 [E_local, 2I/128, H/128], s2 fp32 [E_local, H/128, I/128];
 * shared scales likewise without the expert axis.  The routing lists must have been built with
 * block_rows <= 32 (a block with more rows is reported as B200_ST_BAD_LIST).  H, I multiples of 128, <= 4096. */
size_t b200_moe_fp8_workspace_bytes(int T, int H, int I, int K);
int b200_moe_fp8(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                 const b200_moe_lists* lists, void* cache, void* ws, size_t ws_bytes, void* dbg_h, int stages,
                 int32_t* status, void* stream);

/* Expert-parallel form of b200_moe_fp8, as b200_moe_w8a8_ep is of b200_moe_w8a8: x holds the gathered tokens
 * of all ranks, the lists are this rank's (block_rows <= 32, shared rows for its own tokens), and the down epilogue
 * stores every weighted row into its home rank's cache with ordinary stores over NVLink.  (No counterpart in the
 * reference.) */
int b200_moe_fp8_ep(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                    const b200_moe_lists* lists, void* const* peer_cache_host, int ep_world, int ep_rank,
                    int ep_tokens_per_rank, void* ws, size_t ws_bytes, int32_t* status, void* stream);

/* Barrier among the ranks of an expert-parallel group, as one small kernel on `stream` (no counterpart in the
 * reference).  Every rank owns a flag array uint64 [B200_EP_CHANNELS][8] in memory that all ranks can store to
 * (peer-mapped), zeroed once, and a private epoch array uint64 [B200_EP_CHANNELS], zeroed once.  A call advances
 * this rank's epoch of `channel`, stores it into entry [channel][ep_rank] of every rank's flag array with
 * release stores at system scope (after a system-scope fence, so that everything this rank's earlier kernels on the
 * stream wrote to peers is visible first), then polls its own entries [channel][0..ep_world) until every rank's
 * epoch has arrived.  The poll is bounded by `timeout_ns` of %globaltimer: when it runs out the kernel records
 * B200_ST_WAIT_PEER in `status` and returns; it never traps and never spins without a limit.  Once `status` is
 * non-zero later barriers return at once, so a dead peer costs one timeout, not one per barrier.  All ranks must call
 * with the same channel sequence.  peer_flags_host: HOST array of ep_world DEVICE pointers (entry r = rank r's
 * flag array as mapped into this process).  Plain loads and stores only: no multimem, no TMA. */
#define B200_EP_CHANNELS 4
int b200_ep_barrier(void* const* peer_flags_host, unsigned long long* epochs, int ep_world, int ep_rank, int channel,
                    unsigned long long timeout_ns, int32_t* status, void* stream);

/* All-gather by peer stores (no counterpart in the reference): `bytes` bytes at `src` are stored into every rank's
 * buffer at byte offset dst_offset_bytes (peer_dst_host: HOST array of ep_world DEVICE pointers).  4-byte
 * granularity; ordinary stores.  The caller runs b200_ep_barrier before any rank reads its buffer.  Used for the
 * hidden rows in front of the vocabulary-sharded LM head and for its (max, argmax) pairs. */
int b200_ep_put(const void* src, size_t bytes, size_t dst_offset_bytes, void* const* peer_dst_host, int ep_world,
                void* stream);

/* Combine.  Replaces i8x_dec_combine (i8x_decode.py:425-443) / combine_norm_kernel
 * (qk_route.cu:686-820, without the next-layer norm): out[t] = bf16(sum_j cache[t*K+j] in slot
 * order + sigmoid(x[t].gate_w) * cache[T*K+t]); rows with pos[t] == 0 are written as zeros.
 * gate_w NULL = no shared expert.  H % 8 == 0. */
int b200_moe_combine(const void* cache, const void* x, const void* gate_w, const int64_t* pos, int T, int H, int K,
                     void* out, void* stream);

/* The combine with the next layer's input norm folded in, as combine_norm_kernel does (qk_route.cu:686-820,
 * the tail at :779-819): out as above (may be NULL when only the normed row is wanted);
 * residual[t] <- r = bf16(out[t] + residual[t]); normed[t] = bf16(r * rsqrt(mean r^2 + eps) * (1 + norm_w)).
 * Bit-identical to b200_moe_combine followed by b200_add_rmsnorm. */
int b200_moe_combine_norm(const void* cache, const void* x, const void* gate_w, const int64_t* pos, int T, int H,
                          int K, void* out, void* residual, const void* norm_w, float eps, void* normed,
                          void* stream);
/* The same, and the normed rows also leave in the form the next layer's first projection reads: e4m3 xq_out [T, H] and
 * scales xs_out fp32 [T, H/128] (per token per 128 channels, scale = max(amax / 448, 1e-12): the arithmetic of the
 * projections' own activation quantiser, fp8.py:21-34), to be passed to b200_dense_fp8_split_q or b200_attn_front_q.
 * H == 2048, K <= 12.  (The reference quantises inside its projection kernels.) */
int b200_moe_combine_norm_q(const void* cache, const void* x, const void* gate_w, const int64_t* pos, int T, int H,
                            int K, void* out, void* residual, const void* norm_w, float eps, void* normed, void* xq_out,
                            float* xs_out, void* stream);

/* ------------------------------------------------------------------------------------------
 * Gated DeltaNet speculative verify.  Replaces qk_gdn_verify.gdn_verify_fused
 * (qk_gdn_verify.cu:293, gdn_fused.py:37-57) with an explicit state instead of the ReplaySSM
 * ring: causal conv (width 4, carried 3-token state) + SiLU, q/k L2 norm, gates, delta-rule
 * recurrence over the 4 draft tokens, gated RMSNorm; the state written back is the state after
 * accepted[b] tokens and the conv state is rolled by accepted[b] tokens.
 *   mixed bf16 [B*4, 8192] ([q 2048 | k 2048 | v 4096]); z bf16 [B*4, 4096]; a, b bf16 [B*4, 32];
 *   conv_state bf16 [B, 8192, 3] (in/out); conv_w bf16 [8192, 4]; a_log, dt_bias fp32 [32];
 *   state fp32 [B, 32, 128, 128] (S[v][k], in/out); accepted int32 [B] in 0..4;
 *   norm_w bf16 [128]; out bf16 [B*4, 4096].  state must be 16-byte aligned.
 * Two launches: a small kernel computes everything that does not touch the state (conv, norms, gates,
 * window coefficients) into `ws`, then a streaming kernel moves the state tiles (it starts before the first
 * has finished and requests its first tiles meanwhile).
 */
int b200_gdn_verify(const void* mixed, const void* z, const void* a, const void* b, void* conv_state,
                    const void* conv_w, const float* a_log, const float* dt_bias, float* state,
                    const int32_t* accepted, const void* norm_w, float eps, int B, void* out, void* ws,
                    size_t ws_bytes, int32_t* status, void* stream);
/* Scratch of b200_gdn_verify: the operands its first launch prepares for its second (128-byte aligned). */
size_t b200_gdn_workspace_bytes(int B);

/* The same step on the state layout the reference's engine keeps (ReplaySSM, gdn_fused.py:19-57,
 * qk_gdn_verify.cu:61-73,586-593,631-647,706-717,769-781,883-898): a read-only fp32 checkpoint per slot
 * plus a 16-entry circular ring of (d, k, g) per request.  Logical entry c < write_pos[r] lives at
 * physical entry (cache_base[r] + c) & 15; the state the window sees is
 *   e^{total} H0 + sum_c e^{total - pre_c} d_c k_c^T   (pre_c = g_0 + .. + g_c, total = pre_{write_pos-1})
 * read from the high parts of the d and k rings.  The window's D_s, unit keys k_s (bf16 high part, and
 * low part = bf16(value - high)) and gates g_s (fp32) are appended at logical entries write_pos + s for
 * those below 16; the checkpoint is never written; the cursors are the caller's (rollback = the caller
 * does not advance write_pos).  conv_state is rolled by the whole window ([x1 x2 x3]) and the per-draft
 * windows are recorded per channel as [s1 s2 x0 x1 x2 x3] in window[win_idx[b]].
 *   checkpoint fp32 [state_slots, 32, 128, 128]; conv_state bf16 [state_slots, 8192, 3], both indexed
 *   by state_idx[b] (< 0: padded request, its output rows are zero and nothing else is touched);
 *   window bf16 [window slots, 8192, 6]; d_ring, dlo_ring bf16 [ring slots, 32, 16, 128];
 *   k_ring, klo_ring bf16 [ring slots, 16, 16, 128]; g_ring fp32 [ring slots, 32, 16];
 *   state_idx, ring_idx, win_idx int32 [B]; write_pos, cache_base int32 [ring slots];
 *   the other arguments as above (ws: b200_gdn_workspace_bytes(B)).  Requests of one call must not share a slot. */
int b200_gdn_verify_replay(const void* mixed, const void* z, const void* a, const void* b, void* conv_state,
                           const void* conv_w, void* window, const float* a_log, const float* dt_bias,
                           const float* checkpoint, int state_slots, void* d_ring, void* dlo_ring, void* k_ring,
                           void* klo_ring, float* g_ring, const int32_t* state_idx, const int32_t* ring_idx,
                           const int32_t* win_idx, const int32_t* write_pos, const int32_t* cache_base,
                           const void* norm_w, float eps, int B, void* out, void* ws, size_t ws_bytes,
                           int32_t* status, void* stream);

/* Folds the committed ring entries of B requests into their checkpoints, in place:
 *   H0 <- e^{total} H0 + sum_{c < write_pos} e^{total - pre_c} (d_c high + low) (k_c high + low)^T.
 * The reference leaves this to its engine's pool (gdn_fused.py:24, `replayssm_spec_fold`); it is here so that the
 * ring layout can be driven without that engine.  Cursors are not touched: the caller sets write_pos[ring] to 0
 * afterwards.  Requests with state_idx < 0 or an empty ring are skipped.  Arguments as b200_gdn_verify_replay. */
int b200_gdn_ring_fold(float* checkpoint, const void* d_ring, const void* dlo_ring, const void* k_ring,
                       const void* klo_ring, const float* g_ring, const int32_t* state_idx, const int32_t* ring_idx,
                       const int32_t* write_pos, const int32_t* cache_base, int B, void* stream);

/* ------------------------------------------------------------------------------------------
 * Attention verify core.  Replaces qk_attn_verify.attn_verify_fused (attn_fused.py:110-124;
 * attn_verify_kernel, qk_attn_verify.cu:354-744) behind the projection front above: per request
 * the 4 draft tokens x 16 q heads attend to the request's e4m3 KV cache and causally to each
 * other (new token t sees new tokens <= t, qk_attn_verify.cu:521); S = q . k from e4m3 operands
 * with fp32 accumulation, times `scale`; online softmax in the log2 domain whose running maximum
 * moves only when a tile exceeds it by more than 8 (:210,264-267); P rounded to f16 before P . V
 * (:297-301); KV range split over CTAs and merged by an ordered sum (:690-737);
 * out = bf16(bf16(o / l) * sigmoid(gate)) (:559-562).  The new tokens' K and V rows are written
 * into the cache first (the reference does it at out_cache_loc, :452-466).
 *
 * Cache layout (chosen for this GPU; the reference reads 1-token pages through a per-token table):
 * pages of 128 tokens; kcache e4m3 [num_pages][2 kv heads][128 keys][256 dims]; vcache e4m3
 * [num_pages][2][256 dims][128 keys] (dim-major).  page_table int32 [B, pt_stride]: page of tokens
 * 128 i .. 128 i + 127 of request b; seqlens int32 [B]: tokens of the request INCLUDING the 4
 * drafts (seqlens >= 4; the drafts occupy positions seqlens-4 .. seqlens-1).
 *   q e4m3 [4B,16,256], gate bf16 [4B,16,256], k_new, v_new e4m3 [4B,2,256] (b200_attn_front with
 *   out_fp8 = 1); out bf16 [4B, 4096]; splits: CTAs per (request, kv head), 1..64
 *   (b200_attn_verify_splits(B) fills the GPU); ws: b200_attn_verify_workspace_bytes(B, splits).
 */
int b200_attn_verify_splits(int B);
size_t b200_attn_verify_workspace_bytes(int B, int splits);
int b200_attn_verify(const void* q, const void* gate, const void* k_new, const void* v_new, void* kcache,
                     void* vcache, int num_pages, const int32_t* page_table, int pt_stride,
                     const int32_t* seqlens, int B, float scale, int splits, void* out, void* ws,
                     size_t ws_bytes, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused gated-attention projection front.  Replaces fp8.linear_q + qk_attn_verify.
 * attn_prefill_front (fp8.py:77-108, qk_attn_verify.cu:765-800): fp8 block-scaled GEMM
 * x[T,2048] . W[9216,2048]^T (activations quantised per token per 128 channels, per-128-k
 * promotion), the result rounded to bf16 as the reference's projection stores it, then per head:
 * q/k RMSNorm x * rsqrt(mean x^2 + eps) * (1 + w) -> bf16 and neox RoPE on dims (i, i+32), i < 32
 * -> bf16 (qk_attn_verify.cu:180-208), all in the GEMM epilogue.  Column layout per q head h: q at
 * h*512, gate at h*512+256; K at 8192; V at 8704 (qk_attn_verify.cu:25,443,450).
 *   x bf16 [T,2048]; w e4m3 [9216,2048]; w_s fp32 [72,16]; q_norm_w, k_norm_w bf16 [256];
 *   positions int64 [T] (clamped to [0, max_pos)); cos_sin fp32 [max_pos, 64] = [cos 32 | sin 32];
 *   q [T,16,256], k, v [T,2,256]: e4m3 bytes (cvt.rn.satfinite, qk_attn_verify.cu:142-146) if
 *   out_fp8 else bf16; gate bf16 [T,16,256].  All 16-byte aligned.
 *   ws: b200_attn_front_workspace_bytes(T) bytes, 1024-byte aligned.
 */
size_t b200_attn_front_workspace_bytes(int T);
int b200_attn_front(const void* x, int T, const void* w, const float* w_s, const void* q_norm_w,
                    const void* k_norm_w, const int64_t* positions, const float* cos_sin, int max_pos, float eps,
                    int out_fp8, void* q, void* gate, void* k, void* v, void* ws, size_t ws_bytes, int32_t* status,
                    void* stream);
/* The same on rows that are already quantised (xq e4m3 [T, 2048], 16-byte aligned, xs fp32 [T, 16]: the outputs of
 * b200_moe_combine_norm_q); no workspace, one launch less. */
int b200_attn_front_q(const void* xq, const float* xs, int T, const void* w, const float* w_s, const void* q_norm_w,
                      const void* k_norm_w, const int64_t* positions, const float* cos_sin, int max_pos, float eps,
                      int out_fp8, void* q, void* gate, void* k, void* v, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Decode-width dense projections.  Replace the reference's weight-streaming projections between
 * the named kernels: gdn_in_proj / qkv_proj (qk_proj_decode.cu:409-470, dense8.py:317-353) and
 * o_proj + add + Gemma norm (proj.py:30-112).  The reference streams bf16 or W8A16 weights; the
 * target keeps every weight in the one fp8 block-scaled format.
 *   b200_dense_fp8: out[T,N] = bf16(x[T,H] . W[N,H]^T), x bf16 quantised per token per 128
 *     channels, W e4m3 [N,H] with scales fp32 [ceil(N/128), H/128], per-128-k promotion;
 *     T >= 1 (more than 64 rows: 64-row chunks, every weight tile against each chunk in turn inside one launch),
     H % 128 == 0, H <= 4096; ws: b200_dense_fp8_workspace_bytes(T,H), 1024-aligned.
 *   b200_dense_fp8_split: the same GEMM with the N output features cut into 1..4 consecutive segments, segment i
 *     (seg_cols_host[i] features, a multiple of 32 except the last) written to seg_out_host[i] with row pitch
 *     seg_ld_host[i] elements: the GDN in_proj's [q k v | z | b | a] land in the four buffers the verify kernel
 *     takes (dense8.py:64-68 slices them after the GEMM).  seg_*_host are HOST arrays.
 *   b200_add_rmsnorm: residual <- bf16(proj + residual) (proj is already bf16; the add is fp32:
 *     proj.py:75-77), out = bf16(residual * rsqrt(mean residual^2 + eps) * (1 + w)) (proj.py:78-81).
 */
size_t b200_dense_fp8_workspace_bytes(int T, int H);
int b200_dense_fp8(const void* x, int T, int H, const void* w, const float* w_s, int N, void* out, void* ws,
                   size_t ws_bytes, int32_t* status, void* stream);
int b200_dense_fp8_split(const void* x, int T, int H, const void* w, const float* w_s, int N, int nseg,
                         const int* seg_cols_host, void* const* seg_out_host, const int* seg_ld_host, void* ws,
                         size_t ws_bytes, int32_t* status, void* stream);
/* b200_dense_fp8_split on rows that are already quantised (xq e4m3 [T, H], 16-byte aligned, xs fp32 [T, H/128]: the
 * outputs of b200_moe_combine_norm_q); no workspace, one launch less, the same bits. */
int b200_dense_fp8_split_q(const void* xq, const float* xs, int T, int H, const void* w, const float* w_s, int N, int nseg,
                           const int* seg_cols_host, void* const* seg_out_host, const int* seg_ld_host, int32_t* status,
                           void* stream);
/* The output projection of a mixer fused with what follows it, as proj.project_add_norm does (proj.py:84-112: split-K
 * partials in fp32, then one kernel that sums them, adds the residual and norms):
 *   proj = bf16(x[T,K] . W[N,K]^T) with the K range cut into parts so that weight tiles x parts fill the GPU (a
 *   [2048, 4096] weight has only 16 weight tiles), the parts' fp32 sums added in part order;
 *   residual <- bf16(proj + residual); out = bf16(residual * rsqrt(mean residual^2 + eps) * (1 + norm_w)).
 * The number of parts depends on the weight's shape only, so a row's result does not depend on the batch it is in.
 *   x bf16 [T,K]; w e4m3 [N,K], w_s fp32 [ceil(N/128), K/128]; residual bf16 [T,N] (in/out); norm_w bf16 [N];
 *   out bf16 [T,N]; proj_out bf16 [T,N] or NULL (the rounded projection, for checks);
 *   ws: b200_dense_fp8_add_rmsnorm_workspace_bytes(T,K,N) bytes, 1024-byte aligned.  K % 128 == 0, K <= 4096, N % 8 == 0. */
size_t b200_dense_fp8_add_rmsnorm_workspace_bytes(int T, int K, int N);
int b200_dense_fp8_add_rmsnorm(const void* x, int T, int K, const void* w, const float* w_s, int N, void* residual,
                               const void* norm_w, float eps, void* out, void* proj_out, void* ws, size_t ws_bytes,
                               int32_t* status, void* stream);
int b200_add_rmsnorm(const void* proj, void* residual, const void* w, float eps, int T, int H, void* out,
                     void* stream);

/* ------------------------------------------------------------------------------------------
 * LM head shard with fused argmax.  Replaces the logits GEMM of qwen36_lmhead8
 * (lmhead8.py:171-197, w8a8.py:99-120, qk_proj_decode.cu:1210,1468: vocabulary rows on the MMA M
 * side, weight streamed once); the reference returns logits and has no argmax
 * (node.py:136-151).  Per row of x: the largest fp8 block-scaled logit over this shard's
 * vocabulary rows and its global id (shard_lo + local row); ties go to the lower id, NaN never wins.
 *   x bf16 [T,H], T >= 1 (more than 64 rows: 64-row chunks inside one launch), H % 128 == 0, H <= 4096;
 *   w e4m3 [V_shard,H];
 *   w_s fp32 [ceil(V_shard/128), H/128]; max_out fp32 [T]; idx_out int32 [T];
 *   logits_out fp32 [T,V_shard] or NULL; ws: b200_lmhead_workspace_bytes(T,H,V_shard) bytes,
 *   1024-byte aligned.
 */
size_t b200_lmhead_workspace_bytes(int T, int H, int V_shard);
int b200_lmhead_argmax(const void* x, int T, int H, const void* w, const float* w_s, int V_shard, int shard_lo,
                       float* max_out, int32_t* idx_out, float* logits_out, void* ws, size_t ws_bytes,
                       int32_t* status, void* stream);
/* Merge S gathered shard results (maxes, idxs: [S,T]) into tokens [T]: largest value, ties to the
 * lower id.  This is the step after the all-gather of (max, argmax) pairs of a vocab-sharded head. */
int b200_argmax_merge(const float* maxes, const int32_t* idxs, int S, int T, int32_t* tokens, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200NODES_H */
