/*
 * b200moe.h -- C ABI of the B200 (sm_100a) FP8 block-scale MoE layer.
 *
 * One handle = one rank's share of an MoE layer of a fixed shape.  All data pointers are
 * DEVICE pointers unless stated otherwise; inputs are borrowed and never modified; every
 * launch is enqueued on the caller's stream and no entry point synchronises the host unless
 * its comment says so.  Every function returns 0 on success, a negative B200MOE_E_* code for
 * an argument/setup error, or a positive cudaError_t value.
 *
 * The reference interfaces each entry point replaces are cited as path:line inside the
 * reference corpus (OpenBMB/JustGoal), with
 *   <def>  = moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048
 *   KF94/  = kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/
 *   GF/    = goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/
 *   SF1/   = goal_single_shape/fable-5.1/moe_fp8_fwd/t1/
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ROUTING_DEEPSEEK 0      /* sigmoid + bias, group-limited top-k            */
#define B200MOE_ROUTING_RENORM_NAIVE 1  /* softmax -> top-k -> renormalise (no groups)     */
#define B200MOE_ROUTING_DEFAULT 2       /* softmax -> top-k, weights = probabilities        */
#define B200MOE_ROUTING_RENORMALIZE 3   /* top-k on the logits -> softmax over the selected */
#define B200MOE_ROUTING_LLAMA4 4        /* top-1 on the logits -> sigmoid (top_k must be 1) */
#define B200MOE_ROUTING_TOPK 5          /* top-k on the logits, uniform weights factor/top_k */
/* Modes 1-5: routing_bias, when given, is added to the logits first; every weight is multiplied by
 * routed_scaling_factor.  The reference corpus ships only mode 0 (GF/moe_common.cuh:271-365); modes
 * 1-5 follow the routing methods published with the operator family
 * (flashinfer-python 0.6.11, flashinfer/trace/templates/moe.py:186-390). */

#define B200MOE_E_BADARG   (-1)   /* null pointer, negative size, unsupported shape        */
#define B200MOE_E_WORKSPACE (-2)  /* workspace too small or misaligned                     */
#define B200MOE_E_DRIVER   (-3)   /* cuTensorMapEncodeTiled unavailable / failed           */
#define B200MOE_E_DEVICE   (-4)   /* not an sm_100 device                                  */
#define B200MOE_E_KERNEL   (-5)   /* a kernel recorded a device-side error (see status)    */
#define B200MOE_E_TOO_LARGE (-6)  /* more tokens than the allocation-free entry point holds */
#define B200MOE_E_BUILD    (-7)   /* library built with an unexpected register allocation   */

#define B200MOE_NOALLOC_MAX_TOKENS 8192

typedef struct b200moe_config {
    int hidden;              /* H, multiple of 128                                         */
    int intermediate;        /* I, multiple of 128                                         */
    int num_experts;         /* E global, multiple of 32, <= 512                           */
    int num_local_experts;   /* experts owned by this rank, <= 256                         */
    int top_k;               /* <= 8                                                       */
    int n_group;             /* DeepSeek routing: number of expert groups (else 1)         */
    int topk_group;          /* DeepSeek routing: groups kept per token (else 1)           */
    int routing_mode;        /* B200MOE_ROUTING_*                                          */
} b200moe_config;

typedef struct b200moe_ctx* b200moe_handle;

/* Offsets (bytes from the workspace base) of the intermediates one forward leaves behind;
 * for tests and debugging only. */
typedef struct b200moe_ws_layout {
    size_t status;        /* int32[8]: [0] device error word, [1] pairs P, [2] padded rows,
                             [3] token tiles, [4] active experts                           */
    size_t counts;        /* int32[E_local] tokens per local expert (sum of the slices)    */
    size_t expert_row0;   /* int32[E_local+1] first (padded) row of each expert            */
    size_t tile_prefix;   /* int32[E_local+1] exclusive prefix of token tiles              */
    size_t topk_idx;      /* int32[T, top_k] global expert ids                             */
    size_t topk_w;        /* float[T, top_k]                                               */
    size_t pair_row;      /* int32[T, top_k] row of a local pair (undefined if not local)  */
    size_t row_token;     /* int32[rows_cap] token of a row, -1 for padding                */
    size_t row_w;         /* float[rows_cap] routing weight of a row                       */
    size_t a_perm;        /* uint8[rows_cap, H] expert-sorted fp8 activations              */
    size_t a_scale_perm;  /* float[H/128, rows_cap]                                        */
    size_t act_hi;        /* uint8[rows_cap, I] e4m3 of SwiGLU output / scale              */
    size_t act_lo;        /* uint8[rows_cap, I] e4m3 of the rounding residual              */
    size_t act_scale;     /* float[I/128, rows_cap]                                        */
    size_t y;             /* fp16[rows_cap, H] expert output per row (before the weight)   */
    size_t sk_count;      /* int32[2][4*SMs+4] per GEMM: arrival counters of chunked units, chunk claim counter */
    size_t slices;        /* int32[ceil(T*top_k/1024)][E_local] histogram of the local experts per
                             slice of 1024 (token, expert) pairs, token-major                */
    size_t sk_partial;    /* fp32 partial accumulators of the chunked units: slot (unit, chunk) */
    size_t trace;         /* int64[2][SMs][16] per-CTA time lines of GEMM1 and GEMM2: slot 0 =
                             %globaltimer at entry, slots 1..11 = SM clocks since entry at:
                             prologue done, first/last TMA issue, first/last MMA, first/last
                             promotion, partial published, partials added, epilogue, exit     */
    size_t tok_count;     /* int32[T][H/256] (narrow token tiles only, else empty): units that have delivered
                             a row of token t for output columns [256 j, 256 j + 256) - the combine fused
                             into the GEMM2 epilogue                                          */
    size_t rows_cap;      /* number of rows the row-indexed buffers hold                   */
    size_t token_tile;    /* tokens per GEMM tile chosen for this T                        */
    size_t total_bytes;
} b200moe_ws_layout;

/* Create / destroy a layer handle on the CURRENT device.  Does one-time kernel attribute
 * setup and allocates 64 bytes of device memory (two words at which the CTAs of the fused
 * front end meet; no later call allocates).  Replaces the one-time setup block of the reference
 * launcher (KF94/kernel.cu:5355-5402) and `moe_init` (SF1/kernel.py:40-44).
 * Calls that use one handle must be ordered with respect to each other on the GPU (one stream,
 * or events between streams): b200moe_forward calls for up to 128 tokens share those two words.
 * Use one handle per stream for forwards that may overlap. */
int b200moe_create(const b200moe_config* cfg, b200moe_handle* out);
int b200moe_destroy(b200moe_handle h);

/* Workspace the caller must provide for a forward over T tokens (256-byte aligned).
 * Replaces `moe_ws_bytes` (SF1/kernel.py:40-44) and the Python-side `_workspace`
 * allocation (KF94/main.py:147-193, GF/main.py:68-94). */
int b200moe_workspace_bytes(b200moe_handle h, int num_tokens, size_t* bytes);
int b200moe_workspace_layout(b200moe_handle h, int num_tokens, b200moe_ws_layout* layout);

/* The operator: routing -> permute -> GEMM1+SwiGLU -> GEMM2 -> weighted combine.
 *   routing_logits      float  [T, E]
 *   routing_bias        bf16   [E] or NULL (= zeros)
 *   hidden_states       e4m3   [T, H]
 *   hidden_states_scale float  [H/128, T]
 *   gemm1_weights       e4m3   [E_local, 2I, H]    gemm1_weights_scale float [E_local, 2I/128, H/128]
 *   gemm2_weights       e4m3   [E_local, H, I]     gemm2_weights_scale float [E_local, H/128, I/128]
 *   output              bf16   [T, H]  (every row is written; rows without a local expert = 0)
 * Same argument order and meaning as the reference's C entry point
 * `extern "C" int moe_run(...)` (KF94/kernel.cu:5336-5348) and its Python operator
 * signature `run(...)` (GF/main.py:102-117, KF94/main.py:196-209). */
int b200moe_forward(b200moe_handle h,
                    const void* routing_logits, const void* routing_bias,
                    const void* hidden_states, const void* hidden_states_scale,
                    const void* gemm1_weights, const void* gemm1_weights_scale,
                    const void* gemm2_weights, const void* gemm2_weights_scale,
                    int num_tokens, int local_expert_offset, float routed_scaling_factor,
                    void* output, void* workspace, size_t workspace_bytes, void* cuda_stream);

/* Routing alone: writes int32 topk_idx[T, top_k] (global expert ids) and float
 * topk_w[T, top_k].  Replaces the reference's exported `moe_routing`
 * (goal_full_shape/opus-5/moe_fp8_fwd/<def>/moe_kernel.cu:1098-1101) and its
 * `route_topk_kernel` launch (KF94/kernel.cu:5426-5431). */
int b200moe_route(b200moe_handle h, const void* routing_logits, const void* routing_bias,
                  int num_tokens, float routed_scaling_factor,
                  int32_t* topk_idx, float* topk_w, void* cuda_stream);

/* Entry points that take topk_idx from the caller (b200moe_forward_routed, _forward_routed_slots,
 * _permute_noalloc) expect the ids of one token's row to be DISTINCT (ids < 0 or outside the local
 * range are ignored): the row buffers hold min(top_k, E_local) rows per token.  A row that repeats a
 * local expert is refused on the device: error word 5, rows beyond the capacity are not written. */

/* The expert part alone, for tokens that were routed elsewhere (expert-parallel receive
 * side): like b200moe_forward but takes topk_idx/topk_w instead of logits, and writes the
 * sum over the LOCAL experts to output [T, H]: output_kind 0 = fp32 (the sum unrounded), 1 = bf16
 * (the operator's output type: right when the local experts are all of a token's experts),
 * 2 = fp16, the form PARTIAL rows travel in between ranks (two bytes like bf16 but 11
 * significant bits: the owner adds the partial rows of up to world ranks in fp32 before the
 * single rounding to bf16, and bf16 partials cost that sum the output tolerance).
 * The reference has no expert-parallel code; this corresponds to the launcher's stages
 * after routing (KF94/kernel.cu:5436-5586). */
int b200moe_forward_routed(b200moe_handle h,
                           const int32_t* topk_idx, const float* topk_w,
                           const void* hidden_states, const void* hidden_states_scale,
                           const void* gemm1_weights, const void* gemm1_weights_scale,
                           const void* gemm2_weights, const void* gemm2_weights_scale,
                           int num_tokens, int local_expert_offset,
                           void* output, int output_kind, void* workspace, size_t workspace_bytes,
                           void* cuda_stream);

/* Expert-parallel dispatch rows.  One row on the wire carries all a receiving rank needs for one
 * token: [H fp8 bytes | H/128 fp32 scales | top_k int32 global expert ids | top_k fp32 weights],
 * padded to a multiple of 16 bytes (b200moe_ep_row_bytes), so the dispatch is one all-to-all.
 *   pack  : wire[i] = row of token send_token[i] (int64, 0 <= token < num_tokens), i < n_rows;
 *           hidden_states fp8 [T, H], hidden_states_scale float [H/128, T], topk_* [T, top_k]
 *   unpack: received wire rows -> hidden_states fp8 [n_rows, H], hidden_states_scale float
 *           [H/128, n_rows], topk_idx / topk_w [n_rows, top_k] (inputs of b200moe_forward_routed)
 * (No counterpart in the reference, which has no distributed code.) */
int b200moe_ep_row_bytes(b200moe_handle h, int* bytes);
int b200moe_ep_pack(b200moe_handle h, const void* hidden_states, const void* hidden_states_scale,
                    const int32_t* topk_idx, const float* topk_w, const long long* send_token,
                    int n_rows, int num_tokens, void* wire, void* cuda_stream);
int b200moe_ep_unpack(b200moe_handle h, const void* wire, int n_rows, void* hidden_states,
                      void* hidden_states_scale, int32_t* topk_idx, float* topk_w, void* cuda_stream);

/* The same exchange over peer memory (NVLink) instead of a library all-to-all.  Every rank owns one
 * buffer that all ranks of the node have mapped (how it is shared - symmetric memory, CUDA IPC - is
 * the host's business; this library only receives the peer addresses):
 *   flags uint32[16], zero before the first step; wire [world][cap] dispatch rows; back [world][cap][H] fp16.
 * A step on every rank, all launches on one stream, `cap` the same on all ranks, T <= cap:
 *   b200moe_ep_push          own tokens' rows stored into wire slot (my_rank, t) of every rank that owns
 *                            one of the token's experts; the slot of every other rank gets expert ids -1
 *   b200moe_ep_barrier       epoch e (strictly increasing over the life of the buffers)
 *   b200moe_ep_unpack_slots  my wire, all world*cap slots -> inputs of b200moe_forward_routed
 *   b200moe_forward_routed   over world*cap tokens, fp16 partial rows out (output_kind 2)
 *   b200moe_ep_return        result rows of present slots stored into back slot (my_rank, t) of the owner
 *   b200moe_ep_barrier       epoch e + 1
 *   b200moe_ep_combine_slots out[t] = fp32 sum, in rank order, of my back slots (r, t) over the ranks r
 *                            that own one of token t's experts; one rounding to bf16
 * peer_* are host arrays of `world` device addresses (entry r = the buffer part on rank r).
 * The barrier's wait gives up after the handle's wait limit (b200moe_set_wait_limit_ns, 2 s by
 * default) and then stores 7 into *status_word (a device int the
 * caller owns and zeroes); the step's output is invalid in that case.  Only plain stores cross
 * NVLink.  (No counterpart in the reference.) */
int b200moe_ep_push(b200moe_handle h, const void* hidden_states, const void* hidden_states_scale,
                    const int32_t* topk_idx, const float* topk_w, int num_tokens, int cap, int world,
                    int my_rank, void* const* peer_wire, void* cuda_stream);
int b200moe_ep_barrier(b200moe_handle h, void* const* peer_flags, int world, int my_rank,
                       unsigned epoch, int* status_word, void* cuda_stream);
int b200moe_ep_unpack_slots(b200moe_handle h, const void* wire, int n_slots, void* hidden_states,
                            void* hidden_states_scale, int32_t* topk_idx, float* topk_w,
                            void* cuda_stream);
int b200moe_ep_return(b200moe_handle h, const void* partial_rows_fp16, const int32_t* topk_idx_slots,
                      int cap, int world, int my_rank, void* const* peer_back, void* cuda_stream);
/* The local experts over the world*cap wire slots, read IN PLACE (no unpack copy: ids, weights, fp8 rows and
 * scales are taken from the packed rows the peers stored; absent slots carry ids -1), with b200moe_ep_return
 * folded into the last kernel: every present slot's fp16 partial row is stored straight into the owner's back
 * slot.  `wire` = this rank's [world][cap] dispatch rows (16-byte aligned).  Replaces the sequence
 * b200moe_ep_unpack_slots -> b200moe_forward_routed -> b200moe_ep_return of a step. */
int b200moe_forward_routed_slots(b200moe_handle h, const void* wire,
                                 const void* gemm1_weights, const void* gemm1_weights_scale,
                                 const void* gemm2_weights, const void* gemm2_weights_scale,
                                 int cap, int world, int my_rank, int local_expert_offset,
                                 void* const* peer_back, void* workspace, size_t workspace_bytes,
                                 void* cuda_stream);
int b200moe_ep_combine_slots(b200moe_handle h, const void* back, const int32_t* topk_idx,
                             int num_tokens, int cap, int world, void* output_bf16, void* cuda_stream);

/* Expert-parallel combine on the token's owner rank: out[t, :] = sum over the ranks r that
 * computed a share of token t (row_of[r, t] >= 0) of partial_rows[row_of[r, t], :], added in
 * fp32 in ascending rank order, rounded once to bf16.  partial_rows is the receive buffer
 * of the combine all-to-all, fp16 [n_rows, H] (b200moe_forward_routed with output_kind 2);
 * row_of is int32 [world, T].  Tokens without
 * any share get zeros.  (No counterpart in the reference, which has no distributed code.) */
int b200moe_ep_combine(b200moe_handle h, const void* partial_rows, const int32_t* row_of,
                       int world, int num_tokens, void* output_bf16, void* cuda_stream);

/* Expert-sorted row map without any workspace from the caller.  (No counterpart in the
 * reference: its launchers always receive caller-allocated workspaces.)
 *
 * Some hosts of this library cannot allocate device memory at the point where they need the
 * permutation: a serving loop that runs under a fixed memory budget with its allocator frozen
 * after start-up, a plugin called from a runtime that owns all device memory, or code that
 * sits between stream operations where a cudaMalloc would stall the device.  For them this
 * entry point does the histogram / scan / permute step (the same kernels b200moe_forward uses)
 * with its scratch -- histogram counters, tile prefix, status words and the token->row map --
 * in a fixed array inside the library image (about 330 KB per GPU that loads the library, held
 * until the process exits).  It calls no cudaMalloc/cudaFree and no allocating routine.
 *
 *   in : topk_idx int32 [T, top_k], topk_w float [T, top_k], local_expert_offset
 *   out: expert_row0 int32 [E_local + 1]   first (16-aligned) row of each local expert
 *        row_token   int32 [rows_capacity] token of each row, -1 for the padding of a segment
 *        row_w       float [rows_capacity] routing weight of each row
 *   rows_capacity must be at least b200moe_ws_layout.rows_cap for this T.
 *
 * Limits and rules: T <= B200MOE_NOALLOC_MAX_TOKENS, else B200MOE_E_TOO_LARGE.  The first call
 * on a device looks up the array's device address (once per device); make that first call
 * outside any stream capture.  All calls on a device share the one array: it is cleared at the
 * start of every call, and two calls that overlap on the GPU (different streams, no ordering
 * between them) race -- serialise them. */
int b200moe_permute_noalloc(b200moe_handle h, const int32_t* topk_idx, const float* topk_w,
                            int num_tokens, int local_expert_offset,
                            int32_t* expert_row0, int32_t* row_token, float* row_w,
                            int rows_capacity, void* cuda_stream);

/* Activation quantiser (the step before the operator): bf16 x[T, H] -> e4m3 q[T, H] and float
 * scale[H/128, T] with scale = amax/448 over each (token, 128 columns) group (1.0 for an all-zero
 * group) and q = round-to-nearest-even(x / scale): the operator's hidden_states /
 * hidden_states_scale inputs.  x 16-byte aligned, H a multiple of 128.  The reference receives
 * pre-quantised tensors from its harness (GF/moe_host.cu:100-103 checks their shapes) and has no
 * such kernel; the grouping and the amax/448 rule are those of its input contract. */
int b200moe_quantize_1x128(const void* x_bf16, int num_tokens, int hidden, void* q_e4m3,
                           float* scale_kblock_major, void* cuda_stream);

/* Synchronises the stream, reads the device error word of the last forward on this
 * workspace into *word (0 = no error) and returns B200MOE_E_KERNEL if it is non-zero.
 * The reference returns cudaGetLastError() only (KF94/kernel.cu:5681); its device waits
 * are unbounded, ours give up after a time limit and report here. */
int b200moe_status(b200moe_handle h, const void* workspace, void* cuda_stream, int* word);

/* Fused combine (off by default).  on != 0: b200moe_forward calls whose token count selects a narrow
 * token tile (b200moe_ws_layout.token_tile < 128) run without the combine launch - the GEMM2 unit
 * that delivers a token's last expert row sums the token's rows (same order, same bits as the
 * combine kernel) and stores the bf16 output; the reference fuses its combine the same way
 * (KF94/kernel.cu:3692-3708, with bf16 reductions in global memory instead of a fixed-order sum).
 * Measured slower than the separate kernel at 64 tokens; kept for hosts that count launches. */
int b200moe_set_fused_combine(b200moe_handle h, int on);

/* Token tile of the GEMMs.  0 (default): chosen from the token count - 16 tokens while an expert
 * expects about seven rows or fewer, 128 from about nine (measured crossovers on the DeepSeek-V3
 * shape), 32 in between.  16 / 32 / 64 / 128 force one kernel family for every token count (tuning
 * and tests; every size gives the same results within the operator's tolerance).  The workspace
 * size depends on the tile: query b200moe_workspace_bytes again after changing it. */
int b200moe_set_token_tile(b200moe_handle h, int tokens);

/* TMA-gathered token rows (off by default).  on != 0: with 128-token tiles GEMM1 reads its token
 * rows straight from hidden_states (or from the packed dispatch rows) with four-row TMA gathers
 * (`cp.async.bulk.tensor...tile::gather4`, as KF94/kernel.cu:932-941,3014-3056) through the
 * token-of-row table, and the activation gather copy is not launched.  Same results bit for bit;
 * measured three times slower on the GEMM (32 gathers per 128-K block from one producer thread),
 * so the copy stays the default. */
int b200moe_set_tma_gather(b200moe_handle h, int on);

/* How long a kernel of this handle waits for another RANK (the barrier flags of the peer-memory
 * exchange) before it gives up, stores its error code and returns: 2 s by default, 1 ns .. 60 s.
 * A rank that stopped between steps then costs its peers one limit, not a hang.  The waits inside
 * one kernel (shared-memory stages, TMEM buffers) keep their fixed 2 s limit.  (No counterpart in
 * the reference, whose device waits are unbounded.) */
int b200moe_set_wait_limit_ns(b200moe_handle h, unsigned long long nanoseconds);

/* Number of this library's kernels one forward over T tokens launches (a count of
 * launches, not of kernels that do useful work). */
int b200moe_launches_per_forward(b200moe_handle h, int num_tokens, int* launches);
/* The same count for b200moe_forward_routed / b200moe_forward_routed_slots over num_tokens tokens (slots). */
int b200moe_launches_routed(b200moe_handle h, int num_tokens, int* launches);

/* Optional stage timing.  enable(slots > 0) creates slots x 7 CUDA events; every forward then
 * records them around its six kernels (slot = call number modulo slots); enable(0) turns it
 * off.  read(slot) waits for that call's last event and writes six durations in
 * milliseconds: route (or count), permute, gather, gemm1, gemm2, combine.  Counterpart of
 * the reference's in-kernel time stamps and pybind timing getters
 * (goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/moe_small.cuh:55-60,
 *  kda05_reproduction_single_shape/fable-5.1/moe_fp8_fwd/t14107/moe_kernel.cu:2966-3009). */
int b200moe_profile_enable(b200moe_handle h, int slots);
int b200moe_profile_read(b200moe_handle h, int slot, float* stage_ms);

const char* b200moe_strerror(int code);
int b200moe_num_sms(void);            /* cf. `moe_num_sms`, SF1/kernel.py:40-44 */

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
