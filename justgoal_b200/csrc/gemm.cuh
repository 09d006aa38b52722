// Grouped FP8 block-scale GEMMs on tcgen05 (sm_100a), weights on the M side ("swap-AB").
//
// One UNIT = (local expert, 128 weight rows, one tile of NTOK expert-sorted token rows), full K.
//   GEMM1 (G1): D_up[128, NTOK]   = W13[e, mt*128 .. +128, :]      . A_perm[rows]^T
//               D_gate[128, NTOK] = W13[e, I + mt*128 .. +128, :]  . A_perm[rows]^T
//               epilogue: c = silu(gate) * up, per-(row, 128 columns) amax -> scale = amax/448,
//               stored as TWO e4m3 values hi = rn(c/scale), lo = rn(c/scale - hi) under one scale.
//   GEMM2 (G2): D[128, NTOK] = W2[e, mt*128 .. +128, :] . (act_hi + act_lo)[rows]^T, two MMAs per
//               K step into the same accumulator; epilogue: y[row, h] = D as fp16 (weighted by the combine).
// Block scales change every 128 K, so each 128-K block is accumulated into a fresh TMEM region
// and promoted into fp32 registers: acc += part * (token_scale[kb] * weight_scale[kb]).
// The same arithmetic is stated by the reference's tcgen05 kernels
// (kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/kernel.cu:3336,3441-3446
//  for the promotion, :3519-3584 for SwiGLU + requantisation,
//  goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/moe_small.cuh:1-16 for the swap-AB orientation);
// unlike them the SwiGLU output keeps a second e4m3 term, because a single e4m3 per element
// does not meet an absolute/relative tolerance of 1e-2 against the unquantised definition.
//
// Schedule: K is cut into GROUPS of KPB 128-K blocks (one TMEM hand-off per group).  The kernel is
// persistent.  Units are numbered so that the token tiles of one (expert, row tiles) are adjacent.  Every CTA
// first runs floor(U / grid) WHOLE units, round-robin (CTAs that run at the same time work on adjacent units, so
// a weight tile shared by several token tiles comes from HBM once).  The remaining U mod grid units are cut
// along K into CHUNKS of a few K blocks, and the CTAs CLAIM those chunks one at a time from a counter in global
// memory: SMs do not stream at the same rate under full load, and a CTA that finishes early simply takes more
// chunks (with equal static shares the finish times of the CTAs spread by 7-10 % of the kernel).  A chunked
// unit is finished by the CTA that runs its LAST chunk: every other chunk stores its fp32 partial to its own slot
// and counts itself in with a release; the finisher waits (bounded) for that count, adds the slots in CHUNK order
// (a fixed order: results are bit-identical from run to run) and runs the epilogue.  Chunks are claimed in order, so
// the finisher only ever waits for chunks that were claimed before its own - no cycle of waiting CTAs can form.
// Inside a CTA the producer claims the work and hands it to the MMA and promotion warps through a small queue
// in shared memory.
//
// Small token counts (GemmParams::routed): GEMM1 follows a front-end kernel that routes, permutes and gathers in one
// launch.  GEMM1's CTAs are resident while it runs; when it announces the routing result they build the expert tables
// themselves and the producer streams the first weight tiles before the front end has completed - only the token
// side of those stages waits for it.  Optionally (GemmParams::fuse_out) GEMM2's epilogue also does the combine.
//
// Warp roles: warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane) + TMEM owner,
// warps 2-3 idle (they complete the first warpgroup so register re-allocation is legal; with the fused combine
// they write the zero rows of tokens that have no pair on this rank),
// warps 4.. = promotion/epilogue (4 or 8 warps; warp % 4 selects the TMEM lane quarter).
// Every wait is bounded (common.cuh); no TMA load uses cluster multicast.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.cuh"
#include "permute.cuh"

namespace b200moe {

struct GemmParams {
    int* status;
    const int* counts;
    const int* expert_row0;
    const int* tile_prefix;
    int num_local;
    int KB;               // K blocks of 128
    int n_mtiles;         // 128-row weight tiles per expert that one unit family covers
    int rows_per_expert;  // rows of the weight matrix per expert (2I for GEMM1, H for GEMM2)
    int gate_offset;      // row offset of the unit's second weight tile (GEMM1: I, the gate half; GEMM2: 128)
    int unit_rows;        // weight rows one unit advances by (GEMM1: 128, GEMM2: 256)
    int valid_rows;       // GEMM2: output columns H (the last unit's second tile may lie beyond)
    int scale_rows;       // weight-scale rows per expert (rows_per_expert / 128)
    const float* w_scale; // [E_local, scale_rows, KB]
    const float* b_scale; // [KB, rows_cap] token-side scales
    int rows_cap;
    uint8_t* act_hi; uint8_t* act_lo; float* act_scale; int I;   // GEMM1 outputs
    const float* row_w; __half* y; int H;                         // GEMM2 output: y[row, h] = O[row, h] as fp16 (the routing
                                                                  // weight is applied by the combine, in fp32)
    int evict_first_weights;
    int* sk_count;        // [4 * gridDim.x + 4] zero at launch: [4 * ut] promotion warps of chunked unit ut that have stored
                          // their partial sums, [4 * gridDim.x] the chunk claim counter
    float* sk_partial;    // [gridDim.x * chunks per unit] slots of SLOT_FLOATS floats: slot (ut, chunk)
    long long* klog;      // [4][KLOG_N]: CTA 0's clock at its first KLOG_N K blocks: TMA issue, data seen by the
                          // MMA warp, group seen by the promotion warps, group folded (hand-back)
    long long* trace;     // [gridDim.x][TRACE_SLOTS]: slot 0 = %globaltimer at entry, others = SM clocks since entry
    // GEMM1 after the fused front end (small token counts), else null: the front end sets *routed to 1 when the routing
    // result of all tokens is visible.  The CTAs then build the expert tables themselves from topk_idx (the same
    // histogram and scan as the front end) and the producer streams the first weight tiles while the front end still
    // permutes and gathers; the token rows are loaded after the front end has completed.
    const int* routed;
    const int32_t* topk_idx;      // [n_pairs] global expert ids (pair_stride == top_k on this path)
    int n_pairs, local_offset;
    // GEMM1 with 128-token tiles reading the token rows straight from the caller's activations (no gather copy), else
    // g4_row_token == null: tm_b0 is then a map over the activations with one-row boxes, a stage's token tile is 32
    // four-row TMA gathers through row_token, and the promotion threads read their token's block scales from the
    // caller's scale tensor: scale(token, kb) = g4_scale[token * g4_tok_stride + kb * g4_kb_stride].
    const int32_t* g4_row_token;
    const float* g4_scale;
    int g4_tok_stride;    // in floats
    int g4_T;
    int ts_stride;        // tokens-on-M tiles: floats between a row's token scales of consecutive K blocks (rows_cap for the
                          // gathered copy, the caller's K-block stride when g4_row_token is set); K blocks * ts_stride < 2^31
    // GEMM2 with the combine fused into its epilogue (narrow token tiles of the operator's own forward), else
    // fuse_out == null.  tok_count[t * n_mtiles + mt] (zero at launch) counts the units that have stored the columns
    // [256 mt, 256 mt + 256) of one of token t's rows; the warp that brings it to the number of the token's local
    // pairs adds those rows up (permute.cuh, combine_token_slab) and writes the bf16 output.  Tokens without a local
    // pair get their zero row from the otherwise idle warps 2-3.
    __nv_bfloat16* fuse_out;
    int* tok_count;
    const int32_t* row_token; const int32_t* pair_row; const int32_t* c_topk;
    int c_stride, top_k, T, c_local_offset;
    int ablate;           // timing experiments only, builds with -DB200MOE_ENABLE_ABLATE (results are wrong when
                          // non-zero): 1 = issue no MMA, 2 = narrow-tile promotion skips tcgen05.ld/FMA, 4 = producer
                          // skips the token-side loads, 8 = the MMA warp consumes the stages alone
};

template <int NTOK, bool G1>
struct GemmCfg {
    static constexpr int NA = 2;                          // weight tiles per stage (GEMM1: up + gate rows; GEMM2: two row tiles)
    static constexpr int NB = G1 ? 1 : 2;                 // token tiles per stage
    static constexpr int A_BYTES = 128 * 128;
    static constexpr int B_BYTES = NTOK * 128;
    static constexpr int SC_OFF = NA * A_BYTES + NB * B_BYTES;
    static constexpr int STAGE_BYTES = SC_OFF + 1024;
    // tokens-on-M tiles read their (per-thread scalar) token scale straight from global memory, one K
    // block ahead; the others get the tile's NTOK scales copied into the stage
    static constexpr bool SCALES_IN_STAGE = NTOK != 128;
    static constexpr int TX_BYTES = NA * A_BYTES + NB * B_BYTES + (SCALES_IN_STAGE ? NTOK * 4 : 0);
    static constexpr int EMPTY_COUNT = 1 + (SCALES_IN_STAGE ? (NTOK >= 64 ? 8 : 4) : 0);   // MMA commit (+ promotion warps)
    static constexpr int STAGES_RAW = (208 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int NACCUM = 2;                      // one accumulator per weight tile
    // Orientation.  Narrow tiles put the weights on the MMA's M side (few tokens = few TMEM columns).
    // A full 128-token tile puts the TOKENS on M (TMEM lanes) and each weight tile's 128 rows on N:
    // a promotion thread then owns one token row, its scale is one scalar per K block (no per-column
    // scale loads or multiplies in the fold) and it stores 64 contiguous output columns as vectors.
    static constexpr bool TOK_ON_M = NTOK == 128;
    // Dependent MMAs into one accumulator serialise on the tensor pipe's latency, which dominates
    // for narrow token tiles; the MMAs of one K block are therefore spread over NSPLIT independent
    // partial accumulators (GEMM1: even/odd K step; GEMM2: hi / lo operand) that the promotion adds.
    static constexpr int NSPLIT = NTOK <= 32 ? 2 : 1;
    static constexpr int CPB = NACCUM * NSPLIT * NTOK;     // TMEM columns per K block
    static constexpr int KPB = (128 / CPB) < 1 ? 1 : (128 / CPB);
    static constexpr int BUFCOLS = KPB * CPB;               // TMEM columns per hand-off buffer
    static constexpr int NACC = (512 / BUFCOLS) > 4 ? 4 : (512 / BUFCOLS);
    static constexpr int TMEM_COLS = NACC * BUFCOLS;
    // Measured and dropped: handing a GEMM1 K block over as two 128-column halves (N = 128 MMAs, four
    // half-buffers in flight) - the N = 128 MMAs compete with the TMA fills for shared-memory bandwidth
    // and a K block took 750 ns instead of 570 ns.
    static constexpr int NTB = NACC;                        // TMEM hand-off barriers per direction
    // promotion warps: 4 (one per TMEM lane quarter) for narrow tiles, 8 (two column groups) from 64 tokens.
    // With tokens on M the fold of a 128 x 256 fp32 block takes ~630 cycles: two tcgen05.ld round trips of
    // 2 x 32 columns per thread (128 accumulator registers leave 64 for staging); 16 warps do not fit the
    // register pool with a deeper staging and measured no gain with the same depth.
    static constexpr int NPW = NTOK >= 64 ? 8 : 4;
    static constexpr int NGRP = NPW / 4;                   // column groups (a group = 4 warps = all 128 lanes)
    static constexpr int NPT = 32 * NPW;                   // promotion threads
    static_assert(EMPTY_COUNT == 1 + (SCALES_IN_STAGE ? NPW : 0), "stage release count");
    static constexpr int NC = NTOK / (NPW / 4);            // token columns per promotion thread
    static constexpr int CH = (NACCUM * NC > 64) ? 16 : (NC < 32 ? NC : 32);   // columns per tcgen05.ld
    static constexpr int NTHREADS = 128 + NPT;
    // Register re-allocation (setmaxnreg).  The increase BLOCKS until the CTA's own pool holds enough
    // registers, and that pool is only what the control warps gave back from the allocation the CTA
    // was launched with - so the numbers below must add up exactly (checked here and, against the
    // register count ptxas actually chose, by the host before the first launch).
    static constexpr bool REALLOC_REGS = NPW >= 8;
    static constexpr int LAUNCH_REGS = (65536 / NTHREADS) / 8 * 8;          // what __launch_bounds__(NTHREADS, 1) yields
    static constexpr int CTRL_REGS = 40;      // measured: 24/240, 40/232, 56/224 and 72/216 run within 1 % of each other
    static constexpr int PROMO_REGS = 232;
    static_assert(!REALLOC_REGS || 128 * CTRL_REGS + NPT * PROMO_REGS <= NTHREADS * LAUNCH_REGS,
                  "setmaxnreg.inc would wait forever: the control warps do not release enough registers");
    static_assert(!REALLOC_REGS || (CTRL_REGS <= LAUNCH_REGS && PROMO_REGS >= LAUNCH_REGS), "setmaxnreg direction");
    // narrow tiles: the promotion warps copy a group's token scales into registers as soon as the
    // stage has landed and release the stage at once, instead of holding it until the group is folded
    static constexpr bool EARLY_SCALES = KPB * NC <= 32 && NPW < 16;
    static constexpr int SLOT_FLOATS = NACCUM * NC * NPT;  // = NACCUM * 128 * NTOK
    // SMALLEST number of K blocks per claimed chunk of a split unit (the producer enlarges the chunks when there are
    // many left-over units: about two chunks per CTA).  A chunk streams CHUNK_BLOCKS * 32 KB of weights and leaves
    // 1 KB * NTOK of partial sums: at NTOK / 8 blocks the partial sums are one eighth of the chunk's traffic for every
    // tile width, and a narrow tile's last few units spread over many CTAs (decode GEMM2: four left-over units become
    // 32 chunks instead of 8)
    static constexpr int CHUNK_BLOCKS = NTOK / 8;
    static constexpr int CHUNK_GROUPS = (CHUNK_BLOCKS / KPB) < 1 ? 1 : (CHUNK_BLOCKS / KPB);
    // GEMM1 with narrow tiles has few, long units (decode: 256 units of 3.7 MB for 148 CTAs): there the units left
    // over after the whole rounds are cut into EQUAL contiguous ranges, one per CTA, processed first (claimed
    // chunks measured 30 % slower there: every CTA finishes units it has to collect six partial sums for, late in
    // the kernel).  Everywhere else the left-over units are cut into chunks that the CTAs claim as they go.
    static constexpr bool STATIC_TAIL = G1 && NTOK <= 32;
    static constexpr int WQ = 4;                           // depth of the in-CTA work queue
    static constexpr int BAR_BYTES = 320;                  // mbarriers + TMEM address word
    static constexpr int TABLE_INTS = 3 * (MAX_LOCAL + 1);
    static constexpr int RED_BYTES = NPW * NC * 4;
    static constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * STAGE_BYTES + BAR_BYTES + WQ * 32 /*work queue*/ +
                                      TABLE_INTS * 4 + RED_BYTES + 32 + 16 + 512 /*token ids of the producer's unit, 16-byte aligned*/;
    static_assert(NTOK % 16 == 0 && NTOK >= 16 && NTOK <= 128, "token tile");
    static_assert(TMEM_COLS >= 32 && TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "tmem");
    static_assert(STAGES >= KPB + 1, "a group must fit the stage ring with room to prefetch");
    static_assert(NC % CH == 0 && (CH == 8 || CH == 16 || CH == 32), "chunking");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};


// Per-CTA time line (SM clock cycles since kernel entry) written by whichever thread reaches the point.
enum : int { TR_ENTRY = 0, TR_PROLOGUE = 1, TR_TMA_FIRST = 2, TR_TMA_LAST = 3, TR_MMA_FIRST = 4, TR_MMA_LAST = 5,
             TR_PROMO_FIRST = 6, TR_PROMO_LAST = 7, TR_PARTIAL = 8, TR_REDUCED = 9, TR_EPILOGUE = 10, TR_EXIT = 11,
             TRACE_SLOTS = 16, KLOG_N = 64 };

struct Unit { int e, mt, tt, row0, nvalid; };

__device__ __forceinline__ bool decode_unit(int u, int n_mtiles, int num_local, int ntok, const int* s_tiles,
                                            const int* s_row0, const int* s_cnt, Unit& o) {
    const int q = u / n_mtiles;
    int lo = 0, hi = num_local;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_tiles[mid] <= q) lo = mid; else hi = mid - 1;
    }
    if (lo >= num_local) return false;
    const int ntt = s_tiles[lo + 1] - s_tiles[lo];
    if (ntt <= 0) return false;
    const int ul = u - s_tiles[lo] * n_mtiles;
    o.e = lo;
    o.mt = ul / ntt;
    o.tt = ul - o.mt * ntt;
    o.row0 = s_row0[lo] + o.tt * ntok;
    o.nvalid = min(ntok, s_cnt[lo] - o.tt * ntok);
    return o.mt < n_mtiles && o.nvalid > 0;
}

// One piece of work: unit u, K groups [gb, ge).  kind WK_WHOLE: the whole unit.  WK_PART: a piece of split unit ut
// that does not end the unit - its partial sum goes to slot `slot`.  WK_FINISH: the piece that ends split unit ut -
// it waits for `nwait` other pieces, adds the slots slot .. slot + nwait - 1 in that order and runs the epilogue.
// u < 0 ends the list.
enum : int { WK_WHOLE = 0, WK_PART = 1, WK_FINISH = 2 };
struct WorkItem { int u, gb, ge, kind, ut, slot, nwait; };

// CTA that owns flat index x when `total` indices are cut into `parts` equal contiguous ranges (part c starts at
// c * total / parts)
// (32-bit arithmetic: total < #SMs * K groups, parts <= #SMs, so every product stays far below 2^31)
__device__ __forceinline__ int range_start(int c, int total, int parts) { return (int)((unsigned)c * (unsigned)total / (unsigned)parts); }
__device__ __forceinline__ int range_owner(int x, int total, int parts) {
    int c = (int)((unsigned)x * (unsigned)parts / (unsigned)total);
    while (c + 1 < parts && range_start(c + 1, total, parts) <= x) ++c;
    while (c > 0 && range_start(c, total, parts) > x) --c;
    return c;
}

// Chunks per chunked unit
__host__ __device__ inline int chunks_per_unit(int KB, int kpb, int chunk_groups) {
    const int NG = (KB + kpb - 1) / kpb;
    return (NG + chunk_groups - 1) / chunk_groups;
}

__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// N consecutive columns of one expert-output row, rounded to fp16 (the per-pair rows the combine weighs and adds
// up in fp32), as 32-byte stores
template <int N>
__device__ __forceinline__ void store_y_row(__half* dst, const float* acc) {
    static_assert(N % 16 == 0, "16 columns per store");
#pragma unroll
    for (int i = 0; i < N; i += 16) {
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __half2 h = __floats2half2_rn(acc[i + 2 * j], acc[i + 2 * j + 1]);
            pk[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        st_global_v8(dst + i, pk[0], pk[1], pk[2], pk[3], pk[4], pk[5], pk[6], pk[7]);
    }
}

template <int N>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, float* v) {
    uint32_t r[N];
    if constexpr (N == 8) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
            : "r"(taddr) : "memory");
    } else if constexpr (N == 16) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr) : "memory");
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr) : "memory");
    }
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = __uint_as_float(r[i]);
}

// G4 (GEMM1 with 128-token tiles only): the token rows come straight from the caller's activations by four-row TMA
// gathers (GemmParams::g4_row_token); a separate instantiation, so the plain kernel's code is unchanged by it.
template <int NTOK, bool G1, bool G4 = false>
__global__ void __launch_bounds__(GemmCfg<NTOK, G1>::NTHREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_b0,
            const __grid_constant__ CUtensorMap tm_b1, const GemmParams p) {
    using C = GemmCfg<NTOK, G1>;
    static_assert(!G4 || (C::TOK_ON_M && G1), "TMA-gathered token rows: GEMM1 with 128-token tiles");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tail = smem + C::STAGES * C::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);     // full[S], empty[S], tfull[NTB], tempty[NTB], red[4], all, wq_full[WQ], wq_empty[WQ]
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tail + C::BAR_BYTES - 8);
    int* s_wq = reinterpret_cast<int*>(tail + C::BAR_BYTES);          // [WQ][8] work items (WorkItem + padding)
    int* s_tiles = s_wq + C::WQ * 8;
    int* s_row0 = s_tiles + (MAX_LOCAL + 1);
    int* s_cnt = s_row0 + (MAX_LOCAL + 1);
    uint32_t* s_red = reinterpret_cast<uint32_t*>(s_cnt + (MAX_LOCAL + 1));
    int* s_flag = reinterpret_cast<int*>(s_red + C::NPW * C::NC);   // 8 ints: [0] routing flag seen (early schedule), [4..5] the producer's chunk sizing
    // [128] token of every row of the producer's unit, 16-byte aligned (read and written as int4)
    int* s_g4 = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(s_flag + 8) + 15) & ~uintptr_t(15));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef B200MOE_ENABLE_ABLATE
    const int kAblate = p.ablate;      // timing experiments (build with -DB200MOE_ENABLE_ABLATE)
#else
    constexpr int kAblate = 0;         // the ablation branches compile away in the product build
#endif
    const long long t_entry = clock64();
    long long* const trace = p.trace ? p.trace + (size_t)blockIdx.x * TRACE_SLOTS : nullptr;
    auto stamp = [&](int slot) { if (trace) trace[slot] = clock64() - t_entry; };
#ifdef B200MOE_ENABLE_KLOG
    long long* const klog = (p.klog && blockIdx.x == 0) ? p.klog : nullptr;
    auto klog_put = [&](int row, int n) { if (klog && n < KLOG_N) klog[row * KLOG_N + n] = clock64() - t_entry; };
#else
    auto klog_put = [&](int, int) {};      // the per-K-block log is a build option (-DB200MOE_ENABLE_KLOG)
#endif
    if (trace && threadIdx.x == 0) trace[TR_ENTRY] = (long long)globaltimer_ns();
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * C::STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * C::STAGES;
    const uint32_t bar_tempty = bar_tfull + 8 * C::NTB;
    const uint32_t bar_red = bar_tempty + 8 * C::NTB;    // one per column group: its 4 warps meet here (bounded)
    const uint32_t bar_all = bar_red + 8 * 4;             // all promotion warps meet here (tokens-on-M epilogue)
    const uint32_t bar_wqfull = bar_all + 8;              // work queue: the producer has published item n
    const uint32_t bar_wqempty = bar_wqfull + 8 * C::WQ;  // ... and the MMA warp and every promotion warp have read it
    static_assert(8 * (2 * C::STAGES + 2 * C::NTB + 5 + 2 * C::WQ) <= C::BAR_BYTES - 8, "barrier area");

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, C::EMPTY_COUNT); }
        for (int b = 0; b < C::NTB; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, C::NPW); }
        for (int g = 0; g < 4; ++g) mbar_init(bar_red + 8 * g, 4);
        mbar_init(bar_all, C::NPW);
        for (int w = 0; w < C::WQ; ++w) { mbar_init(bar_wqfull + 8 * w, 1); mbar_init(bar_wqempty + 8 * w, 1 + C::NPW); }
        mbar_fence_init();
        tma_prefetch_desc(&tm_w); tma_prefetch_desc(&tm_b0);
        if (!G1) tma_prefetch_desc(&tm_b1);
    }
    if (warp == 1) { tmem_alloc(smem_u32(s_tmem), C::TMEM_COLS); tmem_relinquish(); }
    // everything above touches only this CTA's shared memory and TMEM; the tables below are
    // written by the kernels before this one
    bool early = false;             // tables built here, before the previous kernel has completed
    if (G1 && p.routed) {
        if (threadIdx.x == 0) {
            int seen = 0;
            const unsigned long long t0 = globaltimer_ns();
            for (uint32_t it = 1;; ++it) {
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.routed) : "memory");
                if (seen) break;
                if ((it & 0xFFu) == 0 && globaltimer_ns() - t0 > WAIT_LIMIT_NS) break;     // fall back to the tables
            }
            *s_flag = seen;
        }
        for (int i = threadIdx.x; i <= p.num_local; i += blockDim.x) s_cnt[i] = 0;
        __syncthreads();
        early = *s_flag != 0;
    }
    if (early) {
        for (int i = threadIdx.x; i < p.n_pairs; i += blockDim.x) {
            const int le = __ldcg(p.topk_idx + i) - p.local_offset;
            if (le >= 0 && le < p.num_local) atomicAdd(&s_cnt[le], 1);
        }
        __syncthreads();
        if (warp == 0) scan_counts(s_cnt, p.num_local, NTOK, s_row0, s_tiles, nullptr, lane);
    } else {
        pdl_wait();
        for (int i = threadIdx.x; i <= p.num_local; i += blockDim.x) {
            s_tiles[i] = p.tile_prefix[i];
            s_row0[i] = p.expert_row0[i];
            s_cnt[i] = i < p.num_local ? p.counts[i] : 0;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // early schedule: the producer (lane 0 of warp 0, the only lane of that warp that works) waits after its first
    // weight loads; the other warps wait here, before anything that reads the token rows.  The condition is uniform
    // over a warp on purpose: lanes of one warp that wait would hold the producer lane at their reconvergence point.
    if (early && warp != 0) pdl_wait();
    pdl_launch();
    const uint32_t tmem_base = *s_tmem;
    const uint32_t smem_base = smem_u32(smem);
    if (threadIdx.x == 0) stamp(TR_PROLOGUE);

    // Schedule (see the head of this file): q whole units per CTA, then chunks of the remaining units claimed
    // from a global counter.
    const int NG = (p.KB + C::KPB - 1) / C::KPB;
    const int total_units = s_tiles[p.num_local] * p.n_mtiles;
    const int sched_q = total_units / (int)gridDim.x;              // whole units per CTA
    const int sched_U0 = sched_q * (int)gridDim.x;                 // first chunked unit
    int* const claim = p.sk_count + 4 * (int)gridDim.x;

    // Consumer side of the work queue: item n sits in slot n % WQ.  WARP: every lane of the calling warp waits and
    // reads, lane 0 then tells the producer that the warp has its copy; otherwise the caller is a single thread.
    // false = list ended or a wait gave up.
    auto wq_fetch = [&](int n, WorkItem& w, bool& ok, bool whole_warp) -> bool {
        const int slot = n % C::WQ;
        if (!mbar_wait(bar_wqfull + 8 * slot, (uint32_t)(n / C::WQ) & 1u, p.status, ERR_WAIT_GROUP)) { ok = false; return false; }
        const volatile int* q = s_wq + slot * 8;
        w.u = q[0]; w.gb = q[1]; w.ge = q[2]; w.kind = q[3]; w.ut = q[4]; w.slot = q[5]; w.nwait = q[6];
        if (whole_warp) __syncwarp();
        if (!whole_warp || lane == 0) mbar_arrive(bar_wqempty + 8 * slot);
        return w.u >= 0;
    };

    if (warp < 4) {
    // ================================================================ control warpgroup
    if (C::REALLOC_REGS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::CTRL_REGS));
    }
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            // Chunk size of the left-over units: about two chunks per CTA in total, never below CHUNK_GROUPS groups.  A few
            // left-over units are cut finely so that every CTA gets a piece; many are cut into two or three chunks each
            // (every chunk but a unit's last costs a partial-sum slot written and read, and its finisher a wait).
            {
                int chunk_groups = C::CHUNK_GROUPS;
                if (total_units > sched_U0) {
                    const int per_unit = (2 * (int)gridDim.x + (total_units - sched_U0) - 1) / (total_units - sched_U0);
                    chunk_groups = max(chunk_groups, (NG + per_unit - 1) / per_unit);
                }
                s_flag[4] = chunk_groups;
                s_flag[5] = (NG + chunk_groups - 1) / chunk_groups;           // chunks per chunked unit
            }
            // (kept in shared memory between the rare claims rather than in registers for the whole loop)
            volatile int* const s_sched = s_flag + 4;
            const int total_chunks = (total_units - sched_U0) * s_sched[1];
            int stage = 0; uint32_t phase = 0;
            bool ok = true, issued = false;
            bool waited = !early;               // early schedule: has this thread waited for the previous kernel yet
            int nk = 0;
            // the producer decides what this CTA does next and publishes it to the other roles
            int n_item = 0, n_whole = 0;
            auto publish = [&](const WorkItem& w) -> bool {
                const int slot = n_item % C::WQ;
                if (!mbar_wait(bar_wqempty + 8 * slot, ((uint32_t)(n_item / C::WQ) & 1u) ^ 1u, p.status, ERR_WAIT_GROUP)) return false;
                volatile int* q = s_wq + slot * 8;
                q[0] = w.u; q[1] = w.gb; q[2] = w.ge; q[3] = w.kind; q[4] = w.ut; q[5] = w.slot; q[6] = w.nwait;
                mbar_arrive(bar_wqfull + 8 * slot);          // release: the item is visible to whoever sees the phase flip
                ++n_item;
                return true;
            };
            // static tail: this CTA's range [t_lo, t_hi) of the flat (left-over unit, K group) space, as per-unit pieces;
            // pieces that do not end their unit come first, then the one that does (it waits for pieces other CTAs
            // run first, so no chain of waiting CTAs can form), then whole units
            const int tail_units = total_units - sched_U0;
            const int flat = tail_units * NG;
            const int parts = flat < (int)gridDim.x ? (flat > 0 ? flat : 1) : (int)gridDim.x;
            const bool has_tail = C::STATIC_TAIL && flat > 0 && (int)blockIdx.x < parts;
            const int t_lo = has_tail ? range_start((int)blockIdx.x, flat, parts) : 0;
            const int t_hi = has_tail ? range_start((int)blockIdx.x + 1, flat, parts) : 0;
            int st_pass = has_tail ? 0 : 3, st_ut = t_lo / NG;
            while (ok) {
                WorkItem wi;
                wi.kind = WK_WHOLE; wi.ut = -1; wi.slot = 0; wi.nwait = 0;
                bool have = false;
                while (st_pass < 3 && !have) {
                    const int ut_last = (t_hi - 1) / NG;
                    while (st_ut <= ut_last && !have) {
                        const int ut = st_ut++;
                        const int u_lo = ut * NG;
                        const int gb = max(t_lo, u_lo) - u_lo, ge = min(t_hi, u_lo + NG) - u_lo;
                        const int kind = (gb == 0 && ge == NG) ? WK_WHOLE : (ge == NG ? WK_FINISH : WK_PART);
                        const int want = st_pass == 0 ? WK_PART : (st_pass == 1 ? WK_FINISH : WK_WHOLE);
                        if (kind != want) continue;
                        wi.u = sched_U0 + ut; wi.gb = gb; wi.ge = ge; wi.kind = kind; wi.ut = ut;
                        if (kind == WK_PART) {
                            wi.slot = (int)blockIdx.x;              // a CTA stores at most one partial: its own slot
                        } else if (kind == WK_FINISH) {
                            wi.slot = range_owner(u_lo, flat, parts);          // CTA of the unit's first piece
                            wi.nwait = (int)blockIdx.x - wi.slot;
                            if (wi.nwait == 0) wi.kind = WK_WHOLE;             // cannot happen (gb > 0), kept for safety
                        }
                        have = true;
                    }
                    if (!have) { ++st_pass; st_ut = t_lo / NG; }
                }
                if (have) {
                } else if (n_whole < sched_q) {
                    wi.u = n_whole * (int)gridDim.x + (int)blockIdx.x; wi.gb = 0; wi.ge = NG;
                    ++n_whole;
                } else {
                    const int c = (!C::STATIC_TAIL && total_chunks > 0) ? atomicAdd(claim, 1) : total_chunks;
                    if (c >= total_chunks) { wi.u = -1; wi.gb = wi.ge = 0; publish(wi); break; }
                    const int chunk_groups = s_sched[0], CPU_ = s_sched[1];
                    wi.ut = c / CPU_;
                    const int ci = c - wi.ut * CPU_;
                    wi.u = sched_U0 + wi.ut;
                    wi.gb = ci * chunk_groups; wi.ge = min(NG, wi.gb + chunk_groups);
                    if (CPU_ > 1) {
                        // chunks are claimed in order: the one that ends the unit is claimed last and finishes it
                        wi.kind = ci + 1 < CPU_ ? WK_PART : WK_FINISH;
                        wi.slot = wi.kind == WK_PART ? wi.ut * CPU_ + ci : wi.ut * CPU_;
                        wi.nwait = CPU_ - 1;
                    }
                }
                if (!publish(wi)) { ok = false; break; }
                const int u = wi.u, gb = wi.gb, ge = wi.ge;
                Unit un;
                if (!decode_unit(u, p.n_mtiles, p.num_local, NTOK, s_tiles, s_row0, s_cnt, un)) {
                    atomicCAS(p.status, 0, ERR_BAD_SCHEDULE); ok = false; break;
                }
                const int wrow = un.e * p.rows_per_expert + un.mt * p.unit_rows;
                const int kb_end = min(p.KB, ge * C::KPB);
                auto load_weights = [&](int s_, int kb) {
                    const uint32_t st = smem_base + s_ * C::STAGE_BYTES;
                    const uint32_t full = bar_full + 8 * s_;
                    mbar_arrive_expect_tx(full, (kAblate & 4) ? C::NA * C::A_BYTES : C::TX_BYTES);
                    if (p.evict_first_weights) {
                        tma_load_2d_hint(st, &tm_w, kb * 128, wrow, full, pol);
                        tma_load_2d_hint(st + C::A_BYTES, &tm_w, kb * 128, wrow + p.gate_offset, full, pol);
                    } else {
                        tma_load_2d(st, &tm_w, kb * 128, wrow, full);
                        tma_load_2d(st + C::A_BYTES, &tm_w, kb * 128, wrow + p.gate_offset, full);
                    }
                };
                constexpr bool g4 = G4;
                if (g4) {
                    // tokens of the unit's 128 rows (segments start at multiples of 16 rows: 16-byte loads; rows past
                    // the expert's own hold other tokens, -1 or stale values - their results are never stored, and a
                    // row index outside the tensor reads zeros)
                    const int4* src = reinterpret_cast<const int4*>(p.g4_row_token + un.row0);
#pragma unroll 1
                    for (int i = 0; i < 32; ++i) reinterpret_cast<int4*>(s_g4)[i] = __ldg(src + i);
                }
                auto load_tokens = [&](int s_, int kb) {
                    if (kAblate & 4) return;
                    const uint32_t st = smem_base + s_ * C::STAGE_BYTES;
                    const uint32_t full = bar_full + 8 * s_;
                    if (g4) {
#pragma unroll 1
                        for (int g = 0; g < 32; ++g) {
                            const int4 t = reinterpret_cast<const int4*>(s_g4)[g];
                            tma_gather4_2d(st + C::NA * C::A_BYTES + g * 512, &tm_b0, kb * 128, t.x, t.y, t.z, t.w, full);
                        }
                        return;
                    }
                    tma_load_2d(st + C::NA * C::A_BYTES, &tm_b0, kb * 128, un.row0, full);
                    if (!G1) tma_load_2d(st + C::NA * C::A_BYTES + C::B_BYTES, &tm_b1, kb * 128, un.row0, full);
                    if (C::SCALES_IN_STAGE)
                        bulk_load(st + C::SC_OFF, p.b_scale + (size_t)kb * p.rows_cap + un.row0, NTOK * 4, full);
                };
                int kb_first = gb * C::KPB;
                if (G1 && !waited) {
                    // early schedule, first item: the (empty) stage ring takes weight tiles while the front end still
                    // permutes and gathers, then the wait for it, then the token side of the same stages
                    const int npre = min(C::STAGES, kb_end - kb_first);
                    for (int i = 0; i < npre; ++i) load_weights(i, kb_first + i);
                    stamp(TR_TMA_FIRST); issued = true;
                    pdl_wait();
                    waited = true;
                    for (int i = 0; i < npre; ++i) { load_tokens(i, kb_first + i); klog_put(0, nk++); }
                    kb_first += npre;
                    stage = npre;
                    if (stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
                for (int kb = kb_first; kb < kb_end; ++kb) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, p.status, ERR_WAIT_SMEM_EMPTY)) { ok = false; break; }
                    load_weights(stage, kb);
                    load_tokens(stage, kb);
                    if (!issued) { stamp(TR_TMA_FIRST); issued = true; }
                    klog_put(0, nk++);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            stamp(TR_TMA_LAST);
            if (!ok) {
                // gave up: end the list for the other roles (if the queue still moves), then give copies that are
                // still in flight time to land before the CTA's shared memory goes away
                WorkItem end_; end_.u = -1; end_.gb = end_.ge = 0; end_.kind = WK_WHOLE; end_.ut = -1; end_.slot = end_.nwait = 0;
                publish(end_);
                for (int i = 0; i < 64; ++i) __nanosleep(10000);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f8(128, NTOK);
            int stage = 0; uint32_t phase = 0;
            int ab = 0; uint32_t aphase = 0;
            bool ok = true, seen = false;
            int nk = 0;
            int n_item = 0;
            WorkItem wi;
            while (ok && wq_fetch(n_item++, wi, ok, false)) {
                const int gb = wi.gb, ge = wi.ge;
                if (kAblate & 8) {      // timing experiment: consume stages directly, no MMA, no TMEM hand-off
                    const int kb_end = min(p.KB, ge * C::KPB);
                    for (int kb = gb * C::KPB; kb < kb_end && ok; ++kb) {
                        if (!mbar_wait(bar_full + 8 * stage, phase, p.status, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
                        for (int i = 0; i < C::EMPTY_COUNT; ++i) mbar_arrive(bar_empty + 8 * stage);
                        if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                    }
                    continue;
                }
                for (int grp = gb; grp < ge && ok; ++grp) {
                    if (!mbar_wait(bar_tempty + 8 * ab, aphase ^ 1, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
                    const int nj = min(C::KPB, p.KB - grp * C::KPB);
                    for (int j = 0; j < nj; ++j) {
                        klog_put(6, nk);
                        if (!mbar_wait(bar_full + 8 * stage, phase, p.status, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
                        if (!seen) { stamp(TR_MMA_FIRST); seen = true; }
                        klog_put(1, nk++);
                        tc_fence_after();
                        const uint32_t st = smem_base + stage * C::STAGE_BYTES;
                        const uint32_t d = tmem_base + ab * C::BUFCOLS + j * C::CPB;
                        // mm(D, weight tile, token tile): operand order follows the orientation
                        auto mm = [&](uint32_t dd, uint64_t wdesc, uint64_t tdesc, uint32_t accum) {
                            if (C::TOK_ON_M) umma_f8(dd, tdesc, wdesc, idesc, accum);
                            else umma_f8(dd, wdesc, tdesc, idesc, accum);
                        };
                        if (kAblate & 1) {
                        } else if (C::TOK_ON_M) {
                            // The two weight tiles of a stage are adjacent in shared memory (256 rows of 128 B)
                            // and so are their accumulators in TMEM: ONE N = 256 MMA per 32-byte K step covers
                            // both.  (An N = 128 MMA reads 8 KB of operands per 64 tensor-pipe cycles, all the
                            // shared-memory bandwidth of the SM: measured 75 cycles alone, slower beside TMA fills.)
                            constexpr uint32_t idesc2 = make_idesc_f8(128, 256);
                            const uint64_t w = make_smem_desc(st);
                            const uint64_t th = make_smem_desc(st + 2 * C::A_BYTES);
#pragma unroll
                            for (int k = 0; k < 4; ++k) umma_f8(d, th + 2 * k, w + 2 * k, idesc2, k > 0);
                            if (!G1) {      // GEMM2: the low-order term of the activation accumulates on top
                                const uint64_t tl = make_smem_desc(st + 2 * C::A_BYTES + C::B_BYTES);
#pragma unroll
                                for (int k = 0; k < 4; ++k) umma_f8(d, tl + 2 * k, w + 2 * k, idesc2, 1u);
                            }
                        } else if (G1) {
                            const uint64_t a_up = make_smem_desc(st);
                            const uint64_t a_gate = make_smem_desc(st + C::A_BYTES);
                            const uint64_t b = make_smem_desc(st + 2 * C::A_BYTES);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const int sp = k % C::NSPLIT;
                                mm(d + sp * NTOK, a_up + 2 * k, b + 2 * k, k >= C::NSPLIT);
                                mm(d + (C::NSPLIT + sp) * NTOK, a_gate + 2 * k, b + 2 * k, k >= C::NSPLIT);
                            }
                        } else {
                            const uint64_t a0 = make_smem_desc(st);
                            const uint64_t a1 = make_smem_desc(st + C::A_BYTES);
                            const uint64_t bh = make_smem_desc(st + 2 * C::A_BYTES);
                            const uint64_t bl = make_smem_desc(st + 2 * C::A_BYTES + C::B_BYTES);
                            // tile t, operand half o (hi, lo): partial accumulator o when NSPLIT == 2, else both into one
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                mm(d, a0 + 2 * k, bh + 2 * k, k > 0);
                                mm(d + C::NSPLIT * NTOK, a1 + 2 * k, bh + 2 * k, k > 0);
                            }
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                mm(d + (C::NSPLIT - 1) * NTOK, a0 + 2 * k, bl + 2 * k, C::NSPLIT == 1 || k > 0);
                                mm(d + (2 * C::NSPLIT - 1) * NTOK, a1 + 2 * k, bl + 2 * k, C::NSPLIT == 1 || k > 0);
                            }
                        }
                        umma_commit(bar_empty + 8 * stage);
                        if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                    }
                    if (!ok) break;
                    umma_commit(bar_tfull + 8 * ab);
                    if (++ab == C::NACC) { ab = 0; aphase ^= 1; }
                }
            }
            stamp(TR_MMA_LAST);
        }
        __syncwarp();
    } else if (!G1 && p.fuse_out) {
        // ------------------------------------------------------------ warps 2-3, fused combine: zero rows of the
        // tokens that have no pair on this rank (nobody else writes them)
        for (int t = (int)blockIdx.x * 2 + (warp - 2); t < p.T; t += (int)gridDim.x * 2) {
            bool local = false;
            if (lane < p.top_k) {
                const int le = __ldg(p.c_topk + (size_t)t * p.c_stride + lane) - p.c_local_offset;
                local = le >= 0 && le < p.num_local;
            }
            if (__any_sync(0xFFFFFFFFu, local)) continue;
            uint4* o = reinterpret_cast<uint4*>(p.fuse_out + (size_t)t * p.H);
            for (int i = lane; i < p.H / 8; i += 32) o[i] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    } else {
        // ------------------------------------------------------------ promotion + epilogue
        if (C::REALLOC_REGS) {
            asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::PROMO_REGS));
        }
        const int pw = warp - 4;
        const int quarter = warp & 3;                  // TMEM lanes [32*quarter, +32)
        const int grp_id = pw >> 2;                    // column group (0 when NPW == 4)
        const int c0 = grp_id * C::NC;
        const int m = quarter * 32 + lane;             // weight row inside the tile
        const int ptid = threadIdx.x - 128;
        const uint32_t tlane = (uint32_t)(quarter * 32) << 16;
        const uint32_t my_red = bar_red + 8 * grp_id;
        int stage = 0; uint32_t phase = 0;
        int ab = 0; uint32_t aphase = 0;
        uint32_t rphase = 0, allphase = 0;
        bool ok = true, seen = false;
        int ng = 0, nu = 0;
        float acc[C::NACCUM][C::NC];

        // the 4 warps of one column group meet (bounded); false = gave up
        auto group_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(my_red);
            const bool r = mbar_wait(my_red, rphase, p.status, ERR_WAIT_GROUP);
            rphase ^= 1;
            return r;
        };

        // all promotion warps meet (bounded); false = gave up
        auto all_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_all);
            const bool r = mbar_wait(bar_all, allphase, p.status, ERR_WAIT_GROUP);
            allphase ^= 1;
            return r;
        };

        int n_item = 0;
        WorkItem wi;
        while (ok && wq_fetch(n_item++, wi, ok, true)) {
            if (kAblate & 8) continue;          // timing experiment: the MMA warp consumes the stages alone
            const int u = wi.u, gb = wi.gb, ge = wi.ge;
            Unit un;
            if (!decode_unit(u, p.n_mtiles, p.num_local, NTOK, s_tiles, s_row0, s_cnt, un)) break;
#pragma unroll
            for (int a = 0; a < C::NACCUM; ++a)
#pragma unroll
                for (int i = 0; i < C::NC; ++i) acc[a][i] = 0.f;
            // weight-scale rows of the unit's two tiles (the second one of GEMM2's last unit may not exist)
            const int srow0 = un.mt * (p.unit_rows >> 7);
            const int srow1 = min(srow0 + (p.gate_offset >> 7), p.scale_rows - 1);
            const float* ws0 = p.w_scale + ((size_t)un.e * p.scale_rows + srow0) * p.KB;
            const float* ws1 = p.w_scale + ((size_t)un.e * p.scale_rows + srow1) * p.KB;

            // weight scales of a group are fetched one group ahead, so their global-load latency
            // never sits between the TMEM hand-off and the first FMA
            float swn[C::KPB][C::NACCUM];
#pragma unroll
            for (int j = 0; j < C::KPB; ++j) {
                const int kb = min(gb * C::KPB + j, p.KB - 1);
                swn[j][0] = __ldg(ws0 + kb);
                swn[j][1] = __ldg(ws1 + kb);
            }
            // tokens-on-M: this thread's token scale, also one K block ahead (KPB == 1 there)
            const float* tsp = p.b_scale + (size_t)un.row0 + m;
            if (G4) {
                const int tok = __ldg(p.g4_row_token + un.row0 + m);
                tsp = p.g4_scale + (tok >= 0 && tok < p.g4_T ? (size_t)tok * (unsigned)p.g4_tok_stride : 0);   // any finite scale for a row of zeros
            }
            float stokn = C::TOK_ON_M ? __ldcg(tsp + (size_t)min(gb * C::KPB, p.KB - 1) * (G4 ? p.ts_stride : p.rows_cap)) : 0.f;
            for (int grp = gb; grp < ge; ++grp) {
                const int kb0 = grp * C::KPB;
                const int nj = min(C::KPB, p.KB - kb0);
                float sw[C::KPB][C::NACCUM];
#pragma unroll
                for (int j = 0; j < C::KPB; ++j) {
                    sw[j][0] = swn[j][0]; sw[j][1] = swn[j][1];
                    const int kb = min(kb0 + C::KPB + j, p.KB - 1);
                    swn[j][0] = __ldg(ws0 + kb);
                    swn[j][1] = __ldg(ws1 + kb);
                }
                const float stok_cur = stokn;
                if (C::TOK_ON_M) stokn = __ldcg(tsp + (size_t)min(kb0 + 1, p.KB - 1) * (G4 ? p.ts_stride : p.rows_cap));
                const int st0 = stage;
                float scr[C::EARLY_SCALES ? C::KPB : 1][C::EARLY_SCALES ? C::NC : 1];
                if (C::EARLY_SCALES && !(kAblate & 2)) {
#pragma unroll
                    for (int j = 0; j < C::KPB; ++j) {
                        if (j < nj) {
                            int sj = st0 + j; if (sj >= C::STAGES) sj -= C::STAGES;
                            const uint32_t ph = (st0 + j >= C::STAGES) ? (phase ^ 1) : phase;
                            if (!mbar_wait(bar_full + 8 * sj, ph, p.status, ERR_WAIT_SMEM_FULL)) ok = false;
                            const float* scp = reinterpret_cast<const float*>(smem + sj * C::STAGE_BYTES + C::SC_OFF) + c0;
#pragma unroll
                            for (int i = 0; i < C::NC; i += 4) {
                                const float4 s4 = *reinterpret_cast<const float4*>(scp + i);
                                scr[j][i] = s4.x; scr[j][i + 1] = s4.y; scr[j][i + 2] = s4.z; scr[j][i + 3] = s4.w;
                            }
                        }
                    }
                    if (!ok) break;
                    __syncwarp();
                    if (lane == 0) {
                        for (int j = 0; j < nj; ++j) {
                            int sj = st0 + j; if (sj >= C::STAGES) sj -= C::STAGES;
                            mbar_arrive(bar_empty + 8 * sj);
                        }
                    }
                }
                if (!mbar_wait(bar_tfull + 8 * ab, aphase, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
                if (ptid == 0 && !seen) { stamp(TR_PROMO_FIRST); seen = true; }
                if (ptid == 0) klog_put(2, ng);
                tc_fence_after();
                const uint32_t tbuf = tmem_base + tlane + ab * C::BUFCOLS + c0;

                // flattened chunk list (K block, column chunk, accumulator, partial); the tcgen05.ld of
                // chunk k+1 is in flight while chunk k is folded into the accumulators
                constexpr int NCH = C::NC / C::CH;
                constexpr int NK = C::TOK_ON_M ? 0 : C::KPB * NCH * C::NACCUM * C::NSPLIT;
                if constexpr (C::TOK_ON_M) {
                    // Tokens on M: this thread's row is one token, so a K block folds with ONE scalar per
                    // weight tile.  The block is read as 32-column chunks, two tcgen05.ld in flight per
                    // wait (a wait covers every outstanding load, so depth comes from issuing in pairs).
                    constexpr int QC = 32, QPA = C::NC / QC, NQ = C::NACCUM * QPA;
                    static_assert(C::NC % QC == 0 && NQ % 2 == 0, "tokens-on-M chunking");
                    float stg[2][QC];
                    auto qaddr = [&](int q) { return tbuf + (q / QPA) * NTOK + (q % QPA) * QC; };
                    auto qfold = [&](int q, const float* v) {
                        const int a = q / QPA;
                        const float sx = stok_cur * sw[0][a];
                        const float2 s2 = make_float2(sx, sx);
                        float* ac = &acc[a][(q % QPA) * QC];
#pragma unroll
                        for (int i = 0; i < QC; i += 2) {
                            const float2 r0 = __ffma2_rn(make_float2(v[i], v[i + 1]), s2, make_float2(ac[i], ac[i + 1]));
                            ac[i] = r0.x; ac[i + 1] = r0.y;
                        }
                    };
                    // the buffer goes back to the MMA warp as soon as its last tcgen05.ld has
                    // completed; the FMAs of the last chunks run after the release
                    auto release = [&]() {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tempty + 8 * ab);
                    };
                    {
                        // Scheduling fence.  `never` is 0, but ptxas cannot know: with the fold inside a real branch it
                        // does not pull the fold's TMEM loads and FMAs up across the hand-off wait above, and the
                        // kernel measures 3 % faster (prefill GEMM1 414 against 466 us with stage events, results
                        // bit-identical; a plain compiler barrier does not have the effect).  Re-measure when the
                        // fold changes: `python bench.py --workload prefill` with and without the branch.
                        int never;
                        asm volatile("mov.u32 %0, 0;" : "=r"(never));
                        if (never) {
                            release();
                        } else {
                        tmem_ld_chunk<QC>(qaddr(0), stg[0]);
                        tmem_ld_chunk<QC>(qaddr(1), stg[1]);
#pragma unroll
                        for (int q = 0; q < NQ; q += 2) {
                            tmem_wait_ld();
                            if (q + 2 >= NQ) release();
                            qfold(q, stg[0]);
                            if (q + 2 < NQ) tmem_ld_chunk<QC>(qaddr(q + 2), stg[0]);
                            qfold(q + 1, stg[1]);
                            if (q + 3 < NQ) tmem_ld_chunk<QC>(qaddr(q + 3), stg[1]);
                        }
                        }
                    }
                }
                float part[2][C::CH];
                if (!C::TOK_ON_M && !(kAblate & 2)) tmem_ld_chunk<C::CH>(tbuf, part[0]);
#pragma unroll
                for (int k = 0; k < NK; ++k) {
                    const int sp = k % C::NSPLIT;
                    const int a = (k / C::NSPLIT) % C::NACCUM;
                    const int ch = (k / (C::NSPLIT * C::NACCUM)) % NCH;
                    const int j = k / (C::NSPLIT * C::NACCUM * NCH);
                    if (j < nj && !(kAblate & 2)) {
                        tmem_wait_ld();
                        if (k + 1 < NK) {
                            const int sp1 = (k + 1) % C::NSPLIT;
                            const int a1 = ((k + 1) / C::NSPLIT) % C::NACCUM;
                            const int ch1 = ((k + 1) / (C::NSPLIT * C::NACCUM)) % NCH;
                            const int j1 = (k + 1) / (C::NSPLIT * C::NACCUM * NCH);
                            if (j1 < nj)
                                tmem_ld_chunk<C::CH>(tbuf + j1 * C::CPB + (a1 * C::NSPLIT + sp1) * NTOK + ch1 * C::CH,
                                                     part[(k + 1) & 1]);
                        }
                        const float swa = sw[j][a];
                        if (C::EARLY_SCALES) {
#pragma unroll
                            for (int i = 0; i < C::CH; i += 2) {
                                const float2 mm = __fmul2_rn(make_float2(scr[j][ch * C::CH + i], scr[j][ch * C::CH + i + 1]),
                                                             make_float2(swa, swa));
                                float* ac = &acc[a][ch * C::CH + i];
                                const float2 r0 = __ffma2_rn(make_float2(part[k & 1][i], part[k & 1][i + 1]), mm,
                                                             make_float2(ac[0], ac[1]));
                                ac[0] = r0.x; ac[1] = r0.y;
                            }
                        } else {
                            int sj = st0 + j; if (sj >= C::STAGES) sj -= C::STAGES;
                            if (C::SCALES_IN_STAGE && ch == 0 && a == 0 && sp == 0) {
                                // token scales of this K block arrived with the stage's transaction barrier
                                const uint32_t ph = (st0 + j >= C::STAGES) ? (phase ^ 1) : phase;
                                if (!mbar_wait(bar_full + 8 * sj, ph, p.status, ERR_WAIT_SMEM_FULL)) ok = false;
                            }
                            {
                                const float* scp = reinterpret_cast<const float*>(smem + sj * C::STAGE_BYTES + C::SC_OFF) + c0 + ch * C::CH;
#pragma unroll
                                for (int i = 0; i < C::CH; i += 4) {
                                    const float4 s4 = *reinterpret_cast<const float4*>(scp + i);
                                    const float2 m0 = __fmul2_rn(make_float2(s4.x, s4.y), make_float2(swa, swa));
                                    const float2 m1 = __fmul2_rn(make_float2(s4.z, s4.w), make_float2(swa, swa));
                                    float* ac = &acc[a][ch * C::CH + i];
                                    const float2 r0 = __ffma2_rn(make_float2(part[k & 1][i], part[k & 1][i + 1]), m0, make_float2(ac[0], ac[1]));
                                    const float2 r1 = __ffma2_rn(make_float2(part[k & 1][i + 2], part[k & 1][i + 3]), m1, make_float2(ac[2], ac[3]));
                                    ac[0] = r0.x; ac[1] = r0.y; ac[2] = r1.x; ac[3] = r1.y;
                                }
                            }
                        }
                    }
                }
                if (!ok) break;
                // all tcgen05.ld of this buffer have completed (the last wait above) and all scale reads are done
                if (!C::TOK_ON_M) {
                    tc_fence_before();
                    __syncwarp();
                }
                if (!C::TOK_ON_M && lane == 0) {
                    mbar_arrive(bar_tempty + 8 * ab);
                    if (C::SCALES_IN_STAGE && (!C::EARLY_SCALES || (kAblate & 2))) {
                        for (int j = 0; j < nj; ++j) {
                            int sj = st0 + j; if (sj >= C::STAGES) sj -= C::STAGES;
                            mbar_arrive(bar_empty + 8 * sj);
                        }
                    }
                }
                if (ptid == 0) klog_put(3, ng++);
                stage += nj;
                if (stage >= C::STAGES) { stage -= C::STAGES; phase ^= 1; }
                if (++ab == C::NACC) { ab = 0; aphase ^= 1; }
            }
            if (!ok) break;
            if (ptid == 0) stamp(TR_PROMO_LAST);

            if (wi.kind != WK_WHOLE) {
                // ---- piece of a split unit.  The unit is finished by the CTA that runs the piece that ends it.  Every
                // other piece only stores its partial sums and counts its warps in with a release - no meeting of
                // the warps, no answer to wait for.
                int* const arrived = p.sk_count + wi.ut * 4;
                if (wi.kind == WK_PART) {
                    float* slot = p.sk_partial + (size_t)wi.slot * C::SLOT_FLOATS;
#pragma unroll
                    for (int a = 0; a < C::NACCUM; ++a)
#pragma unroll
                        for (int i = 0; i < C::NC; ++i) __stcg(slot + (size_t)(a * C::NC + i) * C::NPT + ptid, acc[a][i]);
                    __syncwarp();        // orders the lanes' stores before lane 0's release below
                    if (lane == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(arrived) : "memory");
                    if (ptid == 0) stamp(TR_PARTIAL);
                    continue;
                }
                // the piece that ends the unit: wait (bounded) until the warps of all other pieces have counted in, then
                // add their partial sums in K order on top of this piece's own - a fixed order, whoever was quick or slow
                const int n_other = wi.nwait;
                const float* const slots = p.sk_partial + (size_t)wi.slot * C::SLOT_FLOATS;
                {
                    const int want = n_other * C::NPW;
                    bool here = true;
                    if (lane == 0) {
                        const unsigned long long t0 = globaltimer_ns();
                        for (uint32_t it = 1;; ++it) {
                            int v;
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(arrived) : "memory");
                            if (v >= want) break;
                            if ((it & 0xFFu) == 0 && globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                                atomicCAS(p.status, 0, ERR_WAIT_CHUNKS); here = false; break;
                            }
                        }
                    }
                    here = __shfl_sync(0xFFFFFFFFu, here, 0);
                    if (!here) { ok = false; break; }
                }
                auto slot_of = [&](int c) -> const float* { return slots + (size_t)c * C::SLOT_FLOATS + ptid; };
                if constexpr (C::NACCUM * C::NC <= 32) {
                    // narrow tiles: the next chunk's slot is in flight while this one is added (same fixed order)
                    float nxt[C::NACCUM * C::NC];
                    const float* src = slot_of(0);
#pragma unroll
                    for (int k = 0; k < C::NACCUM * C::NC; ++k) nxt[k] = __ldcg(src + (size_t)k * C::NPT);
                    for (int c = 0; c < n_other; ++c) {
                        float cur[C::NACCUM * C::NC];
#pragma unroll
                        for (int k = 0; k < C::NACCUM * C::NC; ++k) cur[k] = nxt[k];
                        if (c + 1 < n_other) {
                            src = slot_of(c + 1);
#pragma unroll
                            for (int k = 0; k < C::NACCUM * C::NC; ++k) nxt[k] = __ldcg(src + (size_t)k * C::NPT);
                        }
#pragma unroll
                        for (int a = 0; a < C::NACCUM; ++a)
#pragma unroll
                            for (int i = 0; i < C::NC; ++i) acc[a][i] += cur[a * C::NC + i];
                    }
                } else {
                    for (int c = 0; c < n_other; ++c) {
                        const float* src = slot_of(c);
#pragma unroll
                        for (int a = 0; a < C::NACCUM; ++a)
#pragma unroll
                            for (int i = 0; i < C::NC; ++i) acc[a][i] += __ldcg(src + (size_t)(a * C::NC + i) * C::NPT);
                    }
                }
            }

            if (ptid == 0) { stamp(TR_REDUCED); klog_put(4, nu); }
            if (C::TOK_ON_M && G1) {
                // this thread: token row m, NC consecutive columns j of the 128-wide block -> SwiGLU, amax over
                // the block (own columns, then the other column groups' threads of the same row), two e4m3
                // terms, 16-byte stores
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < C::NC; ++i) {
                    const float v = silu_f(acc[1][i]) * acc[0][i];
                    acc[0][i] = v;
                    amax = fmaxf(amax, fabsf(v));
                }
                float* redf = reinterpret_cast<float*>(s_red);            // [NGRP][128]
                redf[grp_id * 128 + m] = amax;
                if (!all_sync()) { ok = false; break; }
#pragma unroll
                for (int g2 = 0; g2 < C::NGRP; ++g2) amax = fmaxf(amax, redf[g2 * 128 + m]);
                if (!all_sync()) { ok = false; break; }                   // redf is reused by the next unit
                const float scale = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
                const float inv = amax > 0.f ? 448.0f / amax : 0.f;
                if (m < un.nvalid) {
                    const size_t row = (size_t)(un.row0 + m);
                    uint8_t* dhi = p.act_hi + row * p.I + (size_t)un.mt * 128 + c0;
                    uint8_t* dlo = p.act_lo + row * p.I + (size_t)un.mt * 128 + c0;
#pragma unroll
                    for (int v8 = 0; v8 < C::NC / 32; ++v8) {
                        uint32_t wh[8], wl[8];
#pragma unroll
                        for (int w4 = 0; w4 < 8; ++w4) {
                            const int i = v8 * 32 + w4 * 4;
                            const float q0 = acc[0][i] * inv, q1 = acc[0][i + 1] * inv;
                            const float q2 = acc[0][i + 2] * inv, q3 = acc[0][i + 3] * inv;
                            const uint16_t h01 = f32x2_to_e4m3x2(q0, q1), h23 = f32x2_to_e4m3x2(q2, q3);
                            const float2 f01 = e4m3x2_to_f32x2(h01), f23 = e4m3x2_to_f32x2(h23);
                            const uint16_t l01 = f32x2_to_e4m3x2(q0 - f01.x, q1 - f01.y);
                            const uint16_t l23 = f32x2_to_e4m3x2(q2 - f23.x, q3 - f23.y);
                            wh[w4] = (uint32_t)h01 | ((uint32_t)h23 << 16);
                            wl[w4] = (uint32_t)l01 | ((uint32_t)l23 << 16);
                        }
                        st_global_v8(dhi + v8 * 32, wh[0], wh[1], wh[2], wh[3], wh[4], wh[5], wh[6], wh[7]);
                        st_global_v8(dlo + v8 * 32, wl[0], wl[1], wl[2], wl[3], wl[4], wl[5], wl[6], wl[7]);
                    }
                    if (grp_id == 0) p.act_scale[(size_t)un.mt * p.rows_cap + row] = scale;
                }
            } else if (C::TOK_ON_M) {
                // 64 consecutive output columns of this thread's row per accumulator, as 256-bit stores.
                // A unit's rows drain at ~32 B per cycle per SM whatever the pattern (a shuffle transpose that
                // made every lane quad write 128 contiguous bytes was measured equal), so they leave as fp16.
                if (m < un.nvalid) {
                    const size_t row = (size_t)(un.row0 + m);
#pragma unroll
                    for (int a = 0; a < C::NACCUM; ++a) {
                        const int col0 = un.mt * p.unit_rows + a * p.gate_offset + c0;
                        if (col0 < p.valid_rows) store_y_row<C::NC>(p.y + row * p.H + col0, acc[a]);
                    }
                }
            } else if (G1) {
                // SwiGLU, then amax over the 128 rows of the tile for every token column
                uint32_t* red = s_red + pw * C::NC;
#pragma unroll
                for (int i = 0; i < C::NC; ++i) {
                    const float v = silu_f(acc[1][i]) * acc[0][i];
                    acc[0][i] = v;
                    const uint32_t wm = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(fabsf(v)));
                    if (lane == 0) red[i] = wm;
                }
                if (!group_sync()) { ok = false; break; }
                const uint32_t* rg = s_red + grp_id * 4 * C::NC;
                const size_t col = (size_t)un.mt * 128 + m;
#pragma unroll
                for (int i = 0; i < C::NC; i += 2) {
                    float sc2[2], inv2[2];
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t a4 = max(max(rg[i + j], rg[C::NC + i + j]), max(rg[2 * C::NC + i + j], rg[3 * C::NC + i + j]));
                        const float amax = __uint_as_float(a4);
                        sc2[j] = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
                        inv2[j] = amax > 0.f ? 448.0f / amax : 0.f;
                    }
                    const float q0 = acc[0][i] * inv2[0], q1 = acc[0][i + 1] * inv2[1];
                    const uint16_t hi = f32x2_to_e4m3x2(q0, q1);
                    const float2 hf = e4m3x2_to_f32x2(hi);
                    const uint16_t lo = f32x2_to_e4m3x2(q0 - hf.x, q1 - hf.y);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int c = c0 + i + j;
                        if (c < un.nvalid) {
                            const size_t row = (size_t)(un.row0 + c);
                            p.act_hi[row * p.I + col] = (uint8_t)(j ? (hi >> 8) : (hi & 0xFF));
                            p.act_lo[row * p.I + col] = (uint8_t)(j ? (lo >> 8) : (lo & 0xFF));
                            if (quarter == 0 && lane == ((i + j) & 31))
                                p.act_scale[(size_t)un.mt * p.rows_cap + row] = sc2[j];
                        }
                    }
                }
                if (!group_sync()) { ok = false; break; }          // s_red is reused by the next unit
            } else {
                const int col0 = un.mt * p.unit_rows + m;
                const bool second = col0 + p.gate_offset < p.valid_rows;
#pragma unroll
                for (int i = 0; i < C::NC; ++i) {
                    const int c = c0 + i;
                    if (c < un.nvalid) {
                        const size_t row = (size_t)(un.row0 + c);
                        p.y[row * p.H + col0] = __float2half_rn(acc[0][i]);
                        if (second) p.y[row * p.H + col0 + p.gate_offset] = __float2half_rn(acc[1][i]);
                    }
                }
                if (p.fuse_out) {
                    // Fused combine.  The four warps of this column group have now stored all 256 columns of the
                    // group's NC rows: fence, meet, then count the unit in for every row's token (the group's rows
                    // are dealt over its warps and lanes, one atomic per row, all in flight together).
                    __threadfence();
                    if (!group_sync()) { ok = false; break; }
                    const int c = c0 + quarter + 4 * lane;
                    const bool mine = lane < C::NC / 4 && c < un.nvalid;
                    int t = -1;
                    bool last = false;
                    if (mine) {
                        t = __ldg(p.row_token + un.row0 + c);
                        int need = 0;
                        for (int k = 0; k < p.top_k; ++k) {
                            const int le = __ldg(p.c_topk + (size_t)t * p.c_stride + k) - p.c_local_offset;
                            need += le >= 0 && le < p.num_local;
                        }
                        last = atomicAdd(p.tok_count + (size_t)t * p.n_mtiles + un.mt, 1) == need - 1;
                    }
                    unsigned todo = __ballot_sync(0xFFFFFFFFu, last);
                    if (todo) __threadfence();          // the other units' rows, counted in before this one, are visible
                    while (todo) {
                        const int srcl = __ffs(todo) - 1;
                        todo &= todo - 1;
                        const int tt = __shfl_sync(0xFFFFFFFFu, t, srcl);
                        combine_token_slab(p.y, p.c_topk, p.pair_row, p.row_w, p.fuse_out, tt, p.H, p.top_k, p.c_stride,
                                           p.c_local_offset, p.num_local, un.mt * p.unit_rows, lane);
                    }
                }
            }
            if (ptid == 0) klog_put(5, nu++);
        }
    }

    if (warp >= 4 && threadIdx.x == 128) stamp(TR_EPILOGUE);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
    if (threadIdx.x == 0) stamp(TR_EXIT);
}

}  // namespace b200moe
