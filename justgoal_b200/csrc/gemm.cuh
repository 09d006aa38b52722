// Grouped FP8 block-scale GEMMs on tcgen05 (sm_100a), weights on the M side ("swap-AB").
//
// One UNIT = (local expert, 128 weight rows, one tile of NTOK expert-sorted token rows), full K.
//   GEMM1 (G1): D_up[128, NTOK]   = W13[e, mt*128 .. +128, :]      . A_perm[rows]^T
//               D_gate[128, NTOK] = W13[e, I + mt*128 .. +128, :]  . A_perm[rows]^T
//               epilogue: c = silu(gate) * up, per-(row, 128 columns) amax -> scale = amax/448,
//               stored as TWO e4m3 values hi = rn(c/scale), lo = rn(c/scale - hi) under one scale.
//   GEMM2 (G2): D[128, NTOK] = W2[e, mt*128 .. +128, :] . (act_hi + act_lo)[rows]^T, two MMAs per
//               K step into the same accumulator; epilogue: y[row, h] = row_w[row] * D.
// Block scales change every 128 K, so each 128-K block is accumulated into a fresh TMEM buffer
// and promoted into fp32 registers: acc += part * (token_scale[kb] * weight_scale[kb]).
// The same arithmetic is stated by the reference's tcgen05 kernels
// (kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/kernel.cu:3336,3441-3446
//  for the promotion, :3519-3584 for SwiGLU + requantisation,
//  goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/moe_small.cuh:1-16 for the swap-AB orientation);
// unlike them the SwiGLU output keeps a second e4m3 term, because a single e4m3 per element
// does not meet an absolute/relative tolerance of 1e-2 against the unquantised definition.
//
// Warp roles: warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane) + TMEM owner,
// warps 2.. = promotion/epilogue (4 or 8 warps; warp % 4 selects the TMEM lane quarter).
// Every wait is bounded (common.cuh); no TMA load uses cluster multicast.
#pragma once
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
    int gate_offset;      // GEMM1: row offset of the gate half (I)
    int scale_rows;       // weight-scale rows per expert (rows_per_expert / 128)
    const float* w_scale; // [E_local, scale_rows, KB]
    const float* b_scale; // [KB, rows_cap] token-side scales
    int rows_cap;
    uint8_t* act_hi; uint8_t* act_lo; float* act_scale; int I;   // GEMM1 outputs
    const float* row_w; float* y; int H;                          // GEMM2 outputs
    int evict_first_weights;
};

template <int NTOK, bool G1>
struct GemmCfg {
    static constexpr int NA = G1 ? 2 : 1;                 // weight tiles per stage
    static constexpr int NB = G1 ? 1 : 2;                 // token tiles per stage
    static constexpr int A_BYTES = 128 * 128;
    static constexpr int B_BYTES = NTOK * 128;
    static constexpr int SC_OFF = NA * A_BYTES + NB * B_BYTES;
    static constexpr int STAGE_BYTES = SC_OFF + 1024;
    static constexpr int TX_BYTES = NA * A_BYTES + NB * B_BYTES + NTOK * 4;
    static constexpr int STAGES_RAW = (212 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int CPB = (G1 ? 2 : 1) * NTOK;        // TMEM columns per accumulator buffer
    static constexpr int NACC = (512 / CPB) > 4 ? 4 : (512 / CPB);
    static constexpr int TMEM_COLS = NACC * CPB;
    static constexpr int NPW = CPB > 128 ? 8 : 4;          // promotion warps
    static constexpr int NC = NTOK / (NPW / 4);            // token columns per promotion thread
    static constexpr int NACCUM = G1 ? 2 : 1;
    static constexpr int NTHREADS = 64 + 32 * NPW;
    static constexpr int TABLE_INTS = 3 * (MAX_LOCAL + 1);
    static constexpr int RED_BYTES = NPW * NC * 4;
    static constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * STAGE_BYTES + 256 /*barriers*/ +
                                      TABLE_INTS * 4 + RED_BYTES;
    static_assert(NTOK % 16 == 0 && NTOK >= 16 && NTOK <= 128, "token tile");
    static_assert(TMEM_COLS >= 32 && TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "tmem");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};

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

__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int NTOK, bool G1>
__global__ void __launch_bounds__(GemmCfg<NTOK, G1>::NTHREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_b0,
            const __grid_constant__ CUtensorMap tm_b1, const GemmParams p) {
    using C = GemmCfg<NTOK, G1>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tail = smem + C::STAGES * C::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);             // full[S], empty[S], tfull[NACC], tempty[NACC], red[2]
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tail + 240);
    int* s_tiles = reinterpret_cast<int*>(tail + 256);
    int* s_row0 = s_tiles + (MAX_LOCAL + 1);
    int* s_cnt = s_row0 + (MAX_LOCAL + 1);
    uint32_t* s_red = reinterpret_cast<uint32_t*>(s_cnt + (MAX_LOCAL + 1));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * C::STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * C::STAGES;
    const uint32_t bar_tempty = bar_tfull + 8 * C::NACC;
    const uint32_t bar_red = bar_tempty + 8 * C::NACC;    // one per column group: 4 warps meet here (bounded)
    static_assert(8 * (2 * C::STAGES + 2 * C::NACC + 2) <= 240, "barrier area");

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1 + C::NPW); }
        for (int b = 0; b < C::NACC; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, C::NPW); }
        mbar_init(bar_red, 4); mbar_init(bar_red + 8, 4);
        mbar_fence_init();
        tma_prefetch_desc(&tm_w); tma_prefetch_desc(&tm_b0);
        if (!G1) tma_prefetch_desc(&tm_b1);
    }
    if (warp == 1) { tmem_alloc(smem_u32(s_tmem), C::TMEM_COLS); tmem_relinquish(); }
    for (int i = threadIdx.x; i <= p.num_local; i += blockDim.x) {
        s_tiles[i] = p.tile_prefix[i];
        s_row0[i] = p.expert_row0[i];
        s_cnt[i] = i < p.num_local ? p.counts[i] : 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    const int total_units = s_tiles[p.num_local] * p.n_mtiles;
    const uint32_t smem_base = smem_u32(smem);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                Unit un;
                if (!decode_unit(u, p.n_mtiles, p.num_local, NTOK, s_tiles, s_row0, s_cnt, un)) {
                    atomicCAS(p.status, 0, ERR_BAD_SCHEDULE); break;
                }
                const int wrow = un.e * p.rows_per_expert + un.mt * 128;
                for (int kb = 0; kb < p.KB; ++kb) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, p.status, ERR_WAIT_SMEM_EMPTY)) { ok = false; break; }
                    const uint32_t st = smem_base + stage * C::STAGE_BYTES;
                    const uint32_t full = bar_full + 8 * stage;
                    mbar_arrive_expect_tx(full, C::TX_BYTES);
                    if (p.evict_first_weights) {
                        tma_load_2d_hint(st, &tm_w, kb * 128, wrow, full, pol);
                        if (G1) tma_load_2d_hint(st + C::A_BYTES, &tm_w, kb * 128, wrow + p.gate_offset, full, pol);
                    } else {
                        tma_load_2d(st, &tm_w, kb * 128, wrow, full);
                        if (G1) tma_load_2d(st + C::A_BYTES, &tm_w, kb * 128, wrow + p.gate_offset, full);
                    }
                    tma_load_2d(st + C::NA * C::A_BYTES, &tm_b0, kb * 128, un.row0, full);
                    if (!G1) tma_load_2d(st + C::NA * C::A_BYTES + C::B_BYTES, &tm_b1, kb * 128, un.row0, full);
                    bulk_load(st + C::SC_OFF, p.b_scale + (size_t)kb * p.rows_cap + un.row0, NTOK * 4, full);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // give copies that are still in flight time to land before the CTA's shared memory goes away
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
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                for (int kb = 0; kb < p.KB; ++kb) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, p.status, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
                    if (!mbar_wait(bar_tempty + 8 * ab, aphase ^ 1, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t st = smem_base + stage * C::STAGE_BYTES;
                    const uint32_t d = tmem_base + ab * C::CPB;
                    if (G1) {
                        const uint64_t a_up = make_smem_desc(st);
                        const uint64_t a_gate = make_smem_desc(st + C::A_BYTES);
                        const uint64_t b = make_smem_desc(st + 2 * C::A_BYTES);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            umma_f8(d, a_up + 2 * k, b + 2 * k, idesc, k > 0);
                            umma_f8(d + NTOK, a_gate + 2 * k, b + 2 * k, idesc, k > 0);
                        }
                    } else {
                        const uint64_t a = make_smem_desc(st);
                        const uint64_t bh = make_smem_desc(st + C::A_BYTES);
                        const uint64_t bl = make_smem_desc(st + C::A_BYTES + C::B_BYTES);
#pragma unroll
                        for (int k = 0; k < 4; ++k) umma_f8(d, a + 2 * k, bh + 2 * k, idesc, k > 0);
#pragma unroll
                        for (int k = 0; k < 4; ++k) umma_f8(d, a + 2 * k, bl + 2 * k, idesc, 1);
                    }
                    umma_commit(bar_empty + 8 * stage);
                    umma_commit(bar_tfull + 8 * ab);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                    if (++ab == C::NACC) { ab = 0; aphase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ promotion + epilogue
        const int pw = warp - 2;
        const int quarter = warp & 3;                  // TMEM lanes [32*quarter, +32)
        const int grp = pw >> 2;                       // column group (0 when NPW == 4)
        const int c0 = grp * C::NC;
        const int m = quarter * 32 + lane;             // weight row inside the tile
        const uint32_t tlane = (uint32_t)(quarter * 32) << 16;
        int stage = 0; uint32_t phase = 0;
        int ab = 0; uint32_t aphase = 0;
        uint32_t rphase = 0;
        bool ok = true;
        float acc[C::NACCUM][C::NC];
        for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
            Unit un;
            if (!decode_unit(u, p.n_mtiles, p.num_local, NTOK, s_tiles, s_row0, s_cnt, un)) break;
#pragma unroll
            for (int a = 0; a < C::NACCUM; ++a)
#pragma unroll
                for (int i = 0; i < C::NC; ++i) acc[a][i] = 0.f;
            const float* ws0 = p.w_scale + ((size_t)un.e * p.scale_rows + un.mt) * p.KB;
            const float* ws1 = G1 ? ws0 + (size_t)(p.gate_offset >> 7) * p.KB : ws0;
            float sw0n = __ldg(ws0), sw1n = G1 ? __ldg(ws1) : 0.f;
            for (int kb = 0; kb < p.KB; ++kb) {
                const float sw0 = sw0n, sw1 = sw1n;
                if (kb + 1 < p.KB) { sw0n = __ldg(ws0 + kb + 1); if (G1) sw1n = __ldg(ws1 + kb + 1); }
                if (!mbar_wait(bar_tfull + 8 * ab, aphase, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
                // the token scales of this stage arrived with the same transaction barrier as the tiles
                if (!mbar_wait(bar_full + 8 * stage, phase, p.status, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
                tc_fence_after();
                const float* sc = reinterpret_cast<const float*>(smem + stage * C::STAGE_BYTES + C::SC_OFF) + c0;
                const uint32_t tcol = tmem_base + tlane + ab * C::CPB + c0;
#pragma unroll
                for (int ch = 0; ch < C::NC / 16; ++ch) {
                    float4 s4[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) s4[j] = *reinterpret_cast<const float4*>(sc + ch * 16 + j * 4);
                    const float* sv = reinterpret_cast<const float*>(s4);
#pragma unroll
                    for (int a = 0; a < C::NACCUM; ++a) {
                        float part[16];
                        tmem_ld16(tcol + a * NTOK + ch * 16, part);
                        tmem_wait_ld();
                        const float sw = a == 0 ? sw0 : sw1;
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[a][ch * 16 + i] = fmaf(part[i], sv[i] * sw, acc[a][ch * 16 + i]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { mbar_arrive(bar_tempty + 8 * ab); mbar_arrive(bar_empty + 8 * stage); }
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                if (++ab == C::NACC) { ab = 0; aphase ^= 1; }
            }
            if (!ok) break;

            if (G1) {
                // SwiGLU, then amax over the 128 rows of the tile for every token column
                uint32_t* red = s_red + pw * C::NC;
#pragma unroll
                for (int i = 0; i < C::NC; ++i) {
                    const float v = silu_f(acc[1][i]) * acc[0][i];
                    acc[0][i] = v;
                    const uint32_t wm = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(fabsf(v)));
                    if (lane == 0) red[i] = wm;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_red + 8 * grp);
                if (!mbar_wait(bar_red + 8 * grp, rphase, p.status, ERR_WAIT_GROUP)) { ok = false; break; }
                rphase ^= 1;
                const uint32_t* rg = s_red + grp * 4 * C::NC;
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
                __syncwarp();                                   // s_red is reused by the next unit
                if (lane == 0) mbar_arrive(bar_red + 8 * grp);
                if (!mbar_wait(bar_red + 8 * grp, rphase, p.status, ERR_WAIT_GROUP)) { ok = false; break; }
                rphase ^= 1;
            } else {
                const size_t col = (size_t)un.mt * 128 + m;
#pragma unroll
                for (int i = 0; i < C::NC; ++i) {
                    const int c = c0 + i;
                    if (c < un.nvalid) {
                        const size_t row = (size_t)(un.row0 + c);
                        p.y[row * p.H + col] = acc[0][i] * __ldg(p.row_w + row);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

}  // namespace b200moe
