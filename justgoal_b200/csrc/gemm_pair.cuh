// Grouped FP8 block-scale GEMMs for full token tiles on PAIRS of SMs (tcgen05 cta_group::2).
//
// Why pairs.  With 128-token tiles the single-SM kernel (gemm.cuh) sits on the SM's shared-memory bandwidth:
// every 128-K block writes 48 KB into shared memory (TMA) and reads 48 KB out of it again (four N = 256 MMAs of
// 12 KB each), and the two do not overlap - a block takes the sum of the two times, ~1100 cycles against 512
// cycles of MMA.  A pair of CTAs in one cluster runs ONE tcgen05.mma.cta_group::2 over M = 256: each CTA owns
// one 128-token tile of the same expert (its own TMEM lanes) and holds only HALF of the block's weight rows
// (rank 0 the first weight tile, rank 1 the second; the tensor cores read the other half from the peer's shared
// memory).  Per block and SM that is 32 KB written and 32 KB read instead of 48 + 48.
// (Measured and dropped: two N = 128 instructions per K step into separate 128-column accumulators - four
// hand-off buffers instead of two; the token tile is then read twice per K step and the block took 1460 cycles.)
//
// One PAIR UNIT = (local expert, two consecutive 128-token tiles, two 128-row weight tiles), full K.
// Arithmetic, promotion per 128 K, SwiGLU + two-term e4m3 requantisation and the fp16 row store are
// those of gemm.cuh (tokens on M); results agree with it to the last bits of the fp32 sums.  The reference's counterpart is
// its 2-SM tile kernel (kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/
// kernel.cu:4216-4675).
//
// Roles per CTA: warp 0 lane 0 = TMA producer (its token tile + its weight tile; the bytes of
// both CTAs count on the LEADER's "full" barrier), warp 1 lane 0 of the leader = MMA issuer for the pair,
// warp 1 of each CTA owns its TMEM, warps 4..11 = promotion / epilogue of the CTA's own token tile.
// Commits reach both CTAs' barriers; promotion warps of both CTAs release accumulators on the leader.
// Every software wait is bounded (common.cuh); no load uses cluster multicast; the CTAs of a pair leave
// together (cluster barrier) so that nobody signals a barrier of a CTA that is gone.
#pragma once
#include "gemm.cuh"

namespace b200moe {

template <bool G1>
struct PairCfg {
    static constexpr int NTOK = 128;
    static constexpr int NA = G1 ? 1 : 2;                 // token-side operands per stage (GEMM2: hi and lo)
    static constexpr int A_BYTES = 128 * 128;             // this CTA's token tile, one 128-K block
    static constexpr int BH_BYTES = 128 * 128;            // this CTA's weight tile = its half of the N = 256 operand
    static constexpr int B_OFF = NA * A_BYTES;
    static constexpr int STAGE_BYTES = NA * A_BYTES + BH_BYTES;           // 32 KB / 48 KB
    static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;             // 6 / 4
    static constexpr int NBUF = 2;                        // TMEM accumulators of 256 columns (both weight tiles)
    static constexpr int TMEM_COLS = 512;
    static constexpr int NPW = 8, NGRP = 2, NPT = 256, NC = 64;           // promotion warps: 2 column groups x 4 lane quarters
    static constexpr int NTHREADS = 128 + NPT;
    static constexpr int LAUNCH_REGS = (65536 / NTHREADS) / 8 * 8;
    static constexpr int CTRL_REGS = 40, PROMO_REGS = 232;
    static_assert(128 * CTRL_REGS + NPT * PROMO_REGS <= NTHREADS * LAUNCH_REGS, "setmaxnreg.inc would wait forever");
    static constexpr int TABLE_INTS = 4 * (MAX_LOCAL + 1);
    static constexpr int RED_BYTES = NGRP * 128 * 4;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256 + TABLE_INTS * 4 + RED_BYTES + 32;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
    static_assert(8 * (2 * STAGES + 2 * NBUF + 1) <= 240, "barrier area");
};

// ---------------------------------------------------------------- cluster / cta_group::2 helpers
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// Arrive on a barrier of the pair (shared::cluster address).  Default semantics (release at CTA scope) on purpose:
// what the barrier orders here are TMEM reads against later MMAs, which tcgen05.fence::before_thread_sync and the
// barrier itself cover; a cluster-scope release made every hand-back wait for the thread's outstanding global
// loads (the prefetched scales) and cost ~1 us per accumulator.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of one CTA of a pair; the transaction bytes are counted on the barrier at `bar_cluster`
// (a shared::cluster address: the leader's barrier, whichever CTA issues the load).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[both CTAs' smem, 128 rows each] * B[both CTAs' smem, N/2 rows each]^T, one K = 32 step
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on the barrier at the same shared-memory offset in BOTH CTAs of the pair once every tcgen05 op issued
// so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}

// Pair unit u -> (expert, weight tiles mt, tile pair tp).  Units of one (expert, mt) are adjacent, so clusters
// that run at the same time share a weight tile through L2; the token tiles of an expert come back every
// `pairs` units.  s_pp = exclusive prefix of tile pairs per expert.
struct PairUnit { int e, mt, row0, nvalid; };
__device__ __forceinline__ bool decode_pair_unit(int u, int n_mtiles, int num_local, const int* s_pp, const int* s_row0,
                                                 const int* s_cnt, int rank, PairUnit& o) {
    const int q = u / n_mtiles;
    int lo = 0, hi = num_local;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_pp[mid] <= q) lo = mid; else hi = mid - 1;
    }
    if (lo >= num_local) return false;
    const int np = s_pp[lo + 1] - s_pp[lo];
    if (np <= 0) return false;
    const int ul = u - s_pp[lo] * n_mtiles;
    o.e = lo;
    o.mt = ul / np;
    const int tile = 2 * (ul - o.mt * np) + rank;
    o.row0 = s_row0[lo] + tile * 128;
    const int left = s_cnt[lo] - tile * 128;
    o.nvalid = left < 0 ? 0 : (left > 128 ? 128 : left);
    return o.mt < n_mtiles;
}

template <bool G1>
__global__ void __launch_bounds__(PairCfg<G1>::NTHREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_b0,
                 const __grid_constant__ CUtensorMap tm_b1, const GemmParams p) {
    using C = PairCfg<G1>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tail = smem + C::STAGES * C::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);     // full[S], empty[S], tfull[NBUF], tempty[NBUF], all
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tail + 240);
    int* s_pp = reinterpret_cast<int*>(tail + 256);
    int* s_row0 = s_pp + (MAX_LOCAL + 1);
    int* s_cnt = s_row0 + (MAX_LOCAL + 1);
    int* s_tiles = s_cnt + (MAX_LOCAL + 1);
    float* s_red = reinterpret_cast<float*>(s_tiles + (MAX_LOCAL + 1));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_rank();
#ifdef B200MOE_PAIR_TRACE
    // timing build only: cycles one thread of every role spends in each of its waits, summed over the kernel
    long long* const trace = p.trace ? p.trace + (size_t)blockIdx.x * TRACE_SLOTS : nullptr;
#define PT_DECL(...) long long __VA_ARGS__
#define PT_T0() const long long pt0_ = clock64()
#define PT_ADD(v) v += clock64() - pt0_
#define PT_PUT(slot, v) do { if (trace) trace[slot] = (v); } while (0)
#else
#define PT_DECL(...)
#define PT_T0()
#define PT_ADD(v)
#define PT_PUT(slot, v)
#endif
    const long long t_entry = clock64();
    (void)t_entry;
    if (threadIdx.x == 0) PT_PUT(0, (long long)globaltimer_ns());
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * C::STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * C::STAGES;
    const uint32_t bar_tempty = bar_tfull + 8 * C::NBUF;
    const uint32_t bar_all = bar_tempty + 8 * C::NBUF;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < C::NBUF; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, 2 * C::NPW); }
        mbar_init(bar_all, C::NPW);
        mbar_fence_init();
        tma_prefetch_desc(&tm_w); tma_prefetch_desc(&tm_b0);
        if (!G1) tma_prefetch_desc(&tm_b1);
    }
    if (warp == 1) { tmem_alloc_pair(smem_u32(s_tmem), C::TMEM_COLS); tmem_relinquish_pair(); }
    pdl_wait();
    pdl_launch();
    for (int i = threadIdx.x; i <= p.num_local; i += blockDim.x) {
        s_tiles[i] = p.tile_prefix[i];
        s_row0[i] = p.expert_row0[i];
        s_cnt[i] = i < p.num_local ? p.counts[i] : 0;
    }
    __syncthreads();
    if (warp == 0) {
        // exclusive prefix of tile pairs per expert (ceil(tiles / 2)), 32 experts per round
        int carry = 0;
        for (int base = 0; base < p.num_local; base += 32) {
            const int e = base + lane;
            const int np = e < p.num_local ? (s_tiles[e + 1] - s_tiles[e] + 1) >> 1 : 0;
            int inc = np;
            for (int off = 1; off < 32; off <<= 1) {
                const int v = __shfl_up_sync(0xFFFFFFFFu, inc, off);
                if (lane >= off) inc += v;
            }
            if (e < p.num_local) s_pp[e] = carry + inc - np;
            carry += __shfl_sync(0xFFFFFFFFu, inc, 31);
        }
        if (lane == 0) s_pp[p.num_local] = carry;
    }
    tc_fence_before();
    __syncthreads();
    cluster_barrier();          // both CTAs: barriers initialised, TMEM allocated
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    const uint32_t smem_base = smem_u32(smem);
    const int cidx = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);
    const int total_units = s_pp[p.num_local] * p.n_mtiles;
    const int my_units = cidx < total_units ? (total_units - cidx + ncl - 1) / ncl : 0;

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::CTRL_REGS));
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            PT_DECL(w_empty = 0);
            for (int ui = 0; ui < my_units && ok; ++ui) {
                PairUnit un;
                if (!decode_pair_unit(cidx + ui * ncl, p.n_mtiles, p.num_local, s_pp, s_row0, s_cnt, (int)crank, un)) {
                    atomicCAS(p.status, 0, ERR_BAD_SCHEDULE); break;
                }
                const int wrow = un.e * p.rows_per_expert + un.mt * p.unit_rows + (int)crank * p.gate_offset;
                for (int kb = 0; kb < p.KB; ++kb) {
                    { PT_T0();
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, p.status, ERR_WAIT_SMEM_EMPTY)) { ok = false; break; }
                    PT_ADD(w_empty); }
                    const uint32_t st = smem_base + stage * C::STAGE_BYTES;
                    const uint32_t full0 = cluster_map(bar_full + 8 * stage, 0);      // the leader's barrier
                    if (crank == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * C::STAGE_BYTES);
                    tma_load_2d_pair(st, &tm_b0, kb * 128, un.row0, full0);
                    if (!G1) tma_load_2d_pair(st + C::A_BYTES, &tm_b1, kb * 128, un.row0, full0);
                    tma_load_2d_pair(st + C::B_OFF, &tm_w, kb * 128, wrow, full0);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            PT_PUT(1, w_empty); PT_PUT(2, clock64() - t_entry);
            // tail: the commits that release the last stages arrive from the leader asynchronously; stay until every
            // stage this CTA filled has been released, so that none of them can find the CTA gone
            for (int i = 0; i < C::STAGES && ok; ++i) {
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, p.status, ERR_WAIT_SMEM_EMPTY)) ok = false;
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) {
                for (int i = 0; i < 64; ++i) __nanosleep(10000);    // copies in flight land before shared memory goes away
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA, for the pair)
        if (lane == 0 && crank == 0) {
            constexpr uint32_t idesc = make_idesc_f8(256, 256);     // M = 256 over the pair, N = both weight tiles
            int stage = 0; uint32_t phase = 0;
            int ab = 0; uint32_t aphase = 0;
            bool ok = true;
            PT_DECL(w_full = 0, w_tempty = 0);
            for (int ui = 0; ui < my_units && ok; ++ui) {
                for (int kb = 0; kb < p.KB && ok; ++kb) {
                    { PT_T0();
                    if (!mbar_wait(bar_tempty + 8 * ab, aphase ^ 1, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
                    PT_ADD(w_tempty); }
                    { PT_T0();
                    if (!mbar_wait(bar_full + 8 * stage, phase, p.status, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
                    PT_ADD(w_full); }
                    tc_fence_after();
                    const uint32_t st = smem_base + stage * C::STAGE_BYTES;
                    const uint32_t d = tmem_base + ab * 256;
                    const uint64_t a0 = make_smem_desc(st);
                    const uint64_t w = make_smem_desc(st + C::B_OFF);
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_f8_pair(d, a0 + 2 * k, w + 2 * k, idesc, k > 0);
                    if (!G1) {      // GEMM2: the low-order term of the activation accumulates on top
                        const uint64_t a1 = make_smem_desc(st + C::A_BYTES);
#pragma unroll
                        for (int k = 0; k < 4; ++k) umma_f8_pair(d, a1 + 2 * k, w + 2 * k, idesc, 1u);
                    }
                    umma_commit_pair(bar_empty + 8 * stage);
                    umma_commit_pair(bar_tfull + 8 * ab);
                    if (++ab == C::NBUF) { ab = 0; aphase ^= 1; }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            PT_PUT(3, w_full); PT_PUT(4, w_tempty); PT_PUT(5, clock64() - t_entry);
        }
        __syncwarp();
    }
    } else {
        // ------------------------------------------------------------ promotion + epilogue (own token tile)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::PROMO_REGS));
        const int quarter = warp & 3;
        const int grp_id = (warp - 4) >> 2;
        const int c0 = grp_id * C::NC;
        const int m = quarter * 32 + lane;             // token row inside this CTA's tile = TMEM lane
        const uint32_t tlane = (uint32_t)(quarter * 32) << 16;
        const uint32_t tempty0 = cluster_map(bar_tempty, 0);       // accumulators are released on the leader
        int ab = 0; uint32_t aphase = 0;
        uint32_t allphase = 0;
        bool ok = true;
        float acc[2][C::NC];
        PT_DECL(w_tfull = 0, w_ld = 0, w_rel = 0, w_fma = 0, w_epi = 0);
        (void)0;

        auto all_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_all);
            const bool r = mbar_wait(bar_all, allphase, p.status, ERR_WAIT_GROUP);
            allphase ^= 1;
            return r;
        };

        for (int ui = 0; ui < my_units && ok; ++ui) {
            PairUnit un;
            if (!decode_pair_unit(cidx + ui * ncl, p.n_mtiles, p.num_local, s_pp, s_row0, s_cnt, (int)crank, un)) break;
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int i = 0; i < C::NC; ++i) acc[a][i] = 0.f;
            const int srow0 = un.mt * (p.unit_rows >> 7);
            const int srow1 = min(srow0 + (p.gate_offset >> 7), p.scale_rows - 1);
            const float* ws0 = p.w_scale + ((size_t)un.e * p.scale_rows + srow0) * p.KB;
            const float* ws1 = p.w_scale + ((size_t)un.e * p.scale_rows + srow1) * p.KB;
            const int arow = min(un.row0 + m, p.rows_cap - 1);           // rows of a tile that does not exist are never stored
            const float* tsp = p.b_scale + arow;
            // scales one K block ahead: their load latency never sits between a hand-off and the first FMA
            float swn0 = __ldg(ws0), swn1 = __ldg(ws1);
            float stokn = __ldcg(tsp);
            for (int kb = 0; kb < p.KB; ++kb) {
                const float sx0 = stokn * swn0, sx1 = stokn * swn1;
                const int kn = min(kb + 1, p.KB - 1);
                swn0 = __ldg(ws0 + kn); swn1 = __ldg(ws1 + kn);
                stokn = __ldcg(tsp + (size_t)kn * p.rows_cap);
                { PT_T0();
                if (!mbar_wait(bar_tfull + 8 * ab, aphase, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
                PT_ADD(w_tfull); }
                tc_fence_after();
                const uint32_t tbuf = tmem_base + tlane + ab * 256 + c0;
                // the block as four chunks of 32 columns (two per weight tile), two tcgen05.ld in flight per wait;
                // the buffer goes back as soon as the last load has completed, the last FMAs run after the release
                float stg[2][32];
                auto qaddr = [&](int q) { return tbuf + (q >> 1) * 128 + (q & 1) * 32; };
                auto qfold = [&](int q, const float* v) {
                    const float sx = (q >> 1) ? sx1 : sx0;
                    const float2 s2 = make_float2(sx, sx);
                    float* ac = &acc[q >> 1][(q & 1) * 32];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float2 r0 = __ffma2_rn(make_float2(v[i], v[i + 1]), s2, make_float2(ac[i], ac[i + 1]));
                        ac[i] = r0.x; ac[i + 1] = r0.y;
                    }
                };
                PT_T0();
                tmem_ld_chunk<32>(qaddr(0), stg[0]);
                tmem_ld_chunk<32>(qaddr(1), stg[1]);
                tmem_wait_ld();
                qfold(0, stg[0]);
                tmem_ld_chunk<32>(qaddr(2), stg[0]);
                qfold(1, stg[1]);
                tmem_ld_chunk<32>(qaddr(3), stg[1]);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(tempty0 + 8 * ab);
                PT_ADD(w_ld);
                qfold(2, stg[0]);
                qfold(3, stg[1]);
                if (++ab == C::NBUF) { ab = 0; aphase ^= 1; }
            }
            if (!ok) break;
            PT_T0();

            if (G1) {
                // token row m, 64 consecutive columns j of the 128-wide block: SwiGLU, amax over the block (own
                // columns, then the other column group's thread of the same row), two e4m3 terms, 32-byte stores
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < C::NC; ++i) {
                    const float v = silu_f(acc[1][i]) * acc[0][i];
                    acc[0][i] = v;
                    amax = fmaxf(amax, fabsf(v));
                }
                s_red[grp_id * 128 + m] = amax;
                if (!all_sync()) { ok = false; break; }
#pragma unroll
                for (int g2 = 0; g2 < C::NGRP; ++g2) amax = fmaxf(amax, s_red[g2 * 128 + m]);
                if (!all_sync()) { ok = false; break; }                   // s_red is reused by the next unit
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
            } else {
                if (m < un.nvalid) {
                    const size_t row = (size_t)(un.row0 + m);
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const int col0 = un.mt * p.unit_rows + a * p.gate_offset + c0;
                        if (col0 < p.valid_rows) store_y_row<C::NC>(p.y + row * p.H + col0, acc[a]);
                    }
                }
            }
            PT_ADD(w_epi);
        }
        if (threadIdx.x == 128) {
            PT_PUT(6, w_tfull); PT_PUT(7, w_ld); PT_PUT(8, w_rel); PT_PUT(9, w_fma); PT_PUT(10, w_epi);
            PT_PUT(11, clock64() - t_entry); PT_PUT(12, my_units);
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_barrier();          // the peer may still signal this CTA's barriers or use its TMEM until both are done
    if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, C::TMEM_COLS); }
    if (threadIdx.x == 0) { PT_PUT(13, (long long)globaltimer_ns()); PT_PUT(14, clock64() - t_entry); }
}

}  // namespace b200moe
