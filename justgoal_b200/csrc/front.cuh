// Front end for small token counts (T <= FRONT_MAX_T): routing, histogram, scan, stable permutation and the
// expert-sorted activation gather in ONE launch (front_route_kernel; front_small_kernel is the same without the
// routing, for tokens that were routed elsewhere).
//
// With a few dozen tokens separate kernels are pure launch latency.  The tokens are routed one per warp over the CTAs;
// the CTAs meet once (the routing result of every token must be visible); then every CTA redoes the tiny integer
// work - histogram, scan, ranks - for ALL tokens in its own shared memory, so no CTA waits for another again, and
// copies its share of the rows.  One thread owns one (token, expert) pair: its rank inside its expert is its rank
// among the same-expert pairs of its warp (match.any) plus the counts of the warps before it, which keeps the rows of
// an expert in token order.  CTA 0 alone writes the tables that later kernels read (counts, row maps); all CTAs
// derive identical values.  Same results as count_kernel + permute_kernel + gather_kernel (permute.cuh).
// The next kernel (GEMM1) does not wait for this one to finish before it starts to work: see ST_ROUTED below and
// GemmParams::routed.  The reference fuses the same stages for small batches
// (kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/kernel.cu:724-806) and issues its first
// weight stages during the table build (its MOE_EARLY_W switch, same directory, main.py:50).
#pragma once
#include "permute.cuh"
#include "routing.cuh"

namespace b200moe {

constexpr int FRONT_MAX_T = 128;
constexpr int FRONT_MAX_ROWS = FRONT_MAX_T * 8 + ROW_ALIGN * MAX_LOCAL;   // worst case incl. segment padding
constexpr int FRONT_THREADS = 1024;

struct FrontParams {
    PlanParams plan;              // topk_idx / topk_w in, tables to publish (CTA 0) out
    const uint8_t* hidden;        // [T, H] fp8
    const float* hscale;          // [H/128, T]
    uint8_t* a_perm;              // [rows_cap, H]
    float* a_scale_perm;          // [H/128, rows_cap]
    int H;
    // front_route_kernel only.  `sync` is two words owned by the handle, zero between calls: [0] CTAs that have
    // arrived at the meeting, [1] CTAs that have left it (the last one to leave clears both).  `head` is the part of
    // the workspace that must be zero before the GEMMs run (status, split-unit counters), in 16-byte units: CTA 0
    // clears it, so the forward needs no memset in front of the kernel.
    int* sync;
    uint4* head;
    int head_vec;
};

// The body shared by the two entry kernels below.  FRESH: the routing result was written earlier in this same
// launch by other CTAs (read it past L1).
template <bool FRESH>
__device__ __forceinline__ void front_body(const FrontParams& fp) {
    __shared__ int s_cnt[MAX_LOCAL];
    __shared__ int s_row0[MAX_LOCAL + 1];
    __shared__ int s_tiles[MAX_LOCAL + 1];
    __shared__ int s_row_token[FRONT_MAX_ROWS];
    __shared__ uint8_t s_wcnt[FRONT_THREADS / 32][MAX_LOCAL];    // pairs of expert e among the 32 pairs of warp w
    static_assert(FRONT_THREADS >= FRONT_MAX_T * 8, "one thread per (token, expert) pair");
    const PlanParams& pp = fp.plan;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int T = pp.T, K = pp.top_k, El = pp.num_local;
    const bool publish = blockIdx.x == 0;
    const int n = T * K;

    for (int i = tid; i < El; i += blockDim.x) s_cnt[i] = 0;
    for (int i = tid; i < (int)(sizeof(s_wcnt) / 4); i += blockDim.x) reinterpret_cast<uint32_t*>(s_wcnt)[i] = 0u;
    __syncthreads();

    // ---- this thread's pair (pair i = tid, token-major), the histogram of the local experts, and the pair's rank
    // among the pairs of the same expert inside its warp (stable: pair order)
    const int tok = tid / K;
    const bool valid = tid < n;
    const size_t src = (size_t)tok * pp.pair_stride + (tid - tok * K);
    const int id = valid ? (FRESH ? __ldcg(pp.topk_idx + src) : pp.topk_idx[src]) : -1;
    const float wgt = valid ? (FRESH ? __ldcg(pp.topk_w + src) : pp.topk_w[src]) : 0.f;
    const int le = id - pp.local_offset;
    const bool local = valid && le >= 0 && le < El;
    const unsigned same = __match_any_sync(0xFFFFFFFFu, local ? le : -1 - lane);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (local && rank == 0) {
        s_wcnt[warp][le] = (uint8_t)__popc(same);
        atomicAdd(&s_cnt[le], __popc(same));
    }
    __syncthreads();

    // ---- scan
    if (warp == 0) scan_counts(s_cnt, El, pp.token_tile, s_row0, s_tiles, publish ? pp.status : nullptr, lane);
    // pairs of the same expert in the warps before this one (independent byte loads, no second scan phase)
    int before = 0;
    if (local)
        for (int w2 = 0; w2 < warp; ++w2) before += s_wcnt[w2][le];
    __syncthreads();
    const int total_rows = min(min(s_row0[El], FRONT_MAX_ROWS), pp.rows_cap);
    if (publish) {
        for (int i = tid; i <= El; i += blockDim.x) {
            pp.expert_row0[i] = s_row0[i];
            pp.tile_prefix[i] = s_tiles[i];
            if (i < El) pp.counts[i] = s_cnt[i];
        }
    }
    for (int r = tid; r < total_rows; r += blockDim.x) s_row_token[r] = -1;
    __syncthreads();

    // ---- stable permutation: an expert's pairs take its rows in pair order
    if (local) {
        const int r = s_row0[le] + before + rank;
        if (r < FRONT_MAX_ROWS && r < pp.rows_cap) {
            s_row_token[r] = tok;
            if (publish) { pp.pair_row[tid] = r; pp.row_w[r] = wgt; }
        } else {                    // more rows than the caller's capacity: refuse, write nothing
            atomicCAS(pp.status + ST_ERR, 0, ERR_BAD_SCHEDULE);
        }
    }
    __syncthreads();
    if (publish) {
        for (int r = tid; r < total_rows; r += blockDim.x) {
            const int t = s_row_token[r];
            pp.row_token[r] = t;
            if (t < 0) pp.row_w[r] = 0.f;
        }
    }

    // ---- gather: a row is cut into pieces, one warp per piece, dealt round-robin over all warps of the grid.  The
    // number of pieces grows until every warp has one (a few dozen rows: 16 pieces, one 16-byte load per lane); a
    // warp with more to copy keeps four loads in flight per lane.
    const int H = fp.H, KB = H >> 7, rows_cap = pp.rows_cap;
    const int chunks = H / 16;
    const int n_warps = (int)gridDim.x * (FRONT_THREADS / 32);
    int split = 1;
    while (split < 16 && total_rows * split * 2 <= n_warps) split *= 2;
    const int per_piece = (chunks + split - 1) / split;
    const int n_tasks = total_rows * split;
    for (int task = blockIdx.x * (FRONT_THREADS / 32) + warp; task < n_tasks; task += n_warps) {
        const int r = task / split, piece = task - r * split;
        const int t = s_row_token[r];
        if (t < 0) continue;     // padding rows stay unwritten: their columns are never stored by the GEMMs
        uint4* dst = reinterpret_cast<uint4*>(fp.a_perm + (size_t)r * H);
        const uint4* src = reinterpret_cast<const uint4*>(fp.hidden + (size_t)t * H);
        const int c_end = min(chunks, (piece + 1) * per_piece);
        for (int i = piece * per_piece + lane; i < c_end; i += 128) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + 32 * j < c_end) v[j] = __ldg(src + i + 32 * j);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + 32 * j < c_end) dst[i + 32 * j] = v[j];
        }
        if (piece == split - 1) {
            // the row's block scales (KB <= 64 for every supported hidden size up to 8192: two loads per lane)
            for (int kb = lane; kb < KB; kb += 64) {
                const float s0 = __ldg(fp.hscale + (size_t)kb * T + t);
                const float s1 = kb + 32 < KB ? __ldg(fp.hscale + (size_t)(kb + 32) * T + t) : 0.f;
                fp.a_scale_perm[(size_t)kb * rows_cap + r] = s0;
                if (kb + 32 < KB) fp.a_scale_perm[(size_t)(kb + 32) * rows_cap + r] = s1;
            }
        }
    }
}


// Front end for tokens that were routed by an earlier kernel.
__global__ void __launch_bounds__(FRONT_THREADS, 1) front_small_kernel(const FrontParams fp) {
    pdl_wait();
    pdl_launch();
    front_body<false>(fp);
}

// Front end INCLUDING the routing (the operator's own forward for T <= FRONT_MAX_T): one launch, and nothing else on the
// stream before it (CTA 0 clears the head of the workspace itself), so the kernel may start while the caller's
// previous kernel still runs.  Before the wait for that kernel the CTAs pull the inputs into L2 (a prefetch returns
// no data, so it is harmless if the previous kernel is still writing them; it hides the first-touch latency of
// every input behind that kernel's tail).
// Phase A: the tokens are dealt over the CTAs (one warp per token) and routed; the CTAs then meet at a counter in
// device memory owned by the handle (all CTAs of this small grid are resident; the wait is bounded like every wait
// of the library); phase B is the common body, every CTA redoing the integer work for all tokens.
template <int VPT, int MODE>
__global__ void __launch_bounds__(FRONT_THREADS, 1) front_route_kernel(const FrontParams fp, const RouteParams rp) {
    __shared__ int s_go;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        const size_t gtid = (size_t)blockIdx.x * FRONT_THREADS + threadIdx.x, gth = (size_t)gridDim.x * FRONT_THREADS;
        auto pull = [&](const void* base, size_t bytes) {
            for (size_t off = gtid * 128; off < bytes; off += gth * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const char*>(base) + off));
        };
        pull(rp.logits, (size_t)rp.T * rp.E * 4);
        pull(fp.hidden, (size_t)rp.T * fp.H);
        pull(fp.hscale, (size_t)(fp.H >> 7) * rp.T * 4);
        if (rp.bias) pull(rp.bias, (size_t)rp.E * 2);
    }
    pdl_wait();
    // CTA 0 clears the head of the workspace.  Nothing flags an error in it before the meeting below, and CTA 0
    // arrives there only after its stores (the fence before the arrival orders them).  The next kernel (GEMM1) reads
    // the ST_ROUTED word of the head before this kernel has completed, so CTA 0 lets it start only when the zeros
    // are visible.
    if (blockIdx.x == 0) {
        for (int i = threadIdx.x; i < fp.head_vec; i += FRONT_THREADS) fp.head[i] = make_uint4(0u, 0u, 0u, 0u);
        __threadfence();
        __syncthreads();
    }
    pdl_launch();
    for (int t = (int)blockIdx.x + (int)gridDim.x * warp; t < rp.T; t += (int)gridDim.x * (FRONT_THREADS / 32)) {
        int sel_id; float w;
        route_token<VPT, MODE>(rp, t, lane, sel_id, w);
        if (lane < rp.top_k) {
            rp.topk_idx[(size_t)t * rp.top_k + lane] = sel_id;
            rp.topk_w[(size_t)t * rp.top_k + lane] = w;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* const meet = fp.sync;
        atomicAdd(meet, 1);
        int go = 1;
        const unsigned long long t0 = globaltimer_ns();
        for (uint32_t it = 1;; ++it) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(meet) : "memory");
            if (v >= (int)gridDim.x) break;
            if ((it & 0xFFu) == 0 && globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                atomicCAS(fp.plan.status + ST_ERR, 0, ERR_WAIT_GROUP); go = 0; break;
            }
        }
        // every CTA that leaves has seen the full count: the last one to leave clears both words for the next call
        // (a call that gave up leaves them dirty; b200moe_status() clears them when it reports the error)
        if (go && atomicAdd(meet + 1, 1) == (int)gridDim.x - 1) { meet[0] = 0; meet[1] = 0; }
        // every CTA fenced its routing results before it arrived and this thread has acquired the full count: whoever
        // acquires the word below sees the routing of all tokens (GEMM1 builds its schedule from it and starts to
        // stream weights while this kernel still permutes and gathers)
        if (go && blockIdx.x == 0)
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(fp.plan.status + ST_ROUTED), "r"(1) : "memory");
        s_go = go;
    }
    __syncthreads();
    if (!s_go) return;
    front_body<true>(fp);
}

}  // namespace b200moe

