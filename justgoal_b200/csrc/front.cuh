// Fused permutation + gather for small token counts (T <= FRONT_MAX_T): histogram, scan, stable
// permutation and the expert-sorted activation gather in ONE launch after the routing kernel.
//
// With a few dozen tokens the separate kernels are pure launch latency, so every CTA of this
// kernel redoes the (tiny, integer) histogram and permutation for ALL tokens in its own shared
// memory - no CTA ever waits for another - and then copies its share of the rows.  CTA 0 alone
// writes the tables that later kernels read (counts, row maps); all CTAs derive identical values.
// Same results as count_kernel + permute_kernel + gather_kernel (permute.cuh); the reference
// fuses the same stages for small batches
// (kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/kernel.cu:724-806).
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
    __shared__ int s_idx[FRONT_MAX_T * 8];
    __shared__ float s_w[FRONT_MAX_T * 8];
    __shared__ int s_cnt[MAX_LOCAL];
    __shared__ int s_row0[MAX_LOCAL + 1];
    __shared__ int s_tiles[MAX_LOCAL + 1];
    __shared__ int s_row_token[FRONT_MAX_ROWS];
    const PlanParams& pp = fp.plan;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int T = pp.T, K = pp.top_k, El = pp.num_local;
    const bool publish = blockIdx.x == 0;
    const int n = T * K;

    for (int i = tid; i < El; i += blockDim.x) s_cnt[i] = 0;
    __syncthreads();

    // ---- the routing result of all tokens, and the histogram of the local experts
    for (int i = tid; i < n; i += blockDim.x) {
        const int tok = i / K;
        const size_t src = (size_t)tok * pp.pair_stride + (i - tok * K);
        const int id = FRESH ? __ldcg(pp.topk_idx + src) : pp.topk_idx[src];
        s_idx[i] = id;
        s_w[i] = FRESH ? __ldcg(pp.topk_w + src) : pp.topk_w[src];
        const int le = id - pp.local_offset;
        if (le >= 0 && le < El) atomicAdd(&s_cnt[le], 1);
    }
    __syncthreads();

    // ---- scan
    if (warp == 0) scan_counts(s_cnt, El, pp.token_tile, s_row0, s_tiles, publish ? pp.status : nullptr, lane);
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

    // ---- stable permutation: a warp places one expert's pairs in token order (ballot ranks)
    for (int e = warp; e < El; e += FRONT_THREADS / 32) {
        if (s_cnt[e] == 0) continue;
        const int ge = e + pp.local_offset;
        int placed = 0;
        for (int base = 0; base < n; base += 32) {
            const int i = base + lane;
            const bool hit = i < n && s_idx[i] == ge;
            const unsigned m = __ballot_sync(0xFFFFFFFFu, hit);
            if (hit) {
                const int r = s_row0[e] + placed + __popc(m & ((1u << lane) - 1u));
                if (r < FRONT_MAX_ROWS && r < pp.rows_cap) {
                    s_row_token[r] = i / K;
                    if (publish) { pp.pair_row[i] = r; pp.row_w[r] = s_w[i]; }
                } else {                    // repeated expert ids inside a caller-given row: refuse, write nothing
                    atomicCAS(pp.status + ST_ERR, 0, ERR_BAD_SCHEDULE);
                }
            }
            placed += __popc(m);
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

    // ---- gather: a row is cut into GATHER_SPLIT pieces, one warp per piece, dealt round-robin over all warps of
    // the grid: with a few dozen rows every lane then has 3-4 independent 16-byte loads in flight instead of 14
    constexpr int GATHER_SPLIT = 4;
    const int H = fp.H, KB = H >> 7, rows_cap = pp.rows_cap;
    const int chunks = H / 16, per_piece = (chunks + GATHER_SPLIT - 1) / GATHER_SPLIT;
    const int n_tasks = total_rows * GATHER_SPLIT;
    for (int task = blockIdx.x * (FRONT_THREADS / 32) + warp; task < n_tasks; task += gridDim.x * (FRONT_THREADS / 32)) {
        const int r = task / GATHER_SPLIT, piece = task - r * GATHER_SPLIT;
        const int t = s_row_token[r];
        if (t < 0) continue;     // padding rows stay unwritten: their columns are never stored by the GEMMs
        uint4* dst = reinterpret_cast<uint4*>(fp.a_perm + (size_t)r * H);
        const uint4* src = reinterpret_cast<const uint4*>(fp.hidden + (size_t)t * H);
        const int c_end = min(chunks, (piece + 1) * per_piece);
        for (int i = piece * per_piece + lane; i < c_end; i += 32) dst[i] = __ldg(src + i);
        if (piece == 0)
            for (int kb = lane; kb < KB; kb += 32)
                fp.a_scale_perm[(size_t)kb * rows_cap + r] = __ldg(fp.hscale + (size_t)kb * T + t);
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
    pdl_launch();
    // CTA 0 clears the head of the workspace.  Nothing reads or flags an error in it before the meeting below, and
    // CTA 0 arrives there only after its stores (the fence before the arrival orders them).
    if (blockIdx.x == 0)
        for (int i = threadIdx.x; i < fp.head_vec; i += FRONT_THREADS) fp.head[i] = make_uint4(0u, 0u, 0u, 0u);
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
        s_go = go;
    }
    __syncthreads();
    if (!s_go) return;
    front_body<true>(fp);
}

}  // namespace b200moe

