// Histogram / scan / permute / gather / combine kernels around the grouped GEMMs.
//
// Rows: every local (token, expert) pair gets one ROW in the expert-sorted buffers.  The rows
// of one expert are contiguous, in ascending token order (a stable counting sort, so results
// do not depend on atomic ordering), and each expert's segment starts on a multiple of
// ROW_ALIGN rows so that per-tile scale vectors are 16-byte aligned for bulk copies.
// The reference builds the same lists with atomics (expert order race-dependent):
// kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/kernel.cu:702-806,
// goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/moe_route.cuh:44-72.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"

namespace b200moe {

constexpr int ROW_ALIGN = 16;
constexpr int MAX_LOCAL = 256;

// status word layout (int32[8]) at the head of the workspace
enum : int { ST_ERR = 0, ST_PAIRS = 1, ST_ROWS = 2, ST_TILES = 3, ST_ACTIVE = 4 };

struct PlanParams {
    int T, top_k, num_local, local_offset, token_tile;
    const int32_t* topk_idx;   // [T, top_k]
    const float* topk_w;       // [T, top_k]
    int* status;               // [8]
    int* counts;               // [num_local]
    int* expert_row0;          // [num_local + 1]
    int* tile_prefix;          // [num_local + 1]
    int32_t* pair_row;         // [T, top_k]
    int32_t* row_token;        // [rows_cap]
    float* row_w;              // [rows_cap]
    int rows_cap;
};

// Counts per local expert from an explicit topk_idx (the expert-parallel receive side, where
// routing ran on another rank).
__global__ void count_kernel(const int32_t* __restrict__ topk_idx, int n, int local_offset, int num_local,
                             int* __restrict__ counts) {
    pdl_wait();
    pdl_launch();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int le = topk_idx[i] - local_offset;
        if (le >= 0 && le < num_local) atomicAdd(counts + le, 1);
    }
}

// Warp-parallel exclusive scan over the (<= 256) per-expert counts: lane l owns experts
// [l*per, (l+1)*per).  Fills s_row0[0..n] (first row of each expert, segments padded to
// ROW_ALIGN) and s_tiles[0..n] (exclusive prefix of token tiles); writes the totals into
// status[] when it is not null.  Must be called by the 32 lanes of one warp.
__device__ __forceinline__ void scan_counts(const int* counts, int num_local, int token_tile, int* s_row0, int* s_tiles,
                                            int* status, int tid) {
    const int per = (num_local + 31) / 32;
    int c[MAX_LOCAL / 32];
    int rows = 0, tiles = 0, pairs = 0, active = 0;
#pragma unroll
    for (int k = 0; k < MAX_LOCAL / 32; ++k) {
        const int i = tid * per + k;
        c[k] = (k < per && i < num_local) ? counts[i] : 0;
        rows += (c[k] + ROW_ALIGN - 1) / ROW_ALIGN * ROW_ALIGN;
        tiles += (c[k] + token_tile - 1) / token_tile;
        pairs += c[k]; active += c[k] > 0;
    }
    int rows_in = rows, tiles_in = tiles;
    for (int off = 1; off < 32; off <<= 1) {
        const int r = __shfl_up_sync(0xFFFFFFFFu, rows_in, off);
        const int t = __shfl_up_sync(0xFFFFFFFFu, tiles_in, off);
        if (tid >= off) { rows_in += r; tiles_in += t; }
    }
    for (int off = 16; off; off >>= 1) {
        pairs += __shfl_xor_sync(0xFFFFFFFFu, pairs, off);
        active += __shfl_xor_sync(0xFFFFFFFFu, active, off);
    }
    int r0 = rows_in - rows, t0 = tiles_in - tiles;       // exclusive prefixes of this lane
#pragma unroll
    for (int k = 0; k < MAX_LOCAL / 32; ++k) {
        const int i = tid * per + k;
        if (k < per && i < num_local) {
            s_row0[i] = r0; s_tiles[i] = t0;
            r0 += (c[k] + ROW_ALIGN - 1) / ROW_ALIGN * ROW_ALIGN;
            t0 += (c[k] + token_tile - 1) / token_tile;
        }
    }
    if (tid == 31) {
        s_row0[num_local] = rows_in; s_tiles[num_local] = tiles_in;
        if (status) {
            status[ST_PAIRS] = pairs; status[ST_ROWS] = rows_in;
            status[ST_TILES] = tiles_in; status[ST_ACTIVE] = active;
        }
    }
}

// One CTA per local expert.  Every CTA recomputes the (tiny) prefix over the counts, CTA 0
// publishes it; then the CTA places its expert's pairs in token order.
constexpr int PERMUTE_THREADS = 1024;
__global__ void __launch_bounds__(PERMUTE_THREADS) permute_kernel(const PlanParams p) {
    __shared__ int s_row0[MAX_LOCAL + 1];
    __shared__ int s_tiles[MAX_LOCAL + 1];
    __shared__ int s_scan[PERMUTE_THREADS];
    const int e = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch();

    if (tid < 32) scan_counts(p.counts, p.num_local, p.token_tile, s_row0, s_tiles, e == 0 ? p.status : nullptr, tid);
    __syncthreads();
    if (e == 0) {
        for (int i = tid; i <= p.num_local; i += blockDim.x) {
            p.expert_row0[i] = s_row0[i];
            p.tile_prefix[i] = s_tiles[i];
        }
    }
    const int cnt = p.counts[e];
    const int row0 = s_row0[e];
    const int row_end = s_row0[e + 1];
    // padding rows of this segment carry token -1
    for (int r = row0 + cnt + tid; r < row_end; r += blockDim.x) { p.row_token[r] = -1; p.row_w[r] = 0.f; }
    if (cnt == 0) return;

    // each thread owns a contiguous chunk of tokens -> order by token is preserved
    const int ge = e + p.local_offset;
    const int chunk = (p.T + blockDim.x - 1) / blockDim.x;
    const int t0 = min(tid * chunk, p.T), t1 = min(t0 + chunk, p.T);
    // the thread's chunk is one contiguous run of ints; read it in 16-byte pieces when it can be
    // (independent loads in flight instead of one dependent scalar load per entry)
    const int i0 = t0 * p.top_k, i1 = t1 * p.top_k;
    const bool vec = (p.top_k & 3) == 0;
    int mine = 0;
    if (vec) {
        const int4* v = reinterpret_cast<const int4*>(p.topk_idx + i0);
#pragma unroll 4
        for (int q = 0; q < (i1 - i0) >> 2; ++q) {
            const int4 x = __ldg(v + q);
            mine += (x.x == ge) + (x.y == ge) + (x.z == ge) + (x.w == ge);
        }
    } else {
        for (int i = i0; i < i1; ++i) mine += (p.topk_idx[i] == ge);
    }
    s_scan[tid] = mine;
    __syncthreads();
    // inclusive Hillis-Steele scan over the per-thread counters
    for (int off = 1; off < PERMUTE_THREADS; off <<= 1) {
        const int add = tid >= off ? s_scan[tid - off] : 0;
        __syncthreads();
        s_scan[tid] += add;
        __syncthreads();
    }
    int r = row0 + s_scan[tid] - mine;
    if (mine == 0) return;
    for (int i = i0; i < i1; ++i) {
        if (__ldg(p.topk_idx + i) == ge) {
            p.pair_row[i] = r;
            p.row_token[r] = i / p.top_k;
            p.row_w[r] = p.topk_w[i];
            ++r;
        }
    }
}

// Expert-sorted copy of the fp8 activations and of their scales: a_perm[row] = hidden[token],
// a_scale_perm[kb][row] = hidden_scale[kb][token].  One warp per row, grid-stride.
__global__ void __launch_bounds__(256) gather_kernel(const uint8_t* __restrict__ hidden, const float* __restrict__ hscale,
                                                     const int32_t* __restrict__ row_token, const int* __restrict__ status,
                                                     uint8_t* __restrict__ a_perm, float* __restrict__ a_scale_perm,
                                                     int T, int H, int rows_cap) {
    pdl_wait();
    pdl_launch();
    const int rows = status[ST_ROWS];
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int KB = H >> 7;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const int t = row_token[r];
        uint4* dst = reinterpret_cast<uint4*>(a_perm + (size_t)r * H);
        if (t < 0) continue;   // padding rows stay unwritten: their columns are never stored by the GEMMs
        const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * H);
        for (int i = lane; i < H / 16; i += 32) dst[i] = __ldg(src + i);
        for (int kb = lane; kb < KB; kb += 32) a_scale_perm[(size_t)kb * rows_cap + r] = __ldg(hscale + (size_t)kb * T + t);
    }
}

// y holds fp32 rows (bf16 rows were tried: halves this kernel's traffic, but the extra rounding of
// up to eight partial rows pushed 1 element in 6.4 million over the 1e-2 / 1e-2 tolerance).
// out[t, :] = sum over the token's local pairs (ascending expert order = the order they were
// placed in topk rows is NOT sorted, so sort the <= 8 rows by row index, which is expert
// order) of y[row, :]; fp32 accumulation, one rounding.  Tokens without a local pair get zeros.
template <bool OUT_BF16>
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ topk_idx,
                                                      const int32_t* __restrict__ pair_row, void* __restrict__ out,
                                                      int T, int H, int top_k, int local_offset, int num_local) {
    __shared__ int s_rows[8];
    __shared__ int s_n;
    pdl_wait();
    pdl_launch();
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        __syncthreads();
        if (threadIdx.x < 32) {
            // lanes 0..top_k-1 fetch their pair in parallel; rows are ranked by row index (= expert order)
            const int lane = threadIdx.x;
            int r = 0x7FFFFFFF;
            if (lane < top_k) {
                const int le = topk_idx[(size_t)t * top_k + lane] - local_offset;
                if (le >= 0 && le < num_local) r = pair_row[(size_t)t * top_k + lane];
            }
            int rank = 0;
            for (int j = 0; j < 8; ++j) {
                const int rj = __shfl_sync(0xFFFFFFFFu, r, j);
                rank += (rj < r) || (rj == r && j < lane);
            }
            const unsigned have = __ballot_sync(0xFFFFFFFFu, r != 0x7FFFFFFF);
            if (r != 0x7FFFFFFF) s_rows[rank] = r;
            if (lane == 0) s_n = __popc(have);
        }
        __syncthreads();
        const int n = s_n;
        for (int h = threadIdx.x * 8; h < H; h += blockDim.x * 8) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < n; ++j) {
                const float* src = y + (size_t)s_rows[j] * H + h;
                const float4 a = *reinterpret_cast<const float4*>(src);
                const float4 b = *reinterpret_cast<const float4*>(src + 4);
                acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
                acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
            }
            if (OUT_BF16) {
                uint4 pk;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)t * H + h) = pk;
            } else {
                float* o = reinterpret_cast<float*>(out) + (size_t)t * H + h;
                *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
        }
    }
}

}  // namespace b200moe
