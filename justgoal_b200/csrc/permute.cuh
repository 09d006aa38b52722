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
#include <cuda_fp16.h>
#include "common.cuh"

namespace b200moe {

constexpr int ROW_ALIGN = 16;
constexpr int MAX_LOCAL = 256;
static_assert((ROW_ALIGN & (ROW_ALIGN - 1)) == 0, "row alignment is a power of two");

// status word layout (int32[8]) at the head of the workspace
enum : int { ST_ERR = 0, ST_PAIRS = 1, ST_ROWS = 2, ST_TILES = 3, ST_ACTIVE = 4,
              ST_ROUTED = 5 /* fused front end: 1 once the routing result of every token is visible */ };

struct PlanParams {
    int T, top_k, num_local, local_offset, token_tile;
    const int32_t* topk_idx;   // [T, top_k]: ids of token t start at topk_idx + t * pair_stride
    const float* topk_w;       // [T, top_k]: weights of token t start at topk_w + t * pair_stride
    int pair_stride;           // in 4-byte words: top_k for dense arrays; the row pitch when both live inside packed
                               // dispatch rows (expert-parallel slots read in place)
    int* status;               // [8]
    const int* slices;         // [ceil(T*top_k / SLICE_PAIRS)][num_local] per-slice histogram (input)
    int* counts;               // [num_local] (output: totals)
    int* expert_row0;          // [num_local + 1]
    int* tile_prefix;          // [num_local + 1]
    int32_t* pair_row;         // [T, top_k]
    int32_t* row_token;        // [rows_cap]
    float* row_w;              // [rows_cap]
    int rows_cap;
};

// Per-slice histogram of the local experts from an explicit topk_idx (the expert-parallel receive
// side, where routing ran on another rank); the routing kernel fills the same table itself.
__global__ void count_kernel(const int32_t* __restrict__ topk_idx, int n, int top_k, int pair_stride, int local_offset,
                             int num_local, int* __restrict__ slices) {
    pdl_wait();
    pdl_launch();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int t = i / top_k;
        const int le = topk_idx[(size_t)t * pair_stride + (i - t * top_k)] - local_offset;
        if (le >= 0 && le < num_local) atomicAdd(slices + (size_t)(i / SLICE_PAIRS) * num_local + le, 1);
    }
}

// Warp-parallel exclusive scan over the (<= 256) per-expert counts: lane l owns experts
// [l*per, (l+1)*per).  Fills s_row0[0..n] (first row of each expert, segments padded to
// ROW_ALIGN) and s_tiles[0..n] (exclusive prefix of token tiles); writes the totals into
// status[] when it is not null.  Must be called by the 32 lanes of one warp.
__device__ __forceinline__ void scan_counts(const int* counts, int num_local, int token_tile, int* s_row0, int* s_tiles,
                                            int* status, int tid) {
    // Runs once per launch, on a cold instruction cache: the loops stay rolled and the token tile (a power of two)
    // divides by a shift, so the code is a few dozen instructions instead of eight unrolled copies with divisions.
    const int per = (num_local + 31) / 32;
    const int tsh = 31 - __clz(token_tile);
    const int i0 = tid * per;
    int rows = 0, tiles = 0, pairs = 0, active = 0;
#pragma unroll 1
    for (int k = 0; k < per; ++k) {
        const int c = i0 + k < num_local ? counts[i0 + k] : 0;
        rows += (c + ROW_ALIGN - 1) & ~(ROW_ALIGN - 1);
        tiles += (c + token_tile - 1) >> tsh;
        pairs += c; active += c > 0;
    }
    int rows_in = rows, tiles_in = tiles;
#pragma unroll 1
    for (int off = 1; off < 32; off <<= 1) {
        const int r = __shfl_up_sync(0xFFFFFFFFu, rows_in, off);
        const int t = __shfl_up_sync(0xFFFFFFFFu, tiles_in, off);
        if (tid >= off) { rows_in += r; tiles_in += t; }
    }
#pragma unroll 1
    for (int off = 16; off; off >>= 1) {
        pairs += __shfl_xor_sync(0xFFFFFFFFu, pairs, off);
        active += __shfl_xor_sync(0xFFFFFFFFu, active, off);
    }
    int r0 = rows_in - rows, t0 = tiles_in - tiles;       // exclusive prefixes of this lane
#pragma unroll 1
    for (int k = 0; k < per; ++k) {
        const int i = i0 + k;
        if (i < num_local) {
            const int c = counts[i];
            s_row0[i] = r0; s_tiles[i] = t0;
            r0 += (c + ROW_ALIGN - 1) & ~(ROW_ALIGN - 1);
            t0 += (c + token_tile - 1) >> tsh;
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

// One CTA per slice of SLICE_PAIRS pairs, one thread per pair.  Every CTA sums the per-slice
// histograms (totals -> the same scan in every CTA; slices before its own -> where its pairs start
// inside each expert's segment), ranks its own pairs per expert in pair order (match + popcount inside
// a warp, a prefix over the 32 warps) and places them.  No CTA waits for another; CTA 0 publishes the
// tables and marks the padding rows.
constexpr int PERMUTE_THREADS = SLICE_PAIRS;
__global__ void __launch_bounds__(PERMUTE_THREADS) permute_kernel(const PlanParams p) {
    __shared__ int s_cnt[MAX_LOCAL];
    __shared__ int s_before[MAX_LOCAL];
    __shared__ int s_row0[MAX_LOCAL + 1];
    __shared__ int s_tiles[MAX_LOCAL + 1];
    __shared__ int s_wcnt[32][MAX_LOCAL + 1];      // [warp][expert]; odd stride: a column walk hits 32 banks
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x, NS = gridDim.x, El = p.num_local;
    const unsigned FULL = 0xFFFFFFFFu;
    for (int i = tid; i < 32 * El; i += PERMUTE_THREADS) s_wcnt[i / El][i % El] = 0;
    pdl_wait();
    pdl_launch();

    for (int e = warp; e < El; e += 32) {
        int tot = 0, before = 0;
        for (int s = lane; s < NS; s += 32) {
            const int v = p.slices[(size_t)s * El + e];
            tot += v;
            if (s < c) before += v;
        }
        for (int off = 16; off; off >>= 1) {
            tot += __shfl_xor_sync(FULL, tot, off);
            before += __shfl_xor_sync(FULL, before, off);
        }
        if (lane == 0) { s_cnt[e] = tot; s_before[e] = before; }
    }
    __syncthreads();
    if (warp == 0) scan_counts(s_cnt, El, p.token_tile, s_row0, s_tiles, c == 0 ? p.status : nullptr, lane);

    // this thread's pair: rank among the pairs of the same expert that precede it in the warp
    const int n = p.T * p.top_k;
    const int i = c * SLICE_PAIRS + tid;
    const int tok = i / p.top_k;
    const size_t src = (size_t)tok * p.pair_stride + (i - tok * p.top_k);      // where pair i lives in topk_idx / topk_w
    const int le = i < n ? __ldg(p.topk_idx + src) - p.local_offset : -1;
    const bool local = le >= 0 && le < El;
    const unsigned same = __match_any_sync(FULL, local ? le : -1 - lane);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (local && rank == 0) s_wcnt[warp][le] = __popc(same);
    __syncthreads();
    // exclusive prefix over the warps, per expert: lane w of a warp holds warp w's count
    for (int e = warp; e < El; e += 32) {
        const int v = s_wcnt[lane][e];
        int inc = v;
        for (int off = 1; off < 32; off <<= 1) {
            const int u = __shfl_up_sync(FULL, inc, off);
            if (lane >= off) inc += u;
        }
        s_wcnt[lane][e] = inc - v;
    }
    __syncthreads();

    if (c == 0) {
        for (int k = tid; k <= El; k += PERMUTE_THREADS) {
            p.expert_row0[k] = s_row0[k];
            p.tile_prefix[k] = s_tiles[k];
            if (k < El) p.counts[k] = s_cnt[k];
        }
        // padding rows of every segment carry token -1
        for (int e = warp; e < El; e += 32)
            for (int r = s_row0[e] + s_cnt[e] + lane; r < min(s_row0[e + 1], p.rows_cap); r += 32) {
                p.row_token[r] = -1; p.row_w[r] = 0.f;
            }
    }
    if (local) {
        const int r = s_row0[le] + s_before[le] + s_wcnt[warp][le] + rank;
        if (r < p.rows_cap) {
            p.pair_row[i] = r;
            p.row_token[r] = tok;
            p.row_w[r] = p.topk_w[src];
        } else {
            // only reachable with expert ids from the caller that repeat an expert inside one token's row
            atomicCAS(p.status + ST_ERR, 0, ERR_BAD_SCHEDULE);
        }
    }
}

// Expert-sorted copy of the fp8 activations and of their scales: a_perm[row] = hidden[token],
// a_scale_perm[kb][row] = hidden_scale[kb][token].  One warp per row, grid-stride.
// Source forms: the operator's layouts (row pitch H, scales K-block major in hscale[kb][token]) or - hscale ==
// nullptr - packed dispatch rows read in place (row pitch `src_pitch` bytes, the token's H/128 scales right
// behind its H fp8 bytes).
__global__ void __launch_bounds__(256) gather_kernel(const uint8_t* __restrict__ hidden, const float* __restrict__ hscale,
                                                     const int32_t* __restrict__ row_token, const int* __restrict__ status,
                                                     uint8_t* __restrict__ a_perm, float* __restrict__ a_scale_perm,
                                                     int T, int H, int rows_cap, int src_pitch) {
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
        const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * src_pitch);
        // batches of loads before their stores: several 16-byte loads in flight per lane
        constexpr int GB = 7;
        for (int i0 = lane; i0 < H / 16; i0 += 32 * GB) {
            uint4 v[GB];
#pragma unroll
            for (int u = 0; u < GB; ++u)
                if (i0 + 32 * u < H / 16) v[u] = __ldg(src + i0 + 32 * u);
#pragma unroll
            for (int u = 0; u < GB; ++u)
                if (i0 + 32 * u < H / 16) dst[i0 + 32 * u] = v[u];
        }
        if (hscale) {
            for (int kb = lane; kb < KB; kb += 32) a_scale_perm[(size_t)kb * rows_cap + r] = __ldg(hscale + (size_t)kb * T + t);
        } else {
            const float* ss = reinterpret_cast<const float*>(hidden + (size_t)t * src_pitch + H);
            for (int kb = lane; kb < KB; kb += 32) a_scale_perm[(size_t)kb * rows_cap + r] = __ldg(ss + kb);
        }
    }
}

// y holds one fp16 row per (token, expert) pair: 11 significant bits, half the traffic of fp32 rows in the
// GEMM2 epilogue and here (bf16 rows - 8 bits - were tried first: the extra rounding of up to eight rows pushed
// 1 element in 6.4 million over the 1e-2 / 1e-2 tolerance; fp16's error is an eighth of that).
// The rows are the experts' outputs WITHOUT the routing weight: the weight multiplies in fp32 here, so the routed
// scaling factor enters the result exactly once (doubling it doubles every output bit for bit).
// out[t, :] = sum over the token's local pairs (ascending expert order = the order they were
// placed in topk rows is NOT sorted, so sort the <= 8 rows by row index, which is expert
// order) of y[row, :]; fp32 accumulation, one rounding.  Tokens without a local pair get zeros.
// Output kinds: fp32 rows (no rounding), bf16 rows (the operator's output: one rounding of the whole sum), or
// fp16 rows - the PARTIAL rows of expert parallelism, which the token's owner adds up in fp32 before the one
// rounding to bf16.  fp16 carries 11 significant bits against bf16's 8 at the same two bytes: with bf16
// partials of up to four ranks per token about 3 in 100 000 output elements of the DeepSeek-V3 shape left the
// 1e-2 / 1e-2 tolerance; partial sums stay far below fp16's range (|row| of order 10).
// Expert-parallel form (slots.cap > 0): "token" t is the slot (source rank t / cap, token t % cap) of the
// peer-memory exchange; its fp16 row goes straight into that rank's buffer at slot (my_rank, token) - a plain
// store over NVLink - and slots nobody filled (first expert id < 0) are skipped.
constexpr int EP_P2P_MAX_WORLD = 16;
struct PeerPtrs { void* p[EP_P2P_MAX_WORLD]; };
struct SlotOut { PeerPtrs back; int cap; int my_rank; };

enum : int { OUT_F32 = 0, OUT_BF16 = 1, OUT_F16 = 2 };

__device__ __forceinline__ uint4 pack8_bf16(const float* a) {
    uint4 pk;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(a[2 * q], a[2 * q + 1]);
    return pk;
}
__device__ __forceinline__ uint4 pack8_f16(const float* a) {
    uint4 pk;
    __half2* o2 = reinterpret_cast<__half2*>(&pk);
#pragma unroll
    for (int q = 0; q < 4; ++q) o2[q] = __floats2half2_rn(a[2 * q], a[2 * q + 1]);
    return pk;
}
__device__ __forceinline__ void fma8_f16(float* acc, const uint4& v, float w) {
    const __half2* v2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float2 f = __half22float2(v2[q]);
        acc[2 * q] = fmaf(w, f.x, acc[2 * q]); acc[2 * q + 1] = fmaf(w, f.y, acc[2 * q + 1]);
    }
}
__device__ __forceinline__ void add8_f16(float* acc, const uint4& v) {
    const __half2* v2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float2 f = __half22float2(v2[q]);
        acc[2 * q] += f.x; acc[2 * q + 1] += f.y;
    }
}

// The combine of ONE token over 256 output columns by one warp (lane l: columns h0 + 8 l .. + 7): the same sum as
// combine_kernel below - the token's local rows in row order, weight times row in fp32, one rounding to bf16.  Used
// by the GEMM2 epilogue that delivers a token's last row (gemm.cuh); the rows were written by other CTAs of the same
// launch, so every load goes to L2 (.cg).
__device__ __forceinline__ void combine_token_slab(const __half* y, const int32_t* topk_idx, const int32_t* pair_row,
                                                   const float* row_w, __nv_bfloat16* out, int t, int H, int top_k,
                                                   int pair_stride, int local_offset, int num_local, int h0, int lane) {
    const unsigned FULL = 0xFFFFFFFFu;
    int r = 0x7FFFFFFF;
    if (lane < top_k) {
        const int le = __ldcg(topk_idx + (size_t)t * pair_stride + lane) - local_offset;
        if (le >= 0 && le < num_local) r = __ldcg(pair_row + (size_t)t * top_k + lane);
    }
    const float w = r != 0x7FFFFFFF ? __ldcg(row_w + r) : 0.f;
    int rank = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int rj = __shfl_sync(FULL, r, j);
        rank += (rj < r) || (rj == r && j < lane);
    }
    const int n = __popc(__ballot_sync(FULL, r != 0x7FFFFFFF));
    int rs = 0; float ws = 0.f;                // lane j < n: the j-th row in row order and its weight
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int rj = __shfl_sync(FULL, r, j);
        const float wj = __shfl_sync(FULL, w, j);
        const int kj = __shfl_sync(FULL, rank, j);
        if (rj != 0x7FFFFFFF && kj == lane) { rs = rj; ws = wj; }
    }
    const int h = h0 + lane * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j0 = 0; j0 < n; j0 += 4) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (j0 + u < n) {
                const int row = __shfl_sync(FULL, rs, j0 + u);
                if (h < H) v[u] = __ldcg(reinterpret_cast<const uint4*>(y + (size_t)row * H + h));
            }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (j0 + u < n) {
                const float wu = __shfl_sync(FULL, ws, j0 + u);
                if (h < H) fma8_f16(acc, v[u], wu);
            }
    }
    if (h < H) *reinterpret_cast<uint4*>(out + (size_t)t * H + h) = pack8_bf16(acc);
}

template <int OUT>
__global__ void __launch_bounds__(256) combine_kernel(const __half* __restrict__ y, const int32_t* __restrict__ topk_idx,
                                                      const int32_t* __restrict__ pair_row, const float* __restrict__ row_w,
                                                      void* __restrict__ out, int T, int H, int top_k, int pair_stride,
                                                      int local_offset, int num_local, const SlotOut slots) {
    __shared__ int s_rows[8];
    __shared__ float s_w[8];
    __shared__ int s_n;
    pdl_wait();
    pdl_launch();
    // gridDim.y CTAs share a token's columns (few tokens: more CTAs in flight, shorter latency chain per CTA)
    const int h_per = ((H / 8 + gridDim.y - 1) / gridDim.y) * 8;
    const int h_lo = blockIdx.y * h_per, h_hi = min(H, h_lo + h_per);
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        uint16_t* out_row = reinterpret_cast<uint16_t*>(out) + (size_t)t * H;      // 2-byte kinds
        if (OUT == OUT_F16 && slots.cap > 0) {
            if (topk_idx[(size_t)t * pair_stride] < 0) continue;    // same for the whole CTA
            const int r = t / slots.cap;
            out_row = static_cast<uint16_t*>(slots.back.p[r]) + ((size_t)slots.my_rank * slots.cap + (t - r * slots.cap)) * H;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // lanes 0..top_k-1 fetch their pair in parallel; rows are ranked by row index (= expert order)
            const int lane = threadIdx.x;
            int r = 0x7FFFFFFF;
            if (lane < top_k) {
                const int le = topk_idx[(size_t)t * pair_stride + lane] - local_offset;
                if (le >= 0 && le < num_local) r = pair_row[(size_t)t * top_k + lane];
            }
            int rank = 0;
            for (int j = 0; j < 8; ++j) {
                const int rj = __shfl_sync(0xFFFFFFFFu, r, j);
                rank += (rj < r) || (rj == r && j < lane);
            }
            const unsigned have = __ballot_sync(0xFFFFFFFFu, r != 0x7FFFFFFF);
            if (r != 0x7FFFFFFF) { s_rows[rank] = r; s_w[rank] = __ldg(row_w + r); }
            if (lane == 0) s_n = __popc(have);
        }
        __syncthreads();
        const int n = s_n;
        for (int h = h_lo + threadIdx.x * 8; h < h_hi; h += blockDim.x * 8) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            // four rows' loads in flight at a time (the rows are independent; the sum order stays j = 0, 1, ...)
            for (int j0 = 0; j0 < n; j0 += 4) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (j0 + u < n) v[u] = *reinterpret_cast<const uint4*>(y + (size_t)s_rows[j0 + u] * H + h);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (j0 + u < n) fma8_f16(acc, v[u], s_w[j0 + u]);
            }
            if (OUT == OUT_BF16) {
                *reinterpret_cast<uint4*>(out_row + h) = pack8_bf16(acc);
            } else if (OUT == OUT_F16) {
                *reinterpret_cast<uint4*>(out_row + h) = pack8_f16(acc);
            } else {
                float* o = reinterpret_cast<float*>(out) + (size_t)t * H + h;
                *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
        }
    }
}

// Expert-parallel dispatch rows.  One row on the wire carries everything the receiving rank needs for
// one token: [H fp8 bytes | H/128 fp32 scales | top_k int32 expert ids | top_k fp32 weights], padded to
// 16 bytes - so the dispatch is ONE all-to-all instead of four.
__host__ __device__ inline int ep_row_bytes(int H, int top_k) { return (H + 4 * (H >> 7) + 8 * top_k + 15) & ~15; }

// pack: wire[i] = row of token send_token[i].  One warp per row.
__global__ void __launch_bounds__(256) ep_pack_kernel(const uint8_t* __restrict__ hidden, const float* __restrict__ hscale,
                                                      const int32_t* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                                      const long long* __restrict__ send_token, int n, int T, int H,
                                                      int top_k, uint8_t* __restrict__ wire) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int KB = H >> 7, rb = ep_row_bytes(H, top_k);
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
        const int t = (int)send_token[i];
        uint8_t* dst = wire + (size_t)i * rb;
        const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * H);
        for (int c = lane; c < H / 16; c += 32) reinterpret_cast<uint4*>(dst)[c] = __ldg(src + c);
        float* ds = reinterpret_cast<float*>(dst + H);
        for (int kb = lane; kb < KB; kb += 32) ds[kb] = __ldg(hscale + (size_t)kb * T + t);
        if (lane < top_k) {
            reinterpret_cast<int32_t*>(dst + H + 4 * KB)[lane] = topk_idx[(size_t)t * top_k + lane];
            reinterpret_cast<float*>(dst + H + 4 * KB + 4 * top_k)[lane] = topk_w[(size_t)t * top_k + lane];
        }
    }
}

// unpack: the received rows back into the operator's layouts (scales K-block major).  One warp per row.
__global__ void __launch_bounds__(256) ep_unpack_kernel(const uint8_t* __restrict__ wire, int n, int H, int top_k,
                                                        uint8_t* __restrict__ hidden, float* __restrict__ hscale,
                                                        int32_t* __restrict__ topk_idx, float* __restrict__ topk_w) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int KB = H >> 7, rb = ep_row_bytes(H, top_k);
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
        const uint8_t* src = wire + (size_t)i * rb;
        uint4* dst = reinterpret_cast<uint4*>(hidden + (size_t)i * H);
        for (int c = lane; c < H / 16; c += 32) dst[c] = __ldg(reinterpret_cast<const uint4*>(src) + c);
        const float* ss = reinterpret_cast<const float*>(src + H);
        for (int kb = lane; kb < KB; kb += 32) hscale[(size_t)kb * n + i] = ss[kb];
        if (lane < top_k) {
            topk_idx[(size_t)i * top_k + lane] = reinterpret_cast<const int32_t*>(src + H + 4 * KB)[lane];
            topk_w[(size_t)i * top_k + lane] = reinterpret_cast<const float*>(src + H + 4 * KB + 4 * top_k)[lane];
        }
    }
}

// Expert-parallel combine on the owner rank: out[t] = sum over ranks r with row_of[r][t] >= 0 of
// back[row_of[r][t]] (fp16 partial rows received from the ranks that own the token's experts), fp32,
// ascending rank order, one rounding to bf16.  One CTA per token, 16 bytes per thread and step.
constexpr int EP_MAX_WORLD = 64;
__global__ void __launch_bounds__(256) ep_combine_kernel(const __half* __restrict__ back,
                                                         const int32_t* __restrict__ row_of, int world, int T, int H,
                                                         __nv_bfloat16* __restrict__ out) {
    __shared__ int s_row[EP_MAX_WORLD];
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        __syncthreads();
        if (threadIdx.x < world) s_row[threadIdx.x] = row_of[(size_t)threadIdx.x * T + t];
        __syncthreads();
        for (int h = threadIdx.x * 8; h < H; h += blockDim.x * 8) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < world; ++r) {
                const int row = s_row[r];
                if (row < 0) continue;
                add8_f16(acc, __ldg(reinterpret_cast<const uint4*>(back + (size_t)row * H + h)));
            }
            *reinterpret_cast<uint4*>(out + (size_t)t * H + h) = pack8_bf16(acc);
        }
    }
}

}  // namespace b200moe
