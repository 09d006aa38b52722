// Expert-parallel exchange over peer memory (NVLink), without a library collective in the data path.
//
// Every rank owns one symmetric buffer (same layout on all ranks, mapped into every peer):
//   flags  uint32[EP_P2P_MAX_WORLD]        arrival flags of the barrier, flags[r] is written by rank r
//   wire   [world][cap] dispatch rows      slot (source rank, token of that rank): what others pushed to me
//   back   [world][cap][H] fp16            slot (expert rank, my token): partial results pushed back to me
// A step: push (each token's row is stored straight into the wire slot of every rank that owns one of
// its experts; the other ranks' slots get the marker id -1) -> barrier -> unpack + local experts ->
// return (fp16 partial rows stored straight into the owner's back slot) -> barrier -> owner sums.
// Only plain peer stores cross NVLink (no multimem, no TMA on peer memory).  The barrier is a flag
// exchange with release/acquire at system scope; its wait is bounded like every wait in this library
// (gives up after the handle's wait limit - 2 s unless b200moe_set_wait_limit_ns changed it - records
// ERR_WAIT_PEER and returns; the step's result is then invalid).
// The reference has no distributed code; nothing here has a counterpart in it.
#pragma once
#include "permute.cuh"

namespace b200moe {

constexpr int ERR_WAIT_PEER = 7;           // a rank gave up waiting for a peer's barrier flag
// (EP_P2P_MAX_WORLD and PeerPtrs live in permute.cuh: the combine kernel stores into peer slots too)

// push: one warp per token slot t < cap of this rank.  Tokens t >= T (a step with fewer tokens than the
// slots hold) are marked absent everywhere.
__global__ void __launch_bounds__(256) ep_push_kernel(const uint8_t* __restrict__ hidden, const float* __restrict__ hscale,
                                                      const int32_t* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                                      int T, int cap, int H, int top_k, int experts_per_rank, int world,
                                                      int my_rank, PeerPtrs wire) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int KB = H >> 7, rb = ep_row_bytes(H, top_k);
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < cap; t += warps) {
        int id = -1; float wt = 0.f;
        if (t < T && lane < top_k) { id = topk_idx[(size_t)t * top_k + lane]; wt = topk_w[(size_t)t * top_k + lane]; }
        const int dst_of_lane = id >= 0 ? id / experts_per_rank : -1;
        for (int r = 0; r < world; ++r) {
            const bool has = __ballot_sync(0xFFFFFFFFu, dst_of_lane == r) != 0u;
            uint8_t* dst = static_cast<uint8_t*>(wire.p[r]) + ((size_t)my_rank * cap + t) * rb;
            int32_t* did = reinterpret_cast<int32_t*>(dst + H + 4 * KB);
            if (!has) {
                if (lane < top_k) did[lane] = -1;
                continue;
            }
            const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * H);
            for (int c = lane; c < H / 16; c += 32) reinterpret_cast<uint4*>(dst)[c] = __ldg(src + c);
            float* ds = reinterpret_cast<float*>(dst + H);
            for (int kb = lane; kb < KB; kb += 32) ds[kb] = __ldg(hscale + (size_t)kb * T + t);
            if (lane < top_k) {
                did[lane] = id;
                reinterpret_cast<float*>(dst + H + 4 * KB + 4 * top_k)[lane] = wt;
            }
        }
    }
}

// barrier: rank `my_rank` writes `epoch` into flags[my_rank] of every rank, then waits until its own
// flags[r] has reached `epoch` for every r.  One warp.  Epochs only grow, so flags are never reset.
__global__ void __launch_bounds__(32) ep_barrier_kernel(PeerPtrs flags, int world, int my_rank, uint32_t epoch, int* status,
                                                        unsigned long long limit_ns) {
    const int r = threadIdx.x;
    __threadfence_system();            // everything this rank stored before the barrier, to every peer
    if (r < world) {
        uint32_t* remote = static_cast<uint32_t*>(flags.p[r]) + my_rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
        const uint32_t* mine = static_cast<const uint32_t*>(flags.p[my_rank]) + r;
        const unsigned long long t0 = globaltimer_ns();
        for (uint32_t it = 1;; ++it) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - epoch) >= 0) break;
            if ((it & 0x3Fu) == 0 && globaltimer_ns() - t0 > limit_ns) {
                atomicCAS(status, 0, ERR_WAIT_PEER);       // give up: the kernel returns, the host reads the word
                break;
            }
        }
    }
    __threadfence_system();
}

// unpack of the wire slots (like ep_unpack_kernel), skipping the payload of absent slots: their ids are -1,
// which every later kernel treats as "no local expert".
__global__ void __launch_bounds__(256) ep_unpack_slots_kernel(const uint8_t* wire, int n, int H, int top_k,
                                                              uint8_t* __restrict__ hidden, float* __restrict__ hscale,
                                                              int32_t* __restrict__ topk_idx, float* __restrict__ topk_w) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int KB = H >> 7, rb = ep_row_bytes(H, top_k);
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
        const uint8_t* src = wire + (size_t)i * rb;
        const int32_t* sid = reinterpret_cast<const int32_t*>(src + H + 4 * KB);
        const bool present = sid[0] >= 0;
        if (lane < top_k) {
            topk_idx[(size_t)i * top_k + lane] = present ? sid[lane] : -1;
            topk_w[(size_t)i * top_k + lane] = present ? reinterpret_cast<const float*>(src + H + 4 * KB + 4 * top_k)[lane] : 0.f;
        }
        if (!present) continue;
        uint4* dst = reinterpret_cast<uint4*>(hidden + (size_t)i * H);
        for (int c = lane; c < H / 16; c += 32) dst[c] = reinterpret_cast<const uint4*>(src)[c];
        const float* ss = reinterpret_cast<const float*>(src + H);
        for (int kb = lane; kb < KB; kb += 32) hscale[(size_t)kb * n + i] = ss[kb];
    }
}

// return: result row of slot (source rank r, token t) -> rank r's back slot (my_rank, t).  One warp per slot.
__global__ void __launch_bounds__(256) ep_return_kernel(const __half* __restrict__ part, const int32_t* __restrict__ topk_idx,
                                                        int cap, int H, int top_k, int world, int my_rank, PeerPtrs back) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int n = world * cap;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
        if (topk_idx[(size_t)i * top_k] < 0) continue;
        const int r = i / cap, t = i - r * cap;
        const uint4* src = reinterpret_cast<const uint4*>(part + (size_t)i * H);
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(back.p[r]) + ((size_t)my_rank * cap + t) * H);
        for (int c = lane; c < H / 8; c += 32) dst[c] = __ldg(src + c);
    }
}

// owner-side sum over the back slots: like ep_combine_kernel, the set of ranks that hold a share of token t
// is recomputed from the token's own expert ids.
__global__ void __launch_bounds__(256) ep_combine_slots_kernel(const __half* back,
                                                               const int32_t* __restrict__ topk_idx, int T, int cap, int H,
                                                               int top_k, int experts_per_rank, int world,
                                                               __nv_bfloat16* __restrict__ out) {
    __shared__ int s_has[EP_P2P_MAX_WORLD];
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        __syncthreads();
        if (threadIdx.x < world) {
            int has = 0;
            for (int k = 0; k < top_k; ++k) has |= (topk_idx[(size_t)t * top_k + k] / experts_per_rank) == (int)threadIdx.x;
            s_has[threadIdx.x] = has;
        }
        __syncthreads();
        for (int h = threadIdx.x * 8; h < H; h += blockDim.x * 8) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < world; ++r) {
                if (!s_has[r]) continue;
                add8_f16(acc, *reinterpret_cast<const uint4*>(back + ((size_t)r * cap + t) * H + h));
            }
            *reinterpret_cast<uint4*>(out + (size_t)t * H + h) = pack8_bf16(acc);
        }
    }
}

}  // namespace b200moe
