// Routing kernels: one warp per token, lane l owns experts [l*VPT, (l+1)*VPT).
//
// DeepSeek-V3 mode follows the operator definition: s = 1/(1+exp(-x)) in fp32, v = s + bias,
// group score = sum of the two largest v of a group, keep `topk_group` groups (rank by score
// descending, group index ascending on ties), then `top_k` rounds of arg-max over the kept
// experts (lower expert id wins ties), weights = s / (sum of selected s + 1e-20) * factor,
// computed from the UNBIASED sigmoid.  The reference kernels state the same rules
// (goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/moe_common.cuh:271-365,
//  kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/kernel.cu:125-204).
// The other modes are the remaining routing methods of the same operator family (published with
// the definition as softmax -> top-k "default", top-k -> softmax "renormalize", Llama-4 top-1 ->
// sigmoid, and plain top-k with uniform weights); the reference corpus only ships the DeepSeek
// variant, so those follow the published definitions alone.  In all of them the bias, when
// given, is added to the logits before anything else.
// All comparisons and arithmetic are IEEE fp32 (this file must not be built with fast-math);
// exp is evaluated in fp64 and rounded once so that the fp32 result is the correctly rounded
// one wherever the host's exp is.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"

namespace b200moe {

// routing modes (B200MOE_ROUTING_* in the C header)
enum : int { RM_DEEPSEEK = 0, RM_RENORM_NAIVE = 1, RM_DEFAULT = 2, RM_RENORMALIZE = 3, RM_LLAMA4 = 4, RM_TOPK = 5,
             RM_COUNT = 6 };

struct RouteParams {
    const float* logits;          // [T, E]
    const __nv_bfloat16* bias;    // [E] or nullptr
    int T, E, top_k, n_group, topk_group;
    int local_offset, num_local;
    float scale;                  // routed scaling factor
    int32_t* topk_idx;            // [T, top_k]
    float* topk_w;                // [T, top_k]
    int* slices;                  // [slices][num_local] histogram per slice of SLICE_PAIRS pairs (+= 1 per local pair) or nullptr
};

// Monotone map float -> uint32 (larger float <=> larger key); NaN ordering is unspecified.
__device__ __forceinline__ uint32_t ordered_key(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exp() in double precision, rounded to float.  One out-of-line copy of the double-precision routine: inlined at its
// eight call sites it measured the same, with eight times the code.
__device__ __noinline__ float exp_f64(float x) { return (float)exp((double)x); }

// Routes token t with one warp.  On return lane r < top_k holds selection r: the global expert
// id in sel_id and its weight in w.
template <int VPT, int MODE>
__device__ __forceinline__ void route_token(const RouteParams& p, int t, int lane, int& sel_id, float& w) {
    const unsigned FULL = 0xFFFFFFFFu;

    float s[VPT];   // value the weights are taken from (sigmoid / softmax probability)
    float v[VPT];   // value the selection ranks by
    const float* row = p.logits + (size_t)t * p.E + lane * VPT;
#pragma unroll
    for (int i = 0; i < VPT; ++i) s[i] = __ldg(row + i);

    bool kept = true;
    if (MODE == RM_DEEPSEEK) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const float e = exp_f64(-s[i]);
            s[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
            const float b = p.bias ? __bfloat162float(p.bias[lane * VPT + i]) : 0.0f;
            v[i] = __fadd_rn(s[i], b);
        }
        // top-2 of the group: local, then butterfly over the lanes of the group
        const int lanes_per_group = (p.E / p.n_group) / VPT;
        float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (v[i] > m1) { m2 = m1; m1 = v[i]; } else if (v[i] > m2) { m2 = v[i]; }
        }
        for (int off = 1; off < lanes_per_group; off <<= 1) {
            const float o1 = __shfl_xor_sync(FULL, m1, off);
            const float o2 = __shfl_xor_sync(FULL, m2, off);
            const float hi = fmaxf(m1, o1);
            const float lo = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
            m1 = hi; m2 = lo;
        }
        const float gscore = __fadd_rn(m1, m2);
        const int my_group = lane / lanes_per_group;
        int better = 0;
        for (int g = 0; g < p.n_group; ++g) {
            const float og = __shfl_sync(FULL, gscore, g * lanes_per_group);
            better += (og > gscore) || (og == gscore && g < my_group);
        }
        kept = better < p.topk_group;
    } else if (MODE == RM_RENORM_NAIVE || MODE == RM_DEFAULT) {
        // softmax over all experts; the selection ranks by the probabilities
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (p.bias) s[i] = __fadd_rn(s[i], __bfloat162float(p.bias[lane * VPT + i]));
            mx = fmaxf(mx, s[i]);
        }
        for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, off));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) { s[i] = exp_f64(__fsub_rn(s[i], mx)); sum += s[i]; }
        for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(FULL, sum, off);
#pragma unroll
        for (int i = 0; i < VPT; ++i) { s[i] = __fdiv_rn(s[i], sum); v[i] = s[i]; }
    } else {
        // top-k on the raw (biased) logits; the weights come from the selected logits afterwards
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (p.bias) s[i] = __fadd_rn(s[i], __bfloat162float(p.bias[lane * VPT + i]));
            v[i] = s[i];
        }
    }

    uint32_t key[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) key[i] = kept ? ordered_key(v[i]) : 0u;  // 0 < every real key

    sel_id = -1;            // lane r < top_k ends up holding selection r
    float sel_s = 0.f;
    float ssum = 0.f;
    for (int r = 0; r < p.top_k; ++r) {
        uint32_t best = 0; int bi = 0;
#pragma unroll
        for (int i = VPT - 1; i >= 0; --i) if (key[i] >= best) { best = key[i]; bi = i; }  // lowest i on ties
        const uint32_t wmax = __reduce_max_sync(FULL, best);
        const unsigned who = __ballot_sync(FULL, best == wmax);
        const int win = __ffs(who) - 1;
        float sv = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) if (i == bi) sv = s[i];
        const int wi = __shfl_sync(FULL, bi, win);
        const float ws = __shfl_sync(FULL, sv, win);
        if (lane == win) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) if (i == bi) key[i] = 0u;
        }
        // a real key is never 0, so key 0 marks "taken"; with fewer candidates than top_k the
        // remaining rounds would re-pick taken slots, which the shapes accepted by the host exclude
        if (lane == r) { sel_id = win * VPT + wi; sel_s = ws; }
        ssum = __fadd_rn(ssum, ws);
    }
    if (MODE == RM_DEEPSEEK || MODE == RM_RENORM_NAIVE) {
        w = __fmul_rn(__fdiv_rn(sel_s, __fadd_rn(ssum, 1e-20f)), p.scale);
    } else if (MODE == RM_DEFAULT) {
        w = __fmul_rn(sel_s, p.scale);
    } else if (MODE == RM_RENORMALIZE) {
        // softmax over the top_k selected logits; selection 0 is the largest of them
        const float m0 = __shfl_sync(FULL, sel_s, 0);
        const float e = lane < p.top_k ? exp_f64(__fsub_rn(sel_s, m0)) : 0.f;
        float esum = e;
        for (int off = 16; off; off >>= 1) esum += __shfl_xor_sync(FULL, esum, off);
        w = __fmul_rn(__fdiv_rn(e, esum), p.scale);
    } else if (MODE == RM_LLAMA4) {
        const float e = exp_f64(-sel_s);
        w = __fmul_rn(__fdiv_rn(1.0f, __fadd_rn(1.0f, e)), p.scale);
    } else {
        w = (float)((double)p.scale / (double)p.top_k);
    }
}

template <int VPT, int MODE>
__global__ void __launch_bounds__(256) route_kernel(const RouteParams p) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_wait();
    pdl_launch();
    if (t >= p.T) return;
    int sel_id; float w;
    route_token<VPT, MODE>(p, t, lane, sel_id, w);
    if (lane < p.top_k) {
        p.topk_idx[(size_t)t * p.top_k + lane] = sel_id;
        p.topk_w[(size_t)t * p.top_k + lane] = w;
        const int le = sel_id - p.local_offset;
        if (p.slices && le >= 0 && le < p.num_local)
            atomicAdd(p.slices + (size_t)((t * p.top_k + lane) / SLICE_PAIRS) * p.num_local + le, 1);
    }
}

}  // namespace b200moe
