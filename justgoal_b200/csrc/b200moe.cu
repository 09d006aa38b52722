// Host side of libb200moe: the C ABI declared in include/b200moe.h.
//
// Mirrors the job of the reference's host launcher (shape checks, tensor-map encoding, kernel
// family choice by token count, launches on the caller's stream, integer return codes:
// kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/kernel.cu:5336-5682,
// goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/moe_host.cu:88-183) for kernels written from
// scratch for sm_100a.  No torch types, no allocation inside forward, no host synchronisation
// except in b200moe_status.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

#include "b200moe.h"
#include "common.cuh"
#include "front.cuh"
#include "ep_p2p.cuh"
#include "gemm.cuh"
#include "gemm_pair.cuh"
#include "permute.cuh"
#include "quant.cuh"
#include "routing.cuh"

using namespace b200moe;

constexpr int PROF_POINTS = 7;   // before route, after route, permute, gather, gemm1, gemm2, combine

struct b200moe_ctx {
    b200moe_config cfg;
    int device;
    int num_sms;
    int prof_slots;            // 0 = profiling off
    long long prof_calls;      // forwards recorded since profiling was enabled
    cudaEvent_t* prof_events;  // [prof_slots][PROF_POINTS]
    int ablate;                // B200MOE_ABLATE environment variable at create (timing experiments; 0 in normal use)
    unsigned long long wait_limit_ns;   // limit of the waits on a PEER (barrier flags); b200moe_set_wait_limit_ns
    int pair_grid[2];          // CTAs of the SM-pair kernels (GEMM1, GEMM2): 2 x clusters that can be resident; 0 = unusable
    int token_tile;            // b200moe_set_token_tile: 0 = chosen from the token count, else 16 / 32 / 64 / 128
    int tma_gather;            // b200moe_set_tma_gather: GEMM1 (128-token tiles) gathers its token rows by TMA; default off
    int fuse_combine;          // b200moe_set_fused_combine: GEMM2 epilogue adds a token's rows up (narrow tiles); default off
    int* d_sync;               // device, 64 bytes, zero between calls: the meeting words of the fused front end
                               // (front.cuh).  One forward per handle may be in flight at a time.
};

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// All kernels of a forward are launched with programmatic stream serialization (unless
// B200MOE_PDL=0): the next kernel's prologue overlaps the tail of the one before, and each
// kernel calls griddepcontrol.wait before it touches anything an earlier kernel wrote.
// B200MOE_PDL is a bit mask over the launch sites (1 route/count, 2 permute, 4 gather, 8 GEMM1,
// 16 GEMM2, 32 combine); default: all.
enum : int { PDL_ROUTE = 1, PDL_PERMUTE = 2, PDL_GATHER = 4, PDL_GEMM1 = 8, PDL_GEMM2 = 16, PDL_COMBINE = 32 };
int pdl_mask() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("B200MOE_PDL"); v = e ? atoi(e) : 63; }
    return v;
}

// Measured: with thousands of tokens the early-resident dependents slow the front kernels down
// (2.17 ms against 1.93 ms at T=4096), with a few dozen tokens the overlap saves ~9 us per forward.
// So the forward turns the attribute on only for small token counts (a shape-only decision).
thread_local int g_call_pdl = 0;
inline void set_call_pdl(int num_tokens) { g_call_pdl = num_tokens <= 512 ? pdl_mask() : 0; }

template <typename... KArgs, typename... Args>
cudaError_t launch_k(int site, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = (g_call_pdl & site) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// 2-D byte tensor [rows][cols] (cols contiguous), box [box_rows][128 bytes], 128-byte swizzle.
int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint64_t pitch = 0) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return B200MOE_E_DRIVER;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch ? pitch : cols};       // bytes between rows (a multiple of 16)
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    static int promo = -1;
    if (promo < 0) { const char* e = getenv("B200MOE_L2PROMO"); promo = e ? atoi(e) : 3; }
    const CUtensorMapL2promotion pm = promo == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                    : promo == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                    : promo == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                 : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, pm,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : B200MOE_E_DRIVER;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Tokens per GEMM tile, from shapes only (never from data): the expected number of rows per
// expert under uniform routing.
// slices of SLICE_PAIRS (token, expert) pairs = CTAs of the permutation kernel (at least one)
int num_slices(const b200moe_config& c, int T) {
    const long long n = (long long)T * c.top_k;
    return n <= 0 ? 1 : (int)((n + SLICE_PAIRS - 1) / SLICE_PAIRS);
}

// Measured on the DeepSeek-V3 shape with 32 local experts (microseconds per forward, tile 16 / 32 / 64 / 128):
// T=64 149/160/202/187, T=192 211/230/244/225, T=256 230/214/244/227, T=320 247/244/245/219, T=512 308/284/292/279,
// T=1024 482/372/353/301, T=1792 -/-/463/372.  The 16-token tile wins while an expert sees fewer rows than the tile
// holds; from about nine expected rows per expert the 128-token tile (tokens on M, one N = 256 MMA per K step) is
// ahead of every narrower one although most of its rows are padding - the step is bound by the weight stream, and
// the narrow tiles' weights-on-M MMAs are short of shared-memory bandwidth from 64 columns on.  The 64-token tile is
// never the best choice; it stays available through b200moe_set_token_tile.
int pick_token_tile(const b200moe_ctx* h, int T) {
    if (h->token_tile) return h->token_tile;
    const b200moe_config& c = h->cfg;
    const double avg = (double)T * c.top_k / c.num_experts;
    if (avg <= 7.0) return 16;
    if (avg <= 9.0) return 32;
    return 128;
}

// Partial-sum slots of the chunked units: (fewer than grid units) x (chunks per unit) x (floats per slot), the larger
// of the two GEMMs (they run one after the other and share the area).
template <int NTOK>
size_t sk_partial_bytes_ntok(const b200moe_config& c, int grid) {
    using C1 = GemmCfg<NTOK, true>; using C2 = GemmCfg<NTOK, false>;
    const size_t a = (size_t)chunks_per_unit(c.hidden / 128, C1::KPB, C1::CHUNK_GROUPS) * C1::SLOT_FLOATS;
    const size_t b = (size_t)chunks_per_unit(c.intermediate / 128, C2::KPB, C2::CHUNK_GROUPS) * C2::SLOT_FLOATS;
    return (a > b ? a : b) * (size_t)grid * 4;
}
size_t sk_partial_bytes(const b200moe_config& c, int grid, int ntok) {
    switch (ntok) {
        case 16: return sk_partial_bytes_ntok<16>(c, grid);
        case 32: return sk_partial_bytes_ntok<32>(c, grid);
        case 64: return sk_partial_bytes_ntok<64>(c, grid);
        default: return sk_partial_bytes_ntok<128>(c, grid);
    }
}

int rows_capacity_for(const b200moe_config& c, int T) {
    const long long per_tok = c.top_k < c.num_local_experts ? c.top_k : c.num_local_experts;
    long long rows = (long long)T * per_tok + (long long)ROW_ALIGN * c.num_local_experts;
    rows = (rows + 127) / 128 * 128 + 128;
    return (int)rows;
}

void layout(const b200moe_ctx* h, int T, b200moe_ws_layout* L) {
    const b200moe_config& c = h->cfg;
    const size_t A = 256;
    const int El = c.num_local_experts, K = c.top_k;
    const size_t rows = (size_t)rows_capacity_for(c, T);
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, A); return o; };
    L->status = take(8 * 4);
    L->counts = take((size_t)El * 4);
    L->sk_count = take((size_t)2 * (4 * h->num_sms + 4) * 4); // [GEMM1 | GEMM2][4 * grid + 4]; zeroed with the head
    L->slices = take((size_t)num_slices(c, T) * El * 4);      // zeroed with the head
    // narrow token tiles: the combine is fused into GEMM2 and counts row deliveries per (token, 256 output columns)
    L->tok_count = take(pick_token_tile(h, T) < 128 ? (size_t)T * ((c.hidden + 255) / 256) * 4 : 0);   // zeroed with the head
    L->expert_row0 = take((size_t)(El + 1) * 4);
    L->tile_prefix = take((size_t)(El + 1) * 4);
    L->topk_idx = take((size_t)T * K * 4);
    L->topk_w = take((size_t)T * K * 4);
    L->pair_row = take((size_t)T * K * 4);
    L->row_token = take(rows * 4);
    L->row_w = take(rows * 4);
    L->a_perm = take(rows * c.hidden);
    L->a_scale_perm = take((size_t)(c.hidden / 128) * rows * 4);
    L->act_hi = take(rows * c.intermediate);
    L->act_lo = take(rows * c.intermediate);
    L->act_scale = take((size_t)(c.intermediate / 128) * rows * 4);
    L->y = take(rows * c.hidden * 2);
    L->sk_partial = take(sk_partial_bytes(c, h->num_sms, (int)pick_token_tile(h, T)));
    L->trace = take((size_t)2 * h->num_sms * TRACE_SLOTS * 8 + 2 * 8 * KLOG_N * 8);   // [GEMM1 | GEMM2][CTA][slot], then K-block logs
    L->rows_cap = rows;
    L->token_tile = (size_t)pick_token_tile(h, T);
    L->total_bytes = off;
}

template <int NTOK, bool G1, bool G4 = false>
cudaError_t set_attr() {
    using C = GemmCfg<NTOK, G1>;
    if (C::REALLOC_REGS) {
        // the kernel's setmaxnreg arithmetic assumes the launch allocation; refuse to run otherwise
        cudaFuncAttributes fa;
        cudaError_t e = cudaFuncGetAttributes(&fa, gemm_kernel<NTOK, G1, G4>);
        if (e != cudaSuccess) return e;
        if (fa.numRegs != C::LAUNCH_REGS) return (cudaError_t)(-B200MOE_E_BUILD + 100000);   // decoded by CU_TRY_ATTR
    }
    return cudaFuncSetAttribute(gemm_kernel<NTOK, G1, G4>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
}

template <int NTOK, bool G1>
cudaError_t launch_gemm(int grid, cudaStream_t st, const CUtensorMap& w, const CUtensorMap& b0, const CUtensorMap& b1,
                        const GemmParams& p) {
    return launch_k(G1 ? PDL_GEMM1 : PDL_GEMM2, gemm_kernel<NTOK, G1>, dim3(grid), dim3(GemmCfg<NTOK, G1>::NTHREADS),
                    GemmCfg<NTOK, G1>::SMEM_BYTES, st, w, b0, b1, p);
}

// GEMM1 over 128-token tiles with TMA-gathered token rows
cudaError_t launch_gemm_g4(int grid, cudaStream_t st, const CUtensorMap& w, const CUtensorMap& b0, const CUtensorMap& b1,
                           const GemmParams& p) {
    return launch_k(PDL_GEMM1, gemm_kernel<128, true, true>, dim3(grid), dim3(GemmCfg<128, true>::NTHREADS),
                    GemmCfg<128, true>::SMEM_BYTES, st, w, b0, b1, p);
}

template <bool G1>
cudaError_t launch_gemm_ntok(int ntok, int grid, cudaStream_t st, const CUtensorMap& w, const CUtensorMap& b0,
                             const CUtensorMap& b1, const GemmParams& p) {
    switch (ntok) {
        case 16: return launch_gemm<16, G1>(grid, st, w, b0, b1, p);
        case 32: return launch_gemm<32, G1>(grid, st, w, b0, b1, p);
        case 64: return launch_gemm<64, G1>(grid, st, w, b0, b1, p);
        default: return launch_gemm<128, G1>(grid, st, w, b0, b1, p);
    }
}

// SM-pair kernels (gemm_pair.cuh): clusters of two CTAs.  The grid is twice the number of clusters the device
// can hold at once (a persistent kernel with a static schedule must not queue a cluster behind another one).
template <bool G1>
cudaError_t launch_cfg_pair(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int grid, cudaStream_t st, bool pdl) {
    cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(PairCfg<G1>::NTHREADS);
    cfg.dynamicSmemBytes = PairCfg<G1>::SMEM_BYTES; cfg.stream = st;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 2 : 1;
    return cudaSuccess;
}

template <bool G1>
int set_attr_pair(int num_sms, int* grid_out) {
    using C = PairCfg<G1>;
    *grid_out = 0;
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, gemm_pair_kernel<G1>);
    if (e != cudaSuccess) return (int)e;
    if (fa.numRegs != C::LAUNCH_REGS) return B200MOE_E_BUILD;
    e = cudaFuncSetAttribute(gemm_pair_kernel<G1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[2];
    launch_cfg_pair<G1>(cfg, attr, (num_sms / 2) * 2, nullptr, false);
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<G1>, &cfg);
    if (e != cudaSuccess) { cudaGetLastError(); return 0; }       // pairs unusable on this device: single-SM kernels run
    if (clusters > num_sms / 2) clusters = num_sms / 2;
    *grid_out = clusters * 2;
    return 0;
}

template <bool G1>
cudaError_t launch_gemm_pair(int grid, cudaStream_t st, const CUtensorMap& w, const CUtensorMap& b0, const CUtensorMap& b1,
                             const GemmParams& p) {
    cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[2];
    launch_cfg_pair<G1>(cfg, attr, grid, st, (g_call_pdl & (G1 ? PDL_GEMM1 : PDL_GEMM2)) != 0);
    return cudaLaunchKernelEx(&cfg, gemm_pair_kernel<G1>, w, b0, b1, p);
}

// Full token tiles run on SM pairs when B200MOE_PAIR=1.  Off by default: measured on B200, both families run
// into the 1 kW power cap within milliseconds, and at the clocks the cap leaves (~1.45-1.55 GHz) the pair
// kernels are 8 % (GEMM1) / 0 % (GEMM2) slower than the single-SM ones although they need fewer cycles per
// 128-K block at full clock (1008 against 1180).
bool use_pairs(const b200moe_ctx* h, int ntok) {
    static int v = -1;
    if (v < 0) { const char* e = getenv("B200MOE_PAIR"); v = e ? atoi(e) : 0; }
    return v != 0 && ntok == 128 && h->pair_grid[0] >= 2 && h->pair_grid[1] >= 2;
}

bool cfg_ok(const b200moe_config& c) {
    if (c.hidden <= 0 || c.hidden % 128 || c.intermediate <= 0 || c.intermediate % 128) return false;
    if (c.num_experts <= 0 || c.num_experts % 32 || c.num_experts > 512) return false;
    const int vpt = c.num_experts / 32;
    if (vpt != 1 && vpt != 2 && vpt != 4 && vpt != 8 && vpt != 16) return false;
    if (c.num_local_experts <= 0 || c.num_local_experts > MAX_LOCAL || c.num_local_experts > c.num_experts) return false;
    if (c.top_k <= 0 || c.top_k > 8 || c.top_k > c.num_experts) return false;
    if (c.routing_mode == B200MOE_ROUTING_DEEPSEEK) {
        if (c.n_group <= 0 || c.num_experts % c.n_group) return false;
        const int gs = c.num_experts / c.n_group;
        if (gs % vpt) return false;                       // a group is a whole number of lanes
        const int lpg = gs / vpt;
        if (lpg & (lpg - 1)) return false;                // ... and a power of two of them
        if (gs < 2) return false;                         // group score needs two experts
        if (c.topk_group <= 0 || c.topk_group > c.n_group) return false;
        if (c.topk_group * gs < c.top_k) return false;    // enough candidates for top_k
    } else if (c.routing_mode == B200MOE_ROUTING_LLAMA4) {
        if (c.top_k != 1) return false;                   // by definition a single expert per token
    } else if (c.routing_mode < 0 || c.routing_mode >= RM_COUNT) {
        return false;
    }
    return true;
}

template <int MODE>
cudaError_t launch_route(int vpt, const RouteParams& rp, cudaStream_t st) {
    const int grid = (rp.T + 7) / 8;
    switch (vpt) {
        case 1: return launch_k(PDL_ROUTE, route_kernel<1, MODE>, dim3(grid), dim3(256), 0, st, rp);
        case 2: return launch_k(PDL_ROUTE, route_kernel<2, MODE>, dim3(grid), dim3(256), 0, st, rp);
        case 4: return launch_k(PDL_ROUTE, route_kernel<4, MODE>, dim3(grid), dim3(256), 0, st, rp);
        case 8: return launch_k(PDL_ROUTE, route_kernel<8, MODE>, dim3(grid), dim3(256), 0, st, rp);
        default: return launch_k(PDL_ROUTE, route_kernel<16, MODE>, dim3(grid), dim3(256), 0, st, rp);
    }
    return cudaGetLastError();
}

template <int MODE>
cudaError_t launch_front_route_mode(int vpt, int grid, const FrontParams& fp, const RouteParams& rp, cudaStream_t st) {
    switch (vpt) {
        case 1: return launch_k(PDL_PERMUTE, front_route_kernel<1, MODE>, dim3(grid), dim3(FRONT_THREADS), 0, st, fp, rp);
        case 2: return launch_k(PDL_PERMUTE, front_route_kernel<2, MODE>, dim3(grid), dim3(FRONT_THREADS), 0, st, fp, rp);
        case 4: return launch_k(PDL_PERMUTE, front_route_kernel<4, MODE>, dim3(grid), dim3(FRONT_THREADS), 0, st, fp, rp);
        case 8: return launch_k(PDL_PERMUTE, front_route_kernel<8, MODE>, dim3(grid), dim3(FRONT_THREADS), 0, st, fp, rp);
        default: return launch_k(PDL_PERMUTE, front_route_kernel<16, MODE>, dim3(grid), dim3(FRONT_THREADS), 0, st, fp, rp);
    }
}
cudaError_t launch_front_route(const b200moe_config& c, int grid, const FrontParams& fp, const RouteParams& rp, cudaStream_t st) {
    const int vpt = c.num_experts / 32;
    switch (c.routing_mode) {
        case B200MOE_ROUTING_DEEPSEEK: return launch_front_route_mode<RM_DEEPSEEK>(vpt, grid, fp, rp, st);
        case B200MOE_ROUTING_RENORM_NAIVE: return launch_front_route_mode<RM_RENORM_NAIVE>(vpt, grid, fp, rp, st);
        case B200MOE_ROUTING_DEFAULT: return launch_front_route_mode<RM_DEFAULT>(vpt, grid, fp, rp, st);
        case B200MOE_ROUTING_RENORMALIZE: return launch_front_route_mode<RM_RENORMALIZE>(vpt, grid, fp, rp, st);
        case B200MOE_ROUTING_LLAMA4: return launch_front_route_mode<RM_LLAMA4>(vpt, grid, fp, rp, st);
        default: return launch_front_route_mode<RM_TOPK>(vpt, grid, fp, rp, st);
    }
}

cudaError_t do_route(const b200moe_config& c, const RouteParams& rp, cudaStream_t st) {
    const int vpt = c.num_experts / 32;
    switch (c.routing_mode) {
        case B200MOE_ROUTING_DEEPSEEK: return launch_route<RM_DEEPSEEK>(vpt, rp, st);
        case B200MOE_ROUTING_RENORM_NAIVE: return launch_route<RM_RENORM_NAIVE>(vpt, rp, st);
        case B200MOE_ROUTING_DEFAULT: return launch_route<RM_DEFAULT>(vpt, rp, st);
        case B200MOE_ROUTING_RENORMALIZE: return launch_route<RM_RENORMALIZE>(vpt, rp, st);
        case B200MOE_ROUTING_LLAMA4: return launch_route<RM_LLAMA4>(vpt, rp, st);
        default: return launch_route<RM_TOPK>(vpt, rp, st);
    }
}

#define CU_TRY(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) return (int)e_; } while (0)

// Optional per-stage CUDA events (b200moe_profile_enable): point k of the current slot.
inline cudaError_t prof_mark(b200moe_ctx* h, int point, cudaStream_t st) {
    if (!h->prof_slots) return cudaSuccess;
    const long long slot = h->prof_calls % h->prof_slots;
    return cudaEventRecord(h->prof_events[slot * PROF_POINTS + point], st);
}

// Everything after routing: permute -> gather -> GEMM1 -> GEMM2 -> combine.
int run_experts(b200moe_ctx* h, const int32_t* topk_idx, const float* topk_w, const void* hidden,
                const void* hidden_scale, const void* w13, const void* s13, const void* w2, const void* s2, int T,
                int local_offset, void* out, int out_kind, uint8_t* ws, const b200moe_ws_layout& L, cudaStream_t st,
                bool fused_front = false, const SlotOut* slot_out = nullptr, int wire_pitch = 0,
                const RouteParams* route_in_front = nullptr, bool allow_fuse = false) {
    // wire_pitch > 0: the tokens are packed dispatch rows read in place - `hidden` points at the first row,
    // topk_idx / topk_w at the ids / weights inside it, rows are wire_pitch bytes apart, hidden_scale is unused
    const b200moe_config& c = h->cfg;
    const int El = c.num_local_experts, H = c.hidden, I = c.intermediate;
    const int ntok = (int)L.token_tile, rows_cap = (int)L.rows_cap;
    int* status = reinterpret_cast<int*>(ws + L.status);
    int* counts = reinterpret_cast<int*>(ws + L.counts);
    int* row0 = reinterpret_cast<int*>(ws + L.expert_row0);
    int* tiles = reinterpret_cast<int*>(ws + L.tile_prefix);
    int32_t* pair_row = reinterpret_cast<int32_t*>(ws + L.pair_row);
    int32_t* row_token = reinterpret_cast<int32_t*>(ws + L.row_token);
    float* row_w = reinterpret_cast<float*>(ws + L.row_w);
    uint8_t* a_perm = ws + L.a_perm;
    float* a_scale = reinterpret_cast<float*>(ws + L.a_scale_perm);
    uint8_t* act_hi = ws + L.act_hi;
    uint8_t* act_lo = ws + L.act_lo;
    float* act_scale = reinterpret_cast<float*>(ws + L.act_scale);
    __half* y = reinterpret_cast<__half*>(ws + L.y);

    CUtensorMap m_w13, m_w2, m_a, m_hi, m_lo;
    int rc;
    const bool pairs = use_pairs(h, ntok);
    if ((rc = make_map(&m_w13, w13, (uint64_t)El * 2 * I, H, 128))) return rc;
    if ((rc = make_map(&m_w2, w2, (uint64_t)El * H, I, 128))) return rc;
    // Optional (b200moe_set_tma_gather), 128-token tiles: GEMM1 reads the token rows straight from the caller's
    // activations with four-row TMA gathers through row_token (one-row boxes; rows `pitch` bytes apart when they sit
    // inside packed dispatch rows) - no gather copy.  Same results; measured three times slower (32 gathers per
    // 128-K block from one producer thread: ~100 ns each), so the copy stays the default.
    const bool g4 = ntok == 128 && !pairs && h->tma_gather;
    if (g4) {
        if ((rc = make_map(&m_a, hidden, (uint64_t)T, H, 1, wire_pitch > 0 ? (uint64_t)wire_pitch : 0))) return rc;
    } else if ((rc = make_map(&m_a, a_perm, rows_cap, H, ntok))) return rc;
    if ((rc = make_map(&m_hi, act_hi, rows_cap, I, ntok))) return rc;
    if ((rc = make_map(&m_lo, act_lo, rows_cap, I, ntok))) return rc;

    PlanParams pp;
    pp.T = T; pp.top_k = c.top_k; pp.num_local = El; pp.local_offset = local_offset; pp.token_tile = ntok;
    pp.topk_idx = topk_idx; pp.topk_w = topk_w; pp.status = status; pp.counts = counts;
    pp.pair_stride = wire_pitch > 0 ? wire_pitch / 4 : c.top_k;
    pp.slices = reinterpret_cast<const int*>(ws + L.slices);
    pp.expert_row0 = row0; pp.tile_prefix = tiles; pp.pair_row = pair_row; pp.row_token = row_token;
    pp.row_w = row_w; pp.rows_cap = rows_cap;
    if (fused_front) {
        // small token counts: histogram + permutation + gather in one launch (front.cuh)
        FrontParams fp;
        fp.plan = pp;
        fp.hidden = static_cast<const uint8_t*>(hidden); fp.hscale = static_cast<const float*>(hidden_scale);
        fp.a_perm = a_perm; fp.a_scale_perm = a_scale; fp.H = H;
        fp.sync = h->d_sync; fp.head = reinterpret_cast<uint4*>(ws); fp.head_vec = route_in_front ? (int)(L.expert_row0 / 16) : 0;
        // enough warps to route 128 tokens at once and to copy a few dozen rows in one pass, few enough that GEMM1 can
        // start on most SMs while this kernel runs (16 and 64 CTAs both measured slower at 64 tokens)
        const int fgrid = h->num_sms < 32 ? h->num_sms : 32;
        if (route_in_front) CU_TRY(launch_front_route(c, fgrid, fp, *route_in_front, st));
        else CU_TRY(launch_k(PDL_PERMUTE, front_small_kernel, dim3(fgrid), dim3(FRONT_THREADS), 0, st, fp));
        CU_TRY(prof_mark(h, 2, st));
        CU_TRY(prof_mark(h, 3, st));
    } else {
        CU_TRY(launch_k(PDL_PERMUTE, permute_kernel, dim3(num_slices(c, T)), dim3(PERMUTE_THREADS), 0, st, pp));
        CU_TRY(prof_mark(h, 2, st));

        if (!g4) {
        const long long max_rows = (long long)T * (c.top_k < El ? c.top_k : El) + (long long)ROW_ALIGN * El;
        int ggrid = (int)((max_rows + 7) / 8);
        if (ggrid > h->num_sms * 8) ggrid = h->num_sms * 8;
        CU_TRY(launch_k(PDL_GATHER, gather_kernel, dim3(ggrid), dim3(256), 0, st, static_cast<const uint8_t*>(hidden),
                        wire_pitch > 0 ? (const float*)nullptr : static_cast<const float*>(hidden_scale),
                        (const int32_t*)row_token, (const int*)status, a_perm, a_scale, T, H, rows_cap,
                        wire_pitch > 0 ? wire_pitch : H));
        }
        CU_TRY(prof_mark(h, 3, st));
    }

    GemmParams g1;
    memset(&g1, 0, sizeof(g1));
    g1.status = status; g1.counts = counts; g1.expert_row0 = row0; g1.tile_prefix = tiles; g1.num_local = El;
    g1.KB = H / 128; g1.n_mtiles = I / 128; g1.rows_per_expert = 2 * I; g1.gate_offset = I; g1.scale_rows = 2 * I / 128;
    g1.unit_rows = 128; g1.valid_rows = 2 * I;
    g1.w_scale = static_cast<const float*>(s13); g1.b_scale = a_scale; g1.rows_cap = rows_cap;
    g1.act_hi = act_hi; g1.act_lo = act_lo; g1.act_scale = act_scale; g1.I = I; g1.H = H;
    static int evf = -1;
    if (evf < 0) { const char* e = getenv("B200MOE_EVICT_FIRST"); evf = e ? atoi(e) : 1; }
    g1.evict_first_weights = evf && ntok < 128;
    g1.ts_stride = rows_cap;
    if (g4) {
        g1.g4_row_token = row_token; g1.g4_T = T;
        if (wire_pitch > 0) {       // scales follow the fp8 row inside a packed dispatch row
            g1.g4_scale = reinterpret_cast<const float*>(static_cast<const uint8_t*>(hidden) + H);
            g1.g4_tok_stride = wire_pitch / 4; g1.ts_stride = 1;
        } else {                    // the operator's [H/128, T] layout
            g1.g4_scale = static_cast<const float*>(hidden_scale); g1.g4_tok_stride = 1; g1.ts_stride = T;
        }
    }
    if (route_in_front && !pairs && wire_pitch == 0) {
        // the fused front end announces the routing result; GEMM1 schedules itself from it (gemm.cuh)
        g1.routed = status + ST_ROUTED; g1.topk_idx = topk_idx; g1.n_pairs = T * c.top_k; g1.local_offset = local_offset;
    }
    g1.sk_count = reinterpret_cast<int*>(ws + L.sk_count);
    g1.sk_partial = reinterpret_cast<float*>(ws + L.sk_partial);
    g1.ablate = h->ablate & 0xFF;
    g1.trace = reinterpret_cast<long long*>(ws + L.trace);
    g1.klog = g1.trace + (size_t)2 * h->num_sms * TRACE_SLOTS;
    if (pairs) CU_TRY(launch_gemm_pair<true>(h->pair_grid[0], st, m_w13, m_a, m_a, g1));
    else if (g4) CU_TRY(launch_gemm_g4(h->num_sms, st, m_w13, m_a, m_a, g1));
    else CU_TRY(launch_gemm_ntok<true>(ntok, h->num_sms, st, m_w13, m_a, m_a, g1));
    CU_TRY(prof_mark(h, 4, st));

    GemmParams g2;
    memset(&g2, 0, sizeof(g2));
    g2.status = status; g2.counts = counts; g2.expert_row0 = row0; g2.tile_prefix = tiles; g2.num_local = El;
    g2.KB = I / 128; g2.n_mtiles = (H + 255) / 256; g2.rows_per_expert = H; g2.gate_offset = 128; g2.scale_rows = H / 128;
    g2.unit_rows = 256; g2.valid_rows = H;
    g2.w_scale = static_cast<const float*>(s2); g2.b_scale = act_scale; g2.rows_cap = rows_cap;
    g2.row_w = row_w; g2.y = y; g2.H = H; g2.I = I; g2.ts_stride = rows_cap;
    g2.evict_first_weights = evf && ntok < 128;
    g2.sk_count = reinterpret_cast<int*>(ws + L.sk_count) + 4 * h->num_sms + 4;
    g2.sk_partial = g1.sk_partial;
    g2.ablate = (h->ablate >> 8) & 0xFF;
    g2.trace = g1.trace + (size_t)h->num_sms * TRACE_SLOTS;
    g2.klog = g1.klog + 8 * KLOG_N;
    // Optional (b200moe_set_fused_combine): the operator's own forward with narrow token tiles lets the GEMM2 unit that
    // delivers a token's last row add the token's rows up and write the bf16 output - no combine launch.  Same bits
    // as combine_kernel; measured 9 us slower per 64-token step (the fence, the delivery atomics and the row loads
    // sit in the epilogue of every unit, where the separate kernel pays them once), so it is off by default.
    const bool fuse = h->fuse_combine && allow_fuse && ntok < 128 && !pairs && out_kind == OUT_BF16 && !slot_out && wire_pitch == 0;
    if (fuse) {
        g2.fuse_out = static_cast<__nv_bfloat16*>(out);
        g2.tok_count = reinterpret_cast<int*>(ws + L.tok_count);
        g2.row_token = row_token; g2.pair_row = pair_row; g2.c_topk = topk_idx; g2.c_stride = pp.pair_stride;
        g2.top_k = c.top_k; g2.T = T; g2.c_local_offset = local_offset;
    }
    if (pairs) CU_TRY(launch_gemm_pair<false>(h->pair_grid[1], st, m_w2, m_hi, m_lo, g2));
    else CU_TRY(launch_gemm_ntok<false>(ntok, h->num_sms, st, m_w2, m_hi, m_lo, g2));
    CU_TRY(prof_mark(h, 5, st));

    if (fuse) {
        CU_TRY(prof_mark(h, 6, st));
        if (h->prof_slots) ++h->prof_calls;
        return 0;
    }
    const int cgrid_x = T < h->num_sms * 8 ? T : h->num_sms * 8;
    const dim3 cgrid(cgrid_x, T <= 256 ? 4 : 1);        // few tokens: four CTAs share a token's columns
    SlotOut so;
    memset(&so, 0, sizeof(so));            // cap == 0: rows go to `out`
    if (slot_out) so = *slot_out;
    if (out_kind == OUT_BF16)
        CU_TRY(launch_k(PDL_COMBINE, combine_kernel<OUT_BF16>, cgrid, dim3(256), 0, st, (const __half*)y, topk_idx,
                        (const int32_t*)pair_row, (const float*)row_w, out, T, H, c.top_k, pp.pair_stride, local_offset, El, so));
    else if (out_kind == OUT_F16)
        CU_TRY(launch_k(PDL_COMBINE, combine_kernel<OUT_F16>, cgrid, dim3(256), 0, st, (const __half*)y, topk_idx,
                        (const int32_t*)pair_row, (const float*)row_w, out, T, H, c.top_k, pp.pair_stride, local_offset, El, so));
    else
        CU_TRY(launch_k(PDL_COMBINE, combine_kernel<OUT_F32>, cgrid, dim3(256), 0, st, (const __half*)y, topk_idx,
                        (const int32_t*)pair_row, (const float*)row_w, out, T, H, c.top_k, pp.pair_stride, local_offset, El, so));
    CU_TRY(prof_mark(h, 6, st));
    if (h->prof_slots) ++h->prof_calls;
    return 0;
}

// ---- scratch of b200moe_permute_noalloc: lives in the library image of every device that
// loads it.  Head: status int[8] at 0, counts int[256] at 256, tile_prefix int[257] at 1536; the
// slice histograms int[64][256] at 4096; then pair_row int[B200MOE_NOALLOC_MAX_TOKENS * 8].
constexpr size_t NOALLOC_HEAD_BYTES = 4096;
constexpr size_t NOALLOC_SLICE_BYTES = (size_t)(B200MOE_NOALLOC_MAX_TOKENS * 8 / SLICE_PAIRS) * MAX_LOCAL * 4;
constexpr size_t NOALLOC_SCRATCH_BYTES = NOALLOC_HEAD_BYTES + NOALLOC_SLICE_BYTES + (size_t)B200MOE_NOALLOC_MAX_TOKENS * 8 * 4;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
constexpr int NOALLOC_MAX_DEVICES = 64;
unsigned char* g_noalloc_dev_ptr[NOALLOC_MAX_DEVICES];   // device address of the array, per device (host copy)
std::mutex g_noalloc_mutex;

int check_ws(b200moe_ctx* h, int T, void* ws, size_t ws_bytes, b200moe_ws_layout* L) {
    layout(h, T, L);
    if (!ws || ws_bytes < L->total_bytes || (reinterpret_cast<uintptr_t>(ws) & 255)) return B200MOE_E_WORKSPACE;
    return 0;
}

}  // namespace

extern "C" {

int b200moe_num_sms(void) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return n;
}

int b200moe_create(const b200moe_config* cfg, b200moe_handle* out) {
    if (!cfg || !out) return B200MOE_E_BADARG;
    if (!cfg_ok(*cfg)) return B200MOE_E_BADARG;
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    int major = 0, sms = 0;
    CU_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    CU_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (major != 10) return B200MOE_E_DEVICE;
    if (!get_encode()) return B200MOE_E_DRIVER;
#define CU_TRY_ATTR(expr) do { cudaError_t e_ = (expr); if ((int)e_ == -B200MOE_E_BUILD + 100000) return B200MOE_E_BUILD; \
                               if (e_ != cudaSuccess) return (int)e_; } while (0)
    CU_TRY_ATTR((set_attr<16, true>()));  CU_TRY_ATTR((set_attr<16, false>()));
    CU_TRY_ATTR((set_attr<32, true>()));  CU_TRY_ATTR((set_attr<32, false>()));
    CU_TRY_ATTR((set_attr<64, true>()));  CU_TRY_ATTR((set_attr<64, false>()));
    CU_TRY_ATTR((set_attr<128, true>())); CU_TRY_ATTR((set_attr<128, false>())); CU_TRY_ATTR((set_attr<128, true, true>()));
#undef CU_TRY_ATTR
    b200moe_ctx* h = new (std::nothrow) b200moe_ctx;
    if (!h) return B200MOE_E_BADARG;
    h->cfg = *cfg; h->device = dev; h->num_sms = sms;
    h->prof_slots = 0; h->prof_calls = 0; h->prof_events = nullptr;
    h->wait_limit_ns = WAIT_LIMIT_NS;
    { const char* e = getenv("B200MOE_FUSE_COMBINE"); h->fuse_combine = e ? atoi(e) != 0 : 0; }
    h->token_tile = 0;
    { const char* e = getenv("B200MOE_GATHER4"); h->tma_gather = e ? atoi(e) != 0 : 0; }
    h->d_sync = nullptr;
    if (cudaMalloc(&h->d_sync, 64) != cudaSuccess || cudaMemset(h->d_sync, 0, 64) != cudaSuccess) {
        const cudaError_t e = cudaGetLastError();
        if (h->d_sync) cudaFree(h->d_sync);
        delete h;
        return e != cudaSuccess ? (int)e : (int)cudaErrorMemoryAllocation;
    }
    int rc_p;
    if ((rc_p = set_attr_pair<true>(sms, &h->pair_grid[0])) || (rc_p = set_attr_pair<false>(sms, &h->pair_grid[1]))) {
        cudaFree(h->d_sync);
        delete h;
        return rc_p;
    }
#ifdef B200MOE_ENABLE_ABLATE
    const char* ab = getenv("B200MOE_ABLATE");
    h->ablate = ab ? atoi(ab) : 0;
#else
    h->ablate = 0;      // the timing switches exist only in builds made for timing experiments
#endif
    *out = h;
    return 0;
}

int b200moe_destroy(b200moe_handle h) {
    if (!h) return B200MOE_E_BADARG;
    b200moe_profile_enable(h, 0);
    cudaFree(h->d_sync);
    delete h;
    return 0;
}

int b200moe_set_token_tile(b200moe_handle h, int tokens) {
    if (!h || (tokens != 0 && tokens != 16 && tokens != 32 && tokens != 64 && tokens != 128)) return B200MOE_E_BADARG;
    h->token_tile = tokens;
    return 0;
}

int b200moe_set_tma_gather(b200moe_handle h, int on) {
    if (!h) return B200MOE_E_BADARG;
    h->tma_gather = on != 0;
    return 0;
}

int b200moe_set_fused_combine(b200moe_handle h, int on) {
    if (!h) return B200MOE_E_BADARG;
    h->fuse_combine = on != 0;
    return 0;
}

int b200moe_set_wait_limit_ns(b200moe_handle h, unsigned long long ns) {
    if (!h || ns == 0 || ns > 60ull * 1000000000ull) return B200MOE_E_BADARG;
    h->wait_limit_ns = ns;
    return 0;
}

int b200moe_profile_enable(b200moe_handle h, int slots) {
    if (!h || slots < 0) return B200MOE_E_BADARG;
    if (h->prof_events) {
        for (int i = 0; i < h->prof_slots * PROF_POINTS; ++i) cudaEventDestroy(h->prof_events[i]);
        delete[] h->prof_events;
        h->prof_events = nullptr;
    }
    h->prof_slots = 0; h->prof_calls = 0;
    if (slots == 0) return 0;
    h->prof_events = new (std::nothrow) cudaEvent_t[(size_t)slots * PROF_POINTS];
    if (!h->prof_events) return B200MOE_E_BADARG;
    for (int i = 0; i < slots * PROF_POINTS; ++i) CU_TRY(cudaEventCreate(&h->prof_events[i]));
    h->prof_slots = slots;
    return 0;
}

int b200moe_profile_read(b200moe_handle h, int slot, float* stage_ms) {
    if (!h || !stage_ms || !h->prof_slots || slot < 0 || slot >= h->prof_slots || slot >= h->prof_calls)
        return B200MOE_E_BADARG;
    cudaEvent_t* ev = h->prof_events + (size_t)slot * PROF_POINTS;
    CU_TRY(cudaEventSynchronize(ev[PROF_POINTS - 1]));
    for (int i = 0; i + 1 < PROF_POINTS; ++i) CU_TRY(cudaEventElapsedTime(stage_ms + i, ev[i], ev[i + 1]));
    return 0;
}

int b200moe_workspace_layout(b200moe_handle h, int num_tokens, b200moe_ws_layout* L) {
    if (!h || !L || num_tokens < 0) return B200MOE_E_BADARG;
    layout(h, num_tokens, L);
    return 0;
}

int b200moe_workspace_bytes(b200moe_handle h, int num_tokens, size_t* bytes) {
    if (!h || !bytes || num_tokens < 0) return B200MOE_E_BADARG;
    b200moe_ws_layout L;
    layout(h, num_tokens, &L);
    *bytes = L.total_bytes;
    return 0;
}

int b200moe_launches_per_forward(b200moe_handle h, int num_tokens, int* launches) {
    if (!h || !launches || num_tokens < 0) return B200MOE_E_BADARG;
    // [route, permute, gather | fused route+permute+gather for small T], gemm1, gemm2, [combine unless fused into gemm2]
    const bool fuse = h->fuse_combine && pick_token_tile(h, num_tokens) < 128 && !use_pairs(h, pick_token_tile(h, num_tokens));
    const bool g4 = pick_token_tile(h, num_tokens) == 128 && !use_pairs(h, 128) && h->tma_gather;
    *launches = num_tokens == 0 ? 0 : (num_tokens <= FRONT_MAX_T ? 4 : 6) - (fuse ? 1 : 0) - (g4 ? 1 : 0);
    return 0;
}

int b200moe_launches_routed(b200moe_handle h, int num_tokens, int* launches) {
    if (!h || !launches || num_tokens < 0) return B200MOE_E_BADARG;
    // count, [permute + gather | both in one launch for small T; no gather when GEMM1 gathers by TMA], gemm1, gemm2, combine
    const bool g4 = pick_token_tile(h, num_tokens) == 128 && !use_pairs(h, 128) && h->tma_gather;
    *launches = num_tokens == 0 ? 0 : (num_tokens <= FRONT_MAX_T ? 5 : 6) - (g4 ? 1 : 0);
    return 0;
}

int b200moe_route(b200moe_handle h, const void* logits, const void* bias, int T, float scale, int32_t* topk_idx,
                  float* topk_w, void* stream) {
    if (!h || T < 0) return B200MOE_E_BADARG;
    if (T == 0) return 0;
    if (!logits || !topk_idx || !topk_w) return B200MOE_E_BADARG;
    const b200moe_config& c = h->cfg;
    RouteParams rp;
    rp.logits = static_cast<const float*>(logits); rp.bias = static_cast<const __nv_bfloat16*>(bias);
    rp.T = T; rp.E = c.num_experts; rp.top_k = c.top_k; rp.n_group = c.n_group; rp.topk_group = c.topk_group;
    rp.local_offset = 0; rp.num_local = 0; rp.scale = scale; rp.topk_idx = topk_idx; rp.topk_w = topk_w;
    rp.slices = nullptr;
    g_call_pdl = 0;                       // a stand-alone launch: nothing before it to overlap with
    CU_TRY(do_route(c, rp, static_cast<cudaStream_t>(stream)));
    return 0;
}

int b200moe_forward(b200moe_handle h, const void* logits, const void* bias, const void* hidden,
                    const void* hidden_scale, const void* w13, const void* s13, const void* w2, const void* s2, int T,
                    int local_offset, float scale, void* output, void* workspace, size_t workspace_bytes,
                    void* stream) {
    if (!h || T < 0) return B200MOE_E_BADARG;
    if (T == 0) return 0;
    if (!logits || !hidden || !hidden_scale || !w13 || !s13 || !w2 || !s2 || !output) return B200MOE_E_BADARG;
    b200moe_ws_layout L;
    int rc = check_ws(h, T, workspace, workspace_bytes, &L);
    if (rc) return rc;
    const b200moe_config& c = h->cfg;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    set_call_pdl(T);
    const bool fused = T <= FRONT_MAX_T;
    // status, K-split counters and slice histograms are contiguous at the head of the workspace: one memset - or none
    // for small token counts, where the fused front end clears the head itself and can then overlap the kernel the
    // caller ran before this call
    if (!fused) CU_TRY(cudaMemsetAsync(ws, 0, L.expert_row0, st));
    CU_TRY(prof_mark(h, 0, st));
    RouteParams rp;
    rp.logits = static_cast<const float*>(logits); rp.bias = static_cast<const __nv_bfloat16*>(bias);
    rp.T = T; rp.E = c.num_experts; rp.top_k = c.top_k; rp.n_group = c.n_group; rp.topk_group = c.topk_group;
    rp.local_offset = local_offset; rp.num_local = c.num_local_experts; rp.scale = scale;
    rp.topk_idx = reinterpret_cast<int32_t*>(ws + L.topk_idx); rp.topk_w = reinterpret_cast<float*>(ws + L.topk_w);
    rp.slices = reinterpret_cast<int*>(ws + L.slices);
    if (fused) rp.slices = nullptr;       // the fused front end routes and builds the histogram itself (one launch)
    else CU_TRY(do_route(c, rp, st));
    CU_TRY(prof_mark(h, 1, st));
    return run_experts(h, rp.topk_idx, rp.topk_w, hidden, hidden_scale, w13, s13, w2, s2, T, local_offset, output,
                       OUT_BF16, ws, L, st, fused, nullptr, 0, fused ? &rp : nullptr, true);
}

int b200moe_forward_routed(b200moe_handle h, const int32_t* topk_idx, const float* topk_w, const void* hidden,
                           const void* hidden_scale, const void* w13, const void* s13, const void* w2, const void* s2,
                           int T, int local_offset, void* output, int output_kind, void* workspace,
                           size_t workspace_bytes, void* stream) {
    if (!h || T < 0 || output_kind < 0 || output_kind > 2) return B200MOE_E_BADARG;
    if (T == 0) return 0;
    if (!topk_idx || !topk_w || !hidden || !hidden_scale || !w13 || !s13 || !w2 || !s2 || !output)
        return B200MOE_E_BADARG;
    b200moe_ws_layout L;
    int rc = check_ws(h, T, workspace, workspace_bytes, &L);
    if (rc) return rc;
    const b200moe_config& c = h->cfg;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    set_call_pdl(T);
    CU_TRY(cudaMemsetAsync(ws, 0, L.expert_row0, st));
    CU_TRY(prof_mark(h, 0, st));
    const int n = T * c.top_k;
    int grid = (n + 255) / 256;
    if (grid > h->num_sms * 4) grid = h->num_sms * 4;
    count_kernel<<<grid, 256, 0, st>>>(topk_idx, n, c.top_k, c.top_k, local_offset, c.num_local_experts,
                                       reinterpret_cast<int*>(ws + L.slices));
    CU_TRY(cudaGetLastError());
    CU_TRY(prof_mark(h, 1, st));
    return run_experts(h, topk_idx, topk_w, hidden, hidden_scale, w13, s13, w2, s2, T, local_offset, output,
                       output_kind, ws, L, st);
}

int b200moe_ep_row_bytes(b200moe_handle h, int* bytes) {
    if (!h || !bytes) return B200MOE_E_BADARG;
    *bytes = ep_row_bytes(h->cfg.hidden, h->cfg.top_k);
    return 0;
}

int b200moe_ep_pack(b200moe_handle h, const void* hidden, const void* hidden_scale, const int32_t* topk_idx,
                    const float* topk_w, const long long* send_token, int n_rows, int T, void* wire, void* stream) {
    if (!h || n_rows < 0 || T < 0 || h->cfg.top_k > 32) return B200MOE_E_BADARG;
    if (n_rows == 0) return 0;
    if (!hidden || !hidden_scale || !topk_idx || !topk_w || !send_token || !wire) return B200MOE_E_BADARG;
    int grid = (n_rows + 7) / 8;
    if (grid > h->num_sms * 8) grid = h->num_sms * 8;
    ep_pack_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(hidden), static_cast<const float*>(hidden_scale), topk_idx, topk_w, send_token,
        n_rows, T, h->cfg.hidden, h->cfg.top_k, static_cast<uint8_t*>(wire));
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_ep_unpack(b200moe_handle h, const void* wire, int n_rows, void* hidden, void* hidden_scale,
                      int32_t* topk_idx, float* topk_w, void* stream) {
    if (!h || n_rows < 0 || h->cfg.top_k > 32) return B200MOE_E_BADARG;
    if (n_rows == 0) return 0;
    if (!wire || !hidden || !hidden_scale || !topk_idx || !topk_w) return B200MOE_E_BADARG;
    int grid = (n_rows + 7) / 8;
    if (grid > h->num_sms * 8) grid = h->num_sms * 8;
    ep_unpack_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(wire), n_rows, h->cfg.hidden, h->cfg.top_k, static_cast<uint8_t*>(hidden),
        static_cast<float*>(hidden_scale), topk_idx, topk_w);
    CU_TRY(cudaGetLastError());
    return 0;
}

// ---- exchange over peer memory (ep_p2p.cuh)
static bool fill_peers(PeerPtrs& pp, void* const* peers, int world) {
    if (!peers || world < 1 || world > EP_P2P_MAX_WORLD) return false;
    for (int r = 0; r < EP_P2P_MAX_WORLD; ++r) pp.p[r] = r < world ? peers[r] : nullptr;
    for (int r = 0; r < world; ++r) if (!pp.p[r]) return false;
    return true;
}
static int row_grid(b200moe_ctx* h, long long rows) {
    long long g = (rows + 7) / 8;
    if (g > (long long)h->num_sms * 8) g = (long long)h->num_sms * 8;
    return g < 1 ? 1 : (int)g;
}

int b200moe_ep_push(b200moe_handle h, const void* hidden, const void* hidden_scale, const int32_t* topk_idx,
                    const float* topk_w, int T, int cap, int world, int my_rank, void* const* peer_wire, void* stream) {
    PeerPtrs pp;
    if (!h || T < 0 || cap < 1 || T > cap || my_rank < 0 || my_rank >= world || h->cfg.top_k > 32 ||
        !fill_peers(pp, peer_wire, world) || h->cfg.num_local_experts * world != h->cfg.num_experts)
        return B200MOE_E_BADARG;
    if (T > 0 && (!hidden || !hidden_scale || !topk_idx || !topk_w)) return B200MOE_E_BADARG;
    ep_push_kernel<<<row_grid(h, cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(hidden), static_cast<const float*>(hidden_scale), topk_idx, topk_w, T, cap,
        h->cfg.hidden, h->cfg.top_k, h->cfg.num_local_experts, world, my_rank, pp);
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_ep_barrier(b200moe_handle h, void* const* peer_flags, int world, int my_rank, unsigned epoch,
                       int* status_word, void* stream) {
    PeerPtrs pp;
    if (!h || my_rank < 0 || my_rank >= world || !status_word || !fill_peers(pp, peer_flags, world))
        return B200MOE_E_BADARG;
    ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pp, world, my_rank, epoch, status_word,
                                                                       h->wait_limit_ns);
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_ep_unpack_slots(b200moe_handle h, const void* wire, int n_slots, void* hidden, void* hidden_scale,
                            int32_t* topk_idx, float* topk_w, void* stream) {
    if (!h || n_slots < 0 || h->cfg.top_k > 32) return B200MOE_E_BADARG;
    if (n_slots == 0) return 0;
    if (!wire || !hidden || !hidden_scale || !topk_idx || !topk_w) return B200MOE_E_BADARG;
    ep_unpack_slots_kernel<<<row_grid(h, n_slots), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(wire), n_slots, h->cfg.hidden, h->cfg.top_k, static_cast<uint8_t*>(hidden),
        static_cast<float*>(hidden_scale), topk_idx, topk_w);
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_ep_return(b200moe_handle h, const void* partial_rows, const int32_t* topk_idx_slots, int cap, int world,
                      int my_rank, void* const* peer_back, void* stream) {
    PeerPtrs pp;
    if (!h || cap < 1 || my_rank < 0 || my_rank >= world || !partial_rows || !topk_idx_slots ||
        !fill_peers(pp, peer_back, world) || h->cfg.hidden % 8)
        return B200MOE_E_BADARG;
    ep_return_kernel<<<row_grid(h, (long long)world * cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(partial_rows), topk_idx_slots, cap, h->cfg.hidden, h->cfg.top_k, world,
        my_rank, pp);
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_forward_routed_slots(b200moe_handle h, const void* wire, const void* w13, const void* s13, const void* w2,
                                 const void* s2, int cap, int world, int my_rank, int local_offset,
                                 void* const* peer_back, void* workspace, size_t workspace_bytes, void* stream) {
    SlotOut so;
    if (!h || cap < 1 || my_rank < 0 || my_rank >= world || !fill_peers(so.back, peer_back, world) ||
        (long long)cap * world > 0x7FFFFFFF || h->cfg.top_k > 32)
        return B200MOE_E_BADARG;
    if (!wire || !w13 || !s13 || !w2 || !s2 || (reinterpret_cast<uintptr_t>(wire) & 15)) return B200MOE_E_BADARG;
    so.cap = cap; so.my_rank = my_rank;
    const int T = cap * world;
    b200moe_ws_layout L;
    int rc = check_ws(h, T, workspace, workspace_bytes, &L);
    if (rc) return rc;
    const b200moe_config& c = h->cfg;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    // the slots are read where the peers stored them: fp8 row | scales | ids | weights, one row per slot
    const int pitch = ep_row_bytes(c.hidden, c.top_k);
    const uint8_t* rows = static_cast<const uint8_t*>(wire);
    const int32_t* ids = reinterpret_cast<const int32_t*>(rows + c.hidden + 4 * (c.hidden >> 7));
    const float* wts = reinterpret_cast<const float*>(rows + c.hidden + 4 * (c.hidden >> 7) + 4 * c.top_k);
    set_call_pdl(T);
    CU_TRY(cudaMemsetAsync(ws, 0, L.expert_row0, st));
    CU_TRY(prof_mark(h, 0, st));
    const int n = T * c.top_k;
    int grid = (n + 255) / 256;
    if (grid > h->num_sms * 4) grid = h->num_sms * 4;
    count_kernel<<<grid, 256, 0, st>>>(ids, n, c.top_k, pitch / 4, local_offset, c.num_local_experts,
                                       reinterpret_cast<int*>(ws + L.slices));
    CU_TRY(cudaGetLastError());
    CU_TRY(prof_mark(h, 1, st));
    // the rows leave through the peer slots; `out` is never dereferenced in that mode
    return run_experts(h, ids, wts, rows, nullptr, w13, s13, w2, s2, T, local_offset, ws, OUT_F16, ws, L, st,
                       false, &so, pitch);
}

int b200moe_ep_combine_slots(b200moe_handle h, const void* back, const int32_t* topk_idx, int T, int cap, int world,
                             void* output_bf16, void* stream) {
    if (!h || T < 0 || cap < 1 || T > cap || world < 1 || world > EP_P2P_MAX_WORLD || h->cfg.hidden % 8 ||
        h->cfg.num_local_experts * world != h->cfg.num_experts)
        return B200MOE_E_BADARG;
    if (T == 0) return 0;
    if (!back || !topk_idx || !output_bf16) return B200MOE_E_BADARG;
    const int grid = T < h->num_sms * 8 ? T : h->num_sms * 8;
    ep_combine_slots_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(back), topk_idx, T, cap, h->cfg.hidden, h->cfg.top_k,
        h->cfg.num_local_experts, world, static_cast<__nv_bfloat16*>(output_bf16));
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_ep_combine(b200moe_handle h, const void* partial_rows, const int32_t* row_of, int world, int T,
                       void* output_bf16, void* stream) {
    if (!h || T < 0 || world < 1 || world > EP_MAX_WORLD) return B200MOE_E_BADARG;
    if (T == 0) return 0;
    if (!partial_rows || !row_of || !output_bf16) return B200MOE_E_BADARG;
    const int H = h->cfg.hidden;
    if (H % 8) return B200MOE_E_BADARG;
    int grid = T < h->num_sms * 8 ? T : h->num_sms * 8;
    ep_combine_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(partial_rows), row_of, world, T, H, static_cast<__nv_bfloat16*>(output_bf16));
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_permute_noalloc(b200moe_handle h, const int32_t* topk_idx, const float* topk_w, int T, int local_offset,
                            int32_t* expert_row0, int32_t* row_token, float* row_w, int rows_capacity, void* stream) {
    if (!h || T < 0) return B200MOE_E_BADARG;
    if (T > B200MOE_NOALLOC_MAX_TOKENS) return B200MOE_E_TOO_LARGE;
    if (!topk_idx || !topk_w || !expert_row0 || !row_token || !row_w) return B200MOE_E_BADARG;
    const b200moe_config& c = h->cfg;
    if (rows_capacity < rows_capacity_for(c, T)) return B200MOE_E_WORKSPACE;
    int dev = -1;
    CU_TRY(cudaGetDevice(&dev));
    if (dev != h->device || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return B200MOE_E_BADARG;
    unsigned char* scratch = nullptr;
    {
        // Once per device, with that device current: the array's name is only a host-side stand-in,
        // the kernels need its device address.
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_dev_ptr[dev]) {
            void* p = nullptr;
            CU_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
            if (!p) return B200MOE_E_DRIVER;
            g_noalloc_dev_ptr[dev] = static_cast<unsigned char*>(p);
        }
        scratch = g_noalloc_dev_ptr[dev];
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int El = c.num_local_experts;
    // the histogram and the status words must start at zero; the array keeps the last call's contents
    const int ns = num_slices(c, T);
    if (c.top_k > 8 || (size_t)ns * El * 4 > NOALLOC_SLICE_BYTES) return B200MOE_E_TOO_LARGE;
    CU_TRY(cudaMemsetAsync(scratch, 0, NOALLOC_HEAD_BYTES + (size_t)ns * El * 4, st));
    if (T > 0) {
        const int n = T * c.top_k;
        int grid = (n + 255) / 256;
        if (grid > h->num_sms * 4) grid = h->num_sms * 4;
        count_kernel<<<grid, 256, 0, st>>>(topk_idx, n, c.top_k, c.top_k, local_offset, El,
                                           reinterpret_cast<int*>(scratch + NOALLOC_HEAD_BYTES));
        CU_TRY(cudaGetLastError());
    }
    PlanParams pp;
    pp.T = T; pp.top_k = c.top_k; pp.num_local = El; pp.local_offset = local_offset;
    pp.token_tile = pick_token_tile(h, T);
    pp.topk_idx = topk_idx; pp.topk_w = topk_w; pp.pair_stride = c.top_k;
    pp.status = reinterpret_cast<int*>(scratch);
    pp.counts = reinterpret_cast<int*>(scratch + 256);
    pp.tile_prefix = reinterpret_cast<int*>(scratch + 1536);
    pp.slices = reinterpret_cast<const int*>(scratch + NOALLOC_HEAD_BYTES);
    pp.pair_row = reinterpret_cast<int32_t*>(scratch + NOALLOC_HEAD_BYTES + NOALLOC_SLICE_BYTES);
    pp.expert_row0 = expert_row0; pp.row_token = row_token; pp.row_w = row_w; pp.rows_cap = rows_capacity;
    permute_kernel<<<ns, PERMUTE_THREADS, 0, st>>>(pp);
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_quantize_1x128(const void* x_bf16, int T, int H, void* q_e4m3, float* scale, void* stream) {
    if (T < 0 || H <= 0 || H % 128) return B200MOE_E_BADARG;
    if (T == 0) return 0;
    if (!x_bf16 || !q_e4m3 || !scale) return B200MOE_E_BADARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(q_e4m3) & 7)) return B200MOE_E_BADARG;
    const int sms = b200moe_num_sms();
    const long long groups = (long long)T * (H >> 7);
    long long grid = (groups + 15) / 16;                   // 16 groups (half warps) per CTA
    if (grid > (long long)sms * 16) grid = (long long)sms * 16;
    quantize_1x128_kernel<<<(int)(grid < 1 ? 1 : grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), T, H, static_cast<uint8_t*>(q_e4m3), scale);
    CU_TRY(cudaGetLastError());
    return 0;
}

int b200moe_status(b200moe_handle h, const void* workspace, void* stream, int* word) {
    if (!h || !workspace || !word) return B200MOE_E_BADARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CU_TRY(cudaMemcpyAsync(word, workspace, sizeof(int), cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    if (*word) CU_TRY(cudaMemset(h->d_sync, 0, 64));      // a front end that gave up at its meeting leaves the words dirty
    return *word ? B200MOE_E_KERNEL : 0;
}

const char* b200moe_strerror(int code) {
    switch (code) {
        case 0: return "ok";
        case B200MOE_E_BADARG: return "bad argument or unsupported shape";
        case B200MOE_E_WORKSPACE: return "workspace too small or not 256-byte aligned";
        case B200MOE_E_DRIVER: return "cuTensorMapEncodeTiled unavailable or failed";
        case B200MOE_E_DEVICE: return "device is not compute capability 10.x";
        case B200MOE_E_KERNEL: return "a kernel gave up a bounded wait or met a bad schedule (see status word)";
        case B200MOE_E_BUILD: return "a GEMM kernel was compiled with a register count other than the one its setmaxnreg "
                                     "arithmetic assumes (different compiler version or flags): rebuild with the stated nvcc";
        case B200MOE_E_TOO_LARGE: return "num_tokens exceeds B200MOE_NOALLOC_MAX_TOKENS (the static scratch array is fixed-size)";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
    }
}

}  // extern "C"
