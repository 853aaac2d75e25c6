// Mixture-of-experts routing: a sigmoid or softmax router with a choice-only correction (optionally limited to the best
// groups of neighbouring experts, optionally with identity experts that own no list), the expert-sorted row lists that the
// grouped linear kernels walk, and the weighted combine. Router scores, weights and gates are fp32.
#include <math.h>

#include "common.cuh"
#include "launch.h"
#include "seqmix.h"

namespace lcc {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// One warp per row. Lane l holds experts l, l + 32, ...; `top` rounds of a warp-wide arg-max (the lower index wins a tie)
// pick the experts in descending order of choice score. The arrival number inside an expert comes from an atomic
// counter: it decides only where the row sits in the expert's list, never a value.
constexpr int kMaxExpertsPerLane = 16;   // experts <= 512
// The choice for one row by one warp; lane 0 returns the k-th expert and its score through `emit`.
// ro.softmax: score = softmax over the E outputs (else a sigmoid each). ro.groups > 0: the outputs form equal groups of
// neighbours; a group scores as its largest choice score, the ro.keep best groups stay (ties: the lower index) and every
// other output's choice score counts as -inf. gch / gkeep: this warp's scratch in shared memory ([E] floats, [groups] flags).
template <typename Emit>
__device__ __forceinline__ void route_row(const float* __restrict__ z, const float* __restrict__ correction, int E, int top,
                                          const MoeRouterOpts& ro, float* gch, unsigned char* gkeep, Emit emit) {
    const int lane = threadIdx.x & 31;
    float sc[kMaxExpertsPerLane], ch[kMaxExpertsPerLane];
    float zmax = -INFINITY, zsum = 0.f;
    if (ro.softmax) {
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) {
            const int e = lane + 32 * i;
            sc[i] = e < E ? z[e] : -INFINITY;
            zmax = fmaxf(zmax, sc[i]);
        }
        zmax = warp_max(zmax);
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) {
            sc[i] = expf(sc[i] - zmax);       // exp(-inf) = 0 past the last output
            zsum += sc[i];
        }
        zsum = 1.f / warp_sum(zsum);
    }
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        sc[i] = e < E ? (ro.topk_softmax ? z[e] : (ro.softmax ? sc[i] * zsum : sigmoid_f(z[e]))) : 0.f;
        ch[i] = e < E ? sc[i] + (correction ? correction[e] : 0.f) : -INFINITY;
    }
    if (ro.groups > 0) {
        const int per = E / ro.groups;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i)
            if (lane + 32 * i < E) gch[lane + 32 * i] = ch[i];
        for (int g = lane; g < ro.groups; g += 32) gkeep[g] = 0;
        __syncwarp();
        for (int k = 0; k < ro.keep; ++k) {
            float best = -INFINITY;
            int bg = 0x7fffffff;
            for (int g = lane; g < ro.groups; g += 32) {
                if (gkeep[g]) continue;
                float m = -INFINITY;
                for (int j = 0; j < per; ++j) m = fmaxf(m, gch[g * per + j]);
                if (m > best || bg == 0x7fffffff) { best = m; bg = g; }   // ascending g: the first of equals stays
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, bg, o);
                if (og != 0x7fffffff && (bg == 0x7fffffff || ob > best || (ob == best && og < bg))) { best = ob; bg = og; }
            }
            if (lane == 0) gkeep[bg] = 1;
            __syncwarp();
        }
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) {
            const int e = lane + 32 * i;
            if (e < E && !gkeep[e / per]) ch[i] = -INFINITY;
        }
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY, bs = 0.f;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) {
            const int e = lane + 32 * i;
            if (e < E && ch[i] > best) { best = ch[i]; be = e; bs = sc[i]; }   // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; bs = os; }
        }
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i)
            if (lane + 32 * i == be) ch[i] = -INFINITY;
        if (lane == 0) emit(k, be, bs);
    }
}

// ro.topk_softmax: route_row emitted the chosen logits in descending order of choice; one lane turns a row's `top` logits into the
// softmax over them (times scale) in place.
__device__ __forceinline__ void softmax_chosen(float* w, int top, float scale) {
    float m = -INFINITY, sum = 0.f;
    for (int k = 0; k < top; ++k) m = fmaxf(m, w[k]);
    for (int k = 0; k < top; ++k) { w[k] = expf(w[k] - m); sum += w[k]; }
    const float inv = scale / sum;
    for (int k = 0; k < top; ++k) w[k] *= inv;
}

constexpr int kRouteScratch = 32 * kMaxExpertsPerLane;   // per warp: choice scores of a row, flags of the kept groups

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction,
                                                        int E, int top, float scale, int* __restrict__ sel,
                                                        float* __restrict__ weight, float* __restrict__ shared_gate,
                                                        int* __restrict__ counts, int* __restrict__ rank, int S, MoeRouterOpts ro) {
    __shared__ float gch[4][kRouteScratch];
    __shared__ unsigned char gkeep[4][kRouteScratch];
    const int warp = threadIdx.x >> 5;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp, lane = threadIdx.x & 31;
    if (r >= S) return;
    const float* z = logits + (size_t)r * ld;
    const int real = E - ro.identity;
    float idw = 0.f;         // lane 0: the weights of the chosen identity experts
    route_row(z, correction, E, top, ro, gch[warp], gkeep[warp], [&](int k, int be, float bs) {
        sel[(size_t)r * top + k] = be;
        weight[(size_t)r * top + k] = ro.topk_softmax ? bs : bs * scale;
        if (be < real) rank[(size_t)r * top + k] = atomicAdd(counts + be, 1);
        else { rank[(size_t)r * top + k] = -1; idw += bs * scale; }
    });
    if (ro.topk_softmax && lane == 0) softmax_chosen(weight + (size_t)r * top, top, scale);
    if (shared_gate && lane == 0) shared_gate[r] = ro.identity > 0 ? idw : sigmoid_f(z[E]);
}

// Few rows (a decode step): one CTA routes every row, counts the lists in shared memory and writes the dense row lists,
// which takes the counter reset, the choice and the list kernel of the general route into one launch.
constexpr int kSmallRouteItems = 1024, kSmallRouteExperts = 512;
__global__ void __launch_bounds__(256) moe_route_small_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction,
                                                              int E, int top, float scale, int* __restrict__ sel,
                                                              float* __restrict__ weight, float* __restrict__ shared_gate,
                                                              int* __restrict__ row_off, int* __restrict__ pos,
                                                              int* __restrict__ src_row, int S, MoeRouterOpts ro) {
    __shared__ int cnt[kSmallRouteExperts + 1];
    __shared__ int rk[kSmallRouteItems];
    __shared__ float gch[8][kRouteScratch];
    __shared__ unsigned char gkeep[8][kRouteScratch];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int real = E - ro.identity;          // lists exist for the real experts only
    for (int e = threadIdx.x; e <= real; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int r = warp; r < S; r += (blockDim.x >> 5)) {
        const float* z = logits + (size_t)r * ld;
        float idw = 0.f;
        route_row(z, correction, E, top, ro, gch[warp], gkeep[warp], [&](int k, int be, float bs) {
            sel[(size_t)r * top + k] = be;
            weight[(size_t)r * top + k] = ro.topk_softmax ? bs : bs * scale;
            if (be < real) rk[r * top + k] = atomicAdd(&cnt[be], 1);
            else { rk[r * top + k] = -1; idw += bs * scale; }
        });
        if (ro.topk_softmax && lane == 0) softmax_chosen(weight + (size_t)r * top, top, scale);
        if (shared_gate && lane == 0) shared_gate[r] = ro.identity > 0 ? idw : sigmoid_f(z[E]);
    }
    __syncthreads();
    if (threadIdx.x == 0) {         // exclusive prefix sum in place
        int o = 0;
        for (int e = 0; e <= real; ++e) { const int c = cnt[e]; cnt[e] = o; o += c; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= real; e += blockDim.x) row_off[e] = cnt[e];
    for (int i = threadIdx.x; i < S * top; i += blockDim.x) {
        if (rk[i] < 0) { pos[i] = -1; continue; }
        const int p = cnt[sel[i]] + rk[i];      // sel[i] was written by a thread of this CTA before the barriers
        pos[i] = p;
        src_row[p] = i / top;
    }
}

// Lists padded to whole tiles of `pad` rows (pad = 1: dense lists): list e starts at the sum of the padded counts before it.
__device__ __forceinline__ int padded(int n, int pad) { return (n + pad - 1) / pad * pad; }

__global__ void moe_index_kernel(const int* __restrict__ sel, const int* __restrict__ rank, const int* __restrict__ counts, int E,
                                 int top, int pad, int* __restrict__ row_off, int* __restrict__ pos, int* __restrict__ src_row,
                                 int* __restrict__ tile_group, int n_tiles, int S) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= E) {
        int o = 0;
        for (int e = 0; e < i; ++e) o += padded(counts[e], pad);
        row_off[i] = o;
    }
    if (tile_group && i < n_tiles) {
        // the list that owns rows [i * pad, (i + 1) * pad), or -1 past the last list
        int o = 0, g = -1;
        for (int e = 0; e < E; ++e) {
            const int n = padded(counts[e], pad);
            if (i * pad >= o && i * pad < o + n) { g = e; break; }
            o += n;
        }
        tile_group[i] = g;
    }
    if (i >= S * top) return;
    const int e = sel[i];
    if (rank[i] < 0) { pos[i] = -1; return; }     // an identity expert: no list
    int o = 0;
    for (int j = 0; j < e; ++j) o += padded(counts[j], pad);
    const int p = o + rank[i];
    pos[i] = p;
    src_row[p] = i / top;
}

// out[i, :] = in[src_row[i], :] for every list row (16-byte pieces); padding rows (src_row < 0) are left alone.
__global__ void __launch_bounds__(128) moe_gather_kernel(const uint4* __restrict__ in, int ld_in16, const int* __restrict__ src_row,
                                                         uint4* __restrict__ out, int ld_out16, int n16) {
    const int r = src_row[blockIdx.x];
    if (r < 0) return;
    for (int c = threadIdx.x; c < n16; c += blockDim.x) out[(size_t)blockIdx.x * ld_out16 + c] = in[(size_t)r * ld_in16 + c];
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ eo, int ld_eo, const int* __restrict__ pos, const float* __restrict__ weight,
                                   int top, const T* __restrict__ so, int ld_so, const float* __restrict__ shared_gate,
                                   T* __restrict__ out, int ld_out, int W) {
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = pos[(size_t)r * top + k];
            if (p >= 0) acc = fmaf(weight[(size_t)r * top + k], ldf(eo + (size_t)p * ld_eo + c), acc);
        }
        if (so) acc = fmaf(shared_gate[r], ldf(so + (size_t)r * ld_so + c), acc);
        stf(out + (size_t)r * ld_out + c, acc);
    }
}

}  // namespace

// a router's options are consistent with its sizes
static bool router_ok(const MoeRouterOpts& ro, int E, int top, const float* shared_gate) {
    if (ro.identity < 0 || ro.identity >= E || (ro.identity > 0 && !shared_gate)) return false;
    if (ro.groups > 0 && (E % ro.groups || ro.keep < 1 || ro.keep > ro.groups || ro.keep * (E / ro.groups) < top)) return false;
    if (ro.topk_softmax && (ro.identity > 0 || ro.groups > 0 || ro.softmax)) return false;
    return ro.groups >= 0;
}

int moe_route(const float* logits, int ld, const float* correction, int E, int top, float scale, int* sel, float* weight,
              float* shared_gate, int* counts, int* rank, int S, cudaStream_t s, const MoeRouterOpts* opt) {
    const MoeRouterOpts ro = opt ? *opt : MoeRouterOpts{false, 0, 0, 0};
    if (!logits || !sel || !weight || !counts || !rank || S < 1 || E < 1 || E > 32 * kMaxExpertsPerLane || top < 1 ||
        top > E || ld < E + ((shared_gate && !ro.identity) ? 1 : 0) || !router_ok(ro, E, top, shared_gate))
        return -2;
    count_launch();
    moe_route_kernel<<<(S + 3) / 4, 128, 0, s>>>(logits, ld, correction, E, top, scale, sel, weight, shared_gate, counts, rank, S, ro);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int moe_route_small(const float* logits, int ld, const float* correction, int E, int top, float scale, int* sel, float* weight,
                    float* shared_gate, int* row_off, int* pos, int* src_row, int S, cudaStream_t s, const MoeRouterOpts* opt) {
    const MoeRouterOpts ro = opt ? *opt : MoeRouterOpts{false, 0, 0, 0};
    if (!logits || !sel || !weight || !row_off || !pos || !src_row || S < 1 || E < 1 || E > kSmallRouteExperts ||
        top < 1 || top > E || S * top > kSmallRouteItems || ld < E + ((shared_gate && !ro.identity) ? 1 : 0) || !router_ok(ro, E, top, shared_gate))
        return -2;
    count_launch();
    moe_route_small_kernel<<<1, 256, 0, s>>>(logits, ld, correction, E, top, scale, sel, weight, shared_gate, row_off, pos, src_row, S, ro);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int moe_index(const int* sel, const int* rank, const int* counts, int E, int top, int pad, int* row_off, int* pos, int* src_row,
              int* tile_group, int n_tiles, int S, cudaStream_t s) {
    if (!sel || !rank || !counts || !row_off || !pos || !src_row || S < 1 || E < 1 || top < 1 || pad < 1 || (tile_group && n_tiles < 1))
        return -2;
    int n = S * top > E + 1 ? S * top : E + 1;
    if (tile_group && n_tiles > n) n = n_tiles;
    count_launch();
    moe_index_kernel<<<(n + 255) / 256, 256, 0, s>>>(sel, rank, counts, E, top, pad, row_off, pos, src_row, tile_group, n_tiles, S);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int moe_gather_rows(int dt, const void* in, int ld_in, const int* src_row, void* out, int ld_out, int rows, int W, cudaStream_t s) {
    const int per16 = dt == DT_F32 ? 4 : 8;
    if (!in || !src_row || !out || rows < 1 || W < 1 || (W % per16) || (ld_in % per16) || (ld_out % per16) ||
        ((uintptr_t)in % 16) || ((uintptr_t)out % 16))
        return -2;
    count_launch();
    moe_gather_kernel<<<rows, 128, 0, s>>>((const uint4*)in, ld_in / per16, src_row, (uint4*)out, ld_out / per16, W / per16);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int moe_combine(int dt, const void* eo, int ld_eo, const int* pos, const float* weight, int top, const void* so, int ld_so,
                const float* shared_gate, void* out, int ld_out, int S, int W, cudaStream_t s) {
    if (!eo || !pos || !weight || !out || S < 1 || W < 1 || top < 1 || (so && !shared_gate)) return -2;
    count_launch();
    if (dt == DT_F32)
        moe_combine_kernel<float><<<S, 256, 0, s>>>((const float*)eo, ld_eo, pos, weight, top, (const float*)so, ld_so, shared_gate,
                                                    (float*)out, ld_out, W);
    else
        moe_combine_kernel<bf16><<<S, 256, 0, s>>>((const bf16*)eo, ld_eo, pos, weight, top, (const bf16*)so, ld_so, shared_gate,
                                                   (bf16*)out, ld_out, W);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace lcc
