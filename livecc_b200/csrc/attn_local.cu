// Chunk-local attention over a paged K/V cache with arbitrary head sizes:
//   * q/k RMS norm over the whole projection (all heads at once) and the append of k, v to the pages,
//   * attention of new rows over the keys of their own chunk (chunks counted from position 0 of the sequence) with a
//     softmax sink: p_j = exp(s_j) / (exp(sink_h) + sum_j exp(s_j)) (sink_h = 0 unless given), and a per-head sigmoid output gate.
// Options (AttnOpts): a sliding window instead of / inside the chunks, no sink (ordinary softmax), one gate per output channel.
// Scores, weights and the accumulation are fp32; K and V pages hold the model's storage type.
#include <math.h>
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "launch.h"
#include "mma.cuh"
#include "seqmix.h"

namespace lcc {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ int seq_past(const SeqPos& p, int) { return p.kv_len ? *p.kv_len : p.past; }
__device__ __forceinline__ bool seq_done(const SeqPos& p) { return p.finished && *p.finished; }

// first key a row at position p sees: the start of its chunk, and / or p - window + 1
__device__ __forceinline__ int first_key(int p, int chunk, int window) {
    int lo = chunk > 0 ? (p / chunk) * chunk : 0;
    if (window > 0) lo = max(lo, p - window + 1);
    return lo;
}
// A softmax without a sink starts its running (max, sum) at (kNoSinkMax, 0): finite, so that a tile in which a row sees no
// key leaves both unchanged (exp(-inf - kNoSinkMax) = 0) and the first visible key rescales the empty sum by exp(-huge) = 0.
constexpr float kNoSinkMax = -1e30f;
// sigmoid gate of output element (row t, head h, channel c): one per head, or one per channel
template <typename T>
__device__ __forceinline__ float gate_of(const T* gate, int ld_gate, int t, int h, int c, int DV, bool per_channel) {
    const float z = ldf(gate + (size_t)t * ld_gate + (per_channel ? (size_t)h * DV + c : (size_t)h));
    return 1.f / (1.f + expf(-z));
}

// One CTA per (new row, slice of the heads): one warp per head in turn (query heads, then key heads; few-row steps spread a
// row's heads over several CTAs). Per head: sum of squares over D -> the
// normed channels -> rotation of the first rot_dims channels -> q_out, or the K page; the V page takes its columns of the
// row as they are.
template <typename T> __device__ __forceinline__ float2 ld2(const T* p);
template <> __device__ __forceinline__ float2 ld2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 ld2<bf16>(const bf16* p) { return unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p)); }
template <typename T> __device__ __forceinline__ void st2(T* p, float a, float b);
template <> __device__ __forceinline__ void st2<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <> __device__ __forceinline__ void st2<bf16>(bf16* p, float a, float b) { *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(a, b); }

// PAIRS: the pair-interleaved layout with an even head size and aligned rows: a lane owns neighbouring channels (2j, 2j+1), which
// are one load, one angle, one sincosf and one store; a head of up to 256 channels stays in registers between the two passes.
template <typename T, bool PAIRS>
__global__ void __launch_bounds__(256) qk_headnorm_rope_append_kernel(const T* __restrict__ proj, int ld, int v_col,
                                                                      const float* __restrict__ qn_w, const float* __restrict__ kn_w,
                                                                      float eps, const float* __restrict__ inv_freq, float mag,
                                                                      int rot_dims, int rot_pairs, float* __restrict__ q_out,
                                                                      T* __restrict__ k_pages, T* __restrict__ v_pages,
                                                                      const int* __restrict__ page_table, int page_size, int S, int Hq,
                                                                      int G, int D, int DV, SeqPos pos, AppendOpts ao) {
    if (seq_done(pos)) return;
    const int t = blockIdx.x;
    const int p = seq_past(pos, S) + t;
    const float pf = (float)p;
    const T* row = proj + (size_t)t * ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int page = page_table[p / page_size], slot = p % page_size;
    const int half = rot_dims >> 1;
    for (int hd = blockIdx.y * nwarps + warp; hd < Hq + G; hd += gridDim.y * nwarps) {
        const bool is_q = hd < Hq;
        const T* x = row + (size_t)hd * D;                 // k heads follow the q heads in the row
        const float* w = is_q ? qn_w : kn_w;
        float ss = 0.f;
        if (PAIRS) {
            constexpr int kKeep = 4;                       // pairs a lane keeps: heads of up to 256 channels
            const int np = D >> 1;
            float2 keep[kKeep];
#pragma unroll
            for (int u = 0; u < kKeep; ++u) {
                const int j = lane + 32 * u;
                keep[u] = j < np ? ld2(x + 2 * j) : make_float2(0.f, 0.f);
                ss = fmaf(keep[u].x, keep[u].x, fmaf(keep[u].y, keep[u].y, ss));
            }
            for (int j = lane + 32 * kKeep; j < np; j += 32) { const float2 v = ld2(x + 2 * j); ss = fmaf(v.x, v.x, fmaf(v.y, v.y, ss)); }
            ss = warp_sum(ss);
            const float rn = ((w || ao.unit_norm) ? 1.f / sqrtf(ss / (float)D + eps) : 1.f) * ((is_q && ao.q_head_scale) ? ao.q_head_scale[hd] : 1.f);
            float* qo = q_out + ((size_t)t * Hq + hd) * D;
            T* ko = k_pages + (((size_t)page * G + (hd - Hq)) * page_size + slot) * D;
            auto emit = [&](int j, const float2 v) {
                float a = v.x * rn * (w ? w[2 * j] : 1.f), b = v.y * rn * (w ? w[2 * j + 1] : 1.f);
                if (2 * j < rot_dims) {
                    float sn, cs;
                    sincosf(pf * inv_freq[j], &sn, &cs);
                    sn *= mag; cs *= mag;
                    const float ra = a * cs - b * sn, rb = b * cs + a * sn;
                    a = ra; b = rb;
                }
                if (is_q) st2(qo + 2 * j, a, b); else st2(ko + 2 * j, a, b);
            };
#pragma unroll
            for (int u = 0; u < kKeep; ++u)
                if (lane + 32 * u < np) emit(lane + 32 * u, keep[u]);
            for (int j = lane + 32 * kKeep; j < np; j += 32) emit(j, ld2(x + 2 * j));
            continue;
        }
        for (int c = lane; c < D; c += 32) { const float v = ldf(x + c); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float rn = ((w || ao.unit_norm) ? 1.f / sqrtf(ss / (float)D + eps) : 1.f) * ((is_q && ao.q_head_scale) ? ao.q_head_scale[hd] : 1.f);
        for (int c = lane; c < D; c += 32) {
            float v = ldf(x + c) * rn * (w ? w[c] : 1.f);
            if (c < rot_dims) {
                // the pair (u, v) becomes (u cos - v sin, v cos + u sin): `first` tells which member this channel is
                const bool first = rot_pairs ? !(c & 1) : c < half;
                const int i = rot_pairs ? (c >> 1) : (first ? c : c - half);
                const int pc = rot_pairs ? (c ^ 1) : (first ? c + half : c - half);
                const float o = ldf(x + pc) * rn * (w ? w[pc] : 1.f);
                const float ang = pf * inv_freq[i];
                float sn, cs;
                sincosf(ang, &sn, &cs);
                sn *= mag; cs *= mag;
                v = first ? v * cs - o * sn : v * cs + o * sn;
            }
            if (is_q) q_out[((size_t)t * Hq + hd) * D + c] = v;
            else stf(k_pages + (((size_t)page * G + (hd - Hq)) * page_size + slot) * D + c, v);
        }
    }
    const int nv = G * DV;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < nv; i += gridDim.y * blockDim.x) {
        const int g = i / DV, d = i % DV;
        T* dst = v_pages + (((size_t)page * G + g) * page_size + slot) * DV + d;
        if (ao.v_keep) ((T*)ao.v_keep)[(size_t)t * ao.ld_keep + i] = row[v_col + i];
        if (ao.v_mix) stf(dst, fmaf(ao.mix, ldf((const T*)ao.v_mix + (size_t)t * ao.ld_mix + i), (1.f - ao.mix) * ldf(row + v_col + i)));
        else *dst = row[v_col + i];
    }
}

// One CTA per new row.
template <typename T>
__global__ void __launch_bounds__(256) qk_norm_kv_append_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ qn_w,
                                                                const float* __restrict__ kn_w, float eps, float* __restrict__ q_out,
                                                                T* __restrict__ k_pages, T* __restrict__ v_pages,
                                                                const int* __restrict__ page_table, int page_size, int S, int Hq,
                                                                int G, int D, int DV, SeqPos pos) {
    if (seq_done(pos)) return;
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int p = seq_past(pos, S) + t;
    const T* row = proj + (size_t)t * ld;
    const int nq = Hq * D, nk = G * D, nv = G * DV;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = ldf(row + i); sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = ldf(row + nq + i); sk = fmaf(v, v, sk); }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float rq = 1.f / sqrtf(sq / (float)nq + eps), rk = 1.f / sqrtf(sk / (float)nk + eps);
    for (int i = threadIdx.x; i < nq; i += blockDim.x) q_out[(size_t)t * nq + i] = ldf(row + i) * rq * qn_w[i];
    const int page = page_table[p / page_size], slot = p % page_size;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int g = i / D, d = i % D;
        stf(k_pages + (((size_t)page * G + g) * page_size + slot) * D + d, ldf(row + nq + i) * rk * kn_w[i]);
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int g = i / DV, d = i % DV;
        v_pages[(((size_t)page * G + g) * page_size + slot) * DV + d] = row[nq + nk + i];
    }
}

// Decode steps and portions of fewer than kAttnTiledMin rows: one CTA per (new row, query head). Scores of the row's chunk go to shared memory (fp32), then the weights, then
// thread c accumulates output channel c over the keys.
template <typename T>
__global__ void __launch_bounds__(128) attn_chunk_sink_kernel(const float* __restrict__ q, const T* __restrict__ k_pages,
                                                              const T* __restrict__ v_pages, const int* __restrict__ page_table,
                                                              int page_size, const T* __restrict__ gate, int ld_gate,
                                                              T* __restrict__ out, int ld_out, int S, int Hq, int G, int D, int DV,
                                                              int chunk, float scale, SeqPos pos,
                                                              const float* __restrict__ sink, int ld_v, AttnOpts opt) {
    if (seq_done(pos)) return;
    extern __shared__ float sm[];
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y;
    const float sk = opt.no_sink ? -INFINITY : (sink ? sink[h] : 0.f);   // the row sees itself, so the maximum is finite
    const int g = h / (Hq / G);
    const int p = seq_past(pos, S) + t;
    const int start = first_key(p, chunk, opt.window);
    const int nkeys = p - start + 1;
    float* sq = sm;           // [D]
    float* sc = sm + D;       // [nkeys]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < D; i += blockDim.x) sq[i] = q[((size_t)t * Hq + h) * D + i];
    __syncthreads();
    // scores: one warp per key, lanes over the head dimension
    float mx = sk;  // the sink's score
    for (int jk = warp; jk < nkeys; jk += nwarps) {
        const int pj = start + jk;
        const T* kr = k_pages + (((size_t)page_table[pj / page_size] * G + g) * page_size + pj % page_size) * D;
        float acc = 0.f;
        for (int d = lane; d < D; d += 32) acc = fmaf(sq[d], ldf(kr + d), acc);
        acc = warp_sum(acc) * scale;
        if (lane == 0) sc[jk] = acc;
        mx = fmaxf(mx, acc);
    }
    mx = warp_max(mx);
    __syncthreads();
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < nwarps; ++i) mx = fmaxf(mx, red[i]);
    float sum = 0.f;
    for (int jk = threadIdx.x; jk < nkeys; jk += blockDim.x) {
        const float e = expf(sc[jk] - mx);
        sc[jk] = e;
        sum += e;
    }
    sum = block_sum(sum, red);   // contains the barrier that publishes sc[]
    const float inv = 1.f / (expf(sk - mx) + sum);
    for (int c = threadIdx.x; c < DV; c += blockDim.x) {
        float acc = 0.f;
        for (int jk = 0; jk < nkeys; ++jk) {
            const int pj = start + jk;
            const T* vr = v_pages + (((size_t)page_table[pj / page_size] * G + g) * page_size + pj % page_size) * ld_v;
            acc = fmaf(sc[jk], ldf(vr + c), acc);
        }
        const float gv = gate ? gate_of(gate, ld_gate, t, h, c, DV, opt.gate_channel) : 1.f;
        stf(out + (size_t)t * ld_out + (size_t)h * DV + c, acc * inv * gv);
    }
}

// Few rows over many keys (decode steps of plain causal attention, where the window is the whole sequence and, in a
// replayed step, only the device knows its length): one CTA per (row, head, split). The CTA walks key tiles split,
// split + n_splits, ... of kSplitKeys keys each (so any length works with any grid; the grid only sets the parallelism), keeps
// the running (max, sum, output) over its tiles, and leaves them in the workspace; the CTA that arrives last at the
// (row, head) counter merges the splits with the sink's term, applies the gate and writes the row. The counter goes back to
// zero for the next launch.
constexpr int kSplitKeys = 128, kSplitMaxOut = 4;   // output channels per thread: DV <= 128 * kSplitMaxOut
// The arrival counters take a fixed area at the head of the workspace, whatever the row and head counts of a call: partials
// of one call must never lie where another call (a layer with other sizes) keeps its counters.
constexpr int kSplitMaxHeads = 512, kSplitCounters = (kAttnTiledMin - 1) * kSplitMaxHeads;
template <typename T> struct RowVec;
template <> struct RowVec<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
    }
};
template <> struct RowVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 u = *reinterpret_cast<const float4*>(p);
        v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
    }
};

template <typename T, bool VEC>
__global__ void __launch_bounds__(128) attn_split_kernel(const float* __restrict__ q, const T* __restrict__ k_pages,
                                                         const T* __restrict__ v_pages, const int* __restrict__ page_table,
                                                         int page_size, const T* __restrict__ gate, int ld_gate,
                                                         T* __restrict__ out, int ld_out, int S, int Hq, int G, int D, int DV,
                                                         float scale, SeqPos pos, const float* __restrict__ sink, int ld_v,
                                                         float* __restrict__ part, int* __restrict__ counters, AttnOpts opt) {
    if (seq_done(pos)) return;
    extern __shared__ float sm[];
    __shared__ float red[32];
    __shared__ float redm[4];
    __shared__ int row_of[kSplitKeys];     // a key's row in the page pool: (page * G + g) * page_size + slot
    __shared__ int last_flag;
    float* sq = sm;            // [D]
    float* sc = sm + D;        // [kSplitKeys]
    const int t = blockIdx.y, h = blockIdx.x, z = blockIdx.z, nz = gridDim.z;
    const int g = h / (Hq / G);
    const int nkeys = seq_past(pos, S) + t + 1;
    // with a window the walk starts at the tile that holds the row's first key; keys of that tile before it are masked
    const int kfirst = first_key(nkeys - 1, 0, opt.window), tile0 = kfirst / kSplitKeys;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < D; i += blockDim.x) sq[i] = q[((size_t)t * Hq + h) * D + i] * scale;
    float m = -INFINITY, l = 0.f;
    float o[kSplitMaxOut] = {};                      // scalar form: thread c owns channels c, c + 128, ...
    constexpr int VN = VEC ? RowVec<T>::N : 1, NP = VEC ? 128 * kSplitMaxOut / (32 * RowVec<T>::N) : 1;
    float ov[NP][VN] = {};                           // vector form: a warp's sum over ITS keys of 16-byte pieces lane, lane + 32, ...
    float* osum = sc + kSplitKeys;                   // [4][DV], vector form only
    for (int k0 = (tile0 + z) * kSplitKeys; k0 < nkeys; k0 += nz * kSplitKeys) {
        const int nk = min(kSplitKeys, nkeys - k0);
        __syncthreads();       // sq is staged; the previous tile's weights are consumed
        // every key's row in the page pool first (one page-table read per thread, all in flight together)
        for (int j = threadIdx.x; j < nk; j += blockDim.x) {
            const int pj = k0 + j;
            row_of[j] = (int)(((size_t)page_table[pj / page_size] * G + g) * page_size + pj % page_size);
        }
        __syncthreads();
        float mx = -INFINITY;
        // a warp takes KG consecutive keys at a time and has all their loads in flight before it sums
        constexpr int KG = VEC ? 8 : 4;
        for (int j0 = warp * KG; j0 < nk; j0 += 4 * KG) {
            const T* kr[KG];
#pragma unroll
            for (int j = 0; j < KG; ++j) kr[j] = k_pages + (size_t)row_of[min(j0 + j, nk - 1)] * D;
            float acc[KG];
#pragma unroll
            for (int j = 0; j < KG; ++j) acc[j] = 0.f;
            if constexpr (VEC) {
                constexpr int V = RowVec<T>::N;
                for (int d = lane * V; d < D; d += 32 * V) {
                    float kv[KG][V];
#pragma unroll
                    for (int j = 0; j < KG; ++j) RowVec<T>::load(kr[j] + d, kv[j]);
#pragma unroll
                    for (int j = 0; j < KG; ++j)
#pragma unroll
                        for (int i = 0; i < V; ++i) acc[j] = fmaf(sq[d + i], kv[j][i], acc[j]);
                }
            } else {
                for (int d = lane; d < D; d += 32) {
                    float kv[KG];
#pragma unroll
                    for (int j = 0; j < KG; ++j) kv[j] = ldf(kr[j] + d);
#pragma unroll
                    for (int j = 0; j < KG; ++j) acc[j] = fmaf(sq[d], kv[j], acc[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < KG; ++j) {
                float v = warp_sum(acc[j]);
                if (k0 + j0 + j < kfirst) v = -INFINITY;       // before the window (first tile only)
                if (j0 + j < nk) {
                    if (lane == 0) sc[j0 + j] = v;
                    mx = fmaxf(mx, v);
                }
            }
        }
        if (lane == 0) redm[warp] = mx;
        __syncthreads();
        mx = fmaxf(fmaxf(redm[0], redm[1]), fmaxf(redm[2], redm[3]));
        const float mn = fmaxf(m, mx);
        const float corr = expf(m - mn);            // exp(-inf) = 0 on the first tile
        float sum = 0.f;
        for (int jk = threadIdx.x; jk < nk; jk += blockDim.x) {
            const float e = expf(sc[jk] - mn);
            sc[jk] = e;
            sum += e;
        }
        sum = block_sum(sum, red);                  // contains the barrier that publishes sc[]
        l = fmaf(l, corr, sum);
        m = mn;
        if constexpr (VEC) {
            // a warp takes eight consecutive keys at a time; its lanes read 16-byte pieces of their value rows, all in flight
            // together. The four warps' sums are added after the last tile.
#pragma unroll
            for (int p = 0; p < NP; ++p)
#pragma unroll
                for (int i = 0; i < VN; ++i) ov[p][i] *= corr;
            for (int j0 = warp * 8; j0 < nk; j0 += 32) {
#pragma unroll
                for (int p = 0; p < NP; ++p) {
                    const int c = (lane + 32 * p) * VN;
                    if (c < DV) {
                        float vv[8][VN];
#pragma unroll
                        for (int j = 0; j < 8; ++j) RowVec<T>::load(v_pages + (size_t)row_of[min(j0 + j, nk - 1)] * ld_v + c, vv[j]);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float wj = j0 + j < nk ? sc[j0 + j] : 0.f;
#pragma unroll
                            for (int i = 0; i < VN; ++i) ov[p][i] = fmaf(wj, vv[j][i], ov[p][i]);
                        }
                    }
                }
            }
            continue;
        }
#pragma unroll
        for (int u = 0; u < kSplitMaxOut; ++u) {
            const int c = threadIdx.x + u * 128;
            if (c < DV) {
                float acc = o[u] * corr;
                // eight rows' loads in flight at a time; the rows' places in the pages were left by the score pass
                for (int j0 = 0; j0 < nk; j0 += 8) {
                    float vv[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) vv[j] = ldf(v_pages + (size_t)row_of[min(j0 + j, nk - 1)] * ld_v + c);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (j0 + j < nk) acc = fmaf(sc[j0 + j], vv[j], acc);
                }
                o[u] = acc;
            }
        }
    }
    // partials of this split: [max, sum, out[DV]]
    float* mine = part + (((size_t)t * Hq + h) * nz + z) * (DV + 2);
    if (threadIdx.x == 0) { mine[0] = m; mine[1] = l; }
    if constexpr (VEC) {
        __syncthreads();                             // the last tile's weights are consumed (osum lies behind them)
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            const int c = (lane + 32 * p) * VN;
            if (c < DV)
#pragma unroll
                for (int i = 0; i < VN; ++i) osum[(size_t)warp * DV + c + i] = ov[p][i];
        }
        __syncthreads();
        for (int c = threadIdx.x; c < DV; c += blockDim.x)
            mine[2 + c] = (osum[c] + osum[DV + c]) + (osum[2 * DV + c] + osum[3 * DV + c]);
    } else {
#pragma unroll
        for (int u = 0; u < kSplitMaxOut; ++u) {
            const int c = threadIdx.x + u * 128;
            if (c < DV) mine[2 + c] = o[u];
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_flag = atomicAdd(counters + t * Hq + h, 1) == nz - 1;
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    const float* all = part + ((size_t)t * Hq + h) * nz * (DV + 2);
    const float sk = opt.no_sink ? -INFINITY : (sink ? sink[h] : 0.f);   // split 0 holds the row's first key: mt is finite
    float mt = sk;
    for (int i = 0; i < nz; ++i) mt = fmaxf(mt, __ldcg(all + (size_t)i * (DV + 2)));
    float lt = expf(sk - mt);                       // the sink: weight in the denominator, no value
    for (int i = 0; i < nz; ++i) lt = fmaf(__ldcg(all + (size_t)i * (DV + 2) + 1), expf(__ldcg(all + (size_t)i * (DV + 2)) - mt), lt);
    const float f = 1.f / lt;
    for (int c = threadIdx.x; c < DV; c += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < nz; ++i)
            acc = fmaf(__ldcg(all + (size_t)i * (DV + 2) + 2 + c), expf(__ldcg(all + (size_t)i * (DV + 2)) - mt), acc);
        const float gv = gate ? gate_of(gate, ld_gate, t, h, c, DV, opt.gate_channel) : 1.f;
        stf(out + (size_t)t * ld_out + (size_t)h * DV + c, acc * f * gv);
    }
    if (threadIdx.x == 0) counters[t * Hq + h] = 0;
}

// Prompt portions: one CTA per (64 query rows, query head, 128 output channels). Keys are walked in tiles of 64 from the
// start of the chunk of the tile's first row to its last row. Per key tile the CTA stages the K tile (up to 128 head
// channels at a time) and the V tile into shared memory in the storage type with all its loads in flight together, forms
// the scores as a register-tiled fp32 product (4 x 4 per thread; the fp32 queries are staged once), runs the softmax in
// the running (max, sum) form started at max = 0, sum = 1, which is exactly the sink's term, and passes the weights
// through shared memory into the product with V (4 x 8 per thread).
constexpr int AQ = 64, AK = 64, ADC = 128, AVW = 128, APQ = AQ + 4, APV = AVW + 4;

template <typename T> __device__ __forceinline__ void ld4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void ld4<float>(const float* p, float (&v)[4]) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
}
template <> __device__ __forceinline__ void ld4<bf16>(const bf16* p, float (&v)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

template <typename T>
size_t attn_tiled_smem(int D) {
    const size_t dc = D < ADC ? D : ADC;
    return dc * APQ * 4 + dc * APQ * sizeof(T) + (size_t)AK * APV * sizeof(T) + (size_t)AK * APQ * 4;
}

template <typename T>
__global__ void __launch_bounds__(256) attn_chunk_sink_tiled_kernel(const float* __restrict__ q, const T* __restrict__ k_pages,
                                                                    const T* __restrict__ v_pages, const int* __restrict__ page_table,
                                                                    int page_size, const T* __restrict__ gate, int ld_gate,
                                                                    T* __restrict__ out, int ld_out, int S, int Hq, int G, int D, int DV,
                                                                    int chunk, float scale, SeqPos pos,
                                                                    const float* __restrict__ sink, int ld_v, AttnOpts opt) {
    if (seq_done(pos)) return;
    extern __shared__ __align__(16) uint8_t smem_attn[];
    const int dc = min(D, ADC);
    float* sq_ = reinterpret_cast<float*>(smem_attn);                     // [dc][APQ]
    float* sp_ = sq_ + (size_t)dc * APQ;                                  // [AK][APQ]
    T* sk_ = reinterpret_cast<T*>(sp_ + (size_t)AK * APQ);                // [dc][APQ]
    T* sv_ = sk_ + (size_t)dc * APQ;                                      // [AK][APV]
    // heavy (late) query tiles first, for all heads, then the lighter ones: a tile's work grows with its distance from the
    // start of its chunk, and CTAs are handed out in order of blockIdx.x, then y
    const int t0 = (gridDim.y - 1 - blockIdx.y) * AQ, h = blockIdx.x, c0 = blockIdx.z * AVW;
    const int g = h / (Hq / G);
    const int past = seq_past(pos, S);
    const int rows = min(AQ, S - t0);
    const int pf = past + t0, pl = pf + rows - 1;
    const int kbeg = first_key(pf, chunk, opt.window);       // the first row's first key: no later row starts earlier
    const int tm = (threadIdx.x / 16) * 4, tn = (threadIdx.x % 16) * 4;
    const int lr = threadIdx.x / 16, lc = threadIdx.x % 16;              // staging: 16 threads walk a row
    int p_row[4], lo_row[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        p_row[i] = pf + tm + i;
        lo_row[i] = first_key(p_row[i], chunk, opt.window);
    }
    const float sk = opt.no_sink ? kNoSinkMax : (sink ? sink[blockIdx.x] : 0.f);
    const float l0 = opt.no_sink ? 0.f : 1.f;
    float m[4] = {sk, sk, sk, sk}, l[4] = {l0, l0, l0, l0};
    float o[4][8] = {};
    const float* qh = q + ((size_t)t0 * Hq + h) * D;
    const bool q_once = D <= ADC;
    bool q_staged = false;
    for (int k0 = kbeg; k0 <= pl; k0 += AK) {
        const int nk = min(AK, pl - k0 + 1);
        size_t row_off[4];                               // this thread's 4 key rows of the tile, as (page, group, slot) bases
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int pj = k0 + lr + 16 * j;
            row_off[j] = pj <= pl ? ((size_t)page_table[pj / page_size] * G + g) * page_size + pj % page_size : 0;
        }
        float sc[4][4] = {};
        for (int d0 = 0; d0 < D; d0 += ADC) {
            const int dn = min(ADC, D - d0);
            __syncthreads();
            if (!q_staged) {
                for (int j = 0; j < 4; ++j) {
                    const int r = lr + 16 * j;
                    for (int d = lc; d < dn; d += 16) sq_[d * APQ + r] = r < rows ? qh[(size_t)r * Hq * D + d0 + d] : 0.f;
                }
                q_staged = q_once;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = lr + 16 * j;
                const T* kr = k_pages + row_off[j] * D + d0;
                if (r < nk) {
#pragma unroll 8
                    for (int d = lc; d < dn; d += 16) sk_[d * APQ + r] = kr[d];
                } else {
                    for (int d = lc; d < dn; d += 16) sk_[d * APQ + r] = T(0.f);
                }
            }
            if (d0 == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = lr + 16 * j;
                    const T* vr = v_pages + row_off[j] * ld_v + c0;
                    if (r < nk) {
#pragma unroll 8
                        for (int c = lc; c < AVW; c += 16) sv_[r * APV + c] = c0 + c < DV ? vr[c] : T(0.f);
                    }
                }
            }
            __syncthreads();
#pragma unroll 8
            for (int kk = 0; kk < dn; ++kk) {
                const float4 av = *reinterpret_cast<const float4*>(sq_ + kk * APQ + tm);
                const float a[4] = {av.x, av.y, av.z, av.w};
                float b[4];
                ld4(sk_ + kk * APQ + tn, b);
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) sc[i][j] = fmaf(a[i], b[j], sc[i][j]);
            }
        }
        // running softmax; the 16 threads that share a row are 16 neighbouring lanes of one warp
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int pj = k0 + tn + j;
                const bool ok = pj <= p_row[i] && pj >= lo_row[i] && tm + i < rows;
                sc[i][j] = ok ? sc[i][j] * scale : -INFINITY;
                mx = fmaxf(mx, sc[i][j]);
            }
#pragma unroll
            for (int w = 8; w > 0; w >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));
            const float mn = fmaxf(m[i], mx);          // finite: m starts at the sink's score
            const float corr = expf(m[i] - mn);
            float rs = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float pw = expf(sc[i][j] - mn);  // exp(-inf) = 0 for masked keys
                sp_[(tn + j) * APQ + tm + i] = pw;
                rs += pw;
            }
#pragma unroll
            for (int w = 8; w > 0; w >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, w);
            l[i] = fmaf(l[i], corr, rs);
            m[i] = mn;
#pragma unroll
            for (int c = 0; c < 8; ++c) o[i][c] *= corr;
        }
        __syncthreads();
#pragma unroll 4
        for (int kk = 0; kk < nk; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(sp_ + kk * APQ + tm);
            const float a[4] = {av.x, av.y, av.z, av.w};
            float b0[4], b1[4];
            ld4(sv_ + kk * APV + tn, b0);
            ld4(sv_ + kk * APV + 64 + tn, b1);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    o[i][c] = fmaf(a[i], b0[c], o[i][c]);
                    o[i][4 + c] = fmaf(a[i], b1[c], o[i][4 + c]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + tm + i;
        if (tm + i >= rows) continue;
        const float f = 1.f / l[i];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int col = c0 + (c < 4 ? tn + c : 64 + tn + c - 4);
            if (col < DV) {
                const float gv = gate ? gate_of(gate, ld_gate, t, h, col, DV, opt.gate_channel) : 1.f;
                stf(out + (size_t)t * ld_out + (size_t)h * DV + col, o[i][c] * f * gv);
            }
        }
    }
}

template <typename T>
int launch_attn_tiled(const float* q, const void* k_pages, const void* v_pages, const int* page_table, int page_size,
                      const void* gate, int ld_gate, void* out, int ld_out, int S, int Hq, int G, int D, int DV, int chunk,
                      float scale, SeqPos pos, cudaStream_t s, const float* sink, int ld_v, AttnOpts opt) {
    static SmemAttrOnce once;
    const size_t smem = attn_tiled_smem<T>(ADC);
    if (ensure_dyn_smem(once, attn_chunk_sink_tiled_kernel<T>, (int)smem)) return -100;
    dim3 grid(Hq, (S + AQ - 1) / AQ, (DV + AVW - 1) / AVW);
    count_launch();
    attn_chunk_sink_tiled_kernel<T><<<grid, 256, attn_tiled_smem<T>(D), s>>>(q, (const T*)k_pages, (const T*)v_pages, page_table, page_size,
                                                                            (const T*)gate, ld_gate, (T*)out, ld_out, S, Hq, G, D, DV,
                                                                            chunk, scale, pos, sink, ld_v, opt);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

// bf16 storage, head sizes up to 256: the same tiling on the tensor cores. One CTA per (64 query rows, query head, 128
// output channels) of one or (head size <= 128, aligned rows) two groups of 4 warps; a warp owns 16 query rows, the groups
// take alternate key tiles and merge their (max, sum, output) at the end. Q (rounded to bf16 once), the K tile and the V tile sit in shared
// memory as bf16 rows padded to whole 16-channel steps (zeros; when rows are 16-byte aligned the K/V tiles are double-
// buffered asynchronous copies); scores and the product with V are mma.sync m16n8k16 with
// fp32 accumulators, the softmax (running max and sum started at the sink's term, exp in fp32) works on the accumulator
// fragments, and the weights go to the second product as bf16 A fragments straight from registers.
constexpr int MQ = 64, MK = 64;

// rows that are not 16-byte aligned: element-wise staging
template <typename RowPtr>
__device__ __forceinline__ void stage_bf16_rows(bf16* dst, int ld_dst, int ncp, int ncv, RowPtr rowptr) {
    for (int u = threadIdx.x; u < MK * ncp; u += blockDim.x) {
        const int r = u / ncp, c = u % ncp;
        const bf16* p = rowptr(r);
        dst[(size_t)r * ld_dst + c] = (p && c < ncv) ? p[c] : __float2bfloat16_rn(0.f);
    }
}

// NBUF (VEC8 only): 2 = the next tile's copies fly while this one is computed; 1 = one buffer, which halves the shared memory so
// that two CTAs share an SM and hide each other's copies and tensor-pipe latency instead.
template <bool VEC8, int KH, int NV, int NBUF = 2>
__global__ void __launch_bounds__(128 * KH, (VEC8 && NBUF == 1) ? 2 : 0) attn_chunk_sink_mma_kernel(const float* __restrict__ q, const bf16* __restrict__ k_pages,
                                                                  const bf16* __restrict__ v_pages, const int* __restrict__ page_table,
                                                                  int page_size, const bf16* __restrict__ gate, int ld_gate,
                                                                  bf16* __restrict__ out, int ld_out, int S, int Hq, int G, int D, int DV,
                                                                  int chunk, float scale, SeqPos pos,
                                                                  const float* __restrict__ sink, int ld_v, AttnOpts opt) {
    if (seq_done(pos)) return;
    extern __shared__ __align__(16) uint8_t smem_attn[];
    // NV output tiles of 128 channels per CTA (NV = 2: values of up to 256 channels against one pass over the scores)
    constexpr int MVW = 128 * NV, MLV = MVW + 8;
    const int Dp = (D + 15) / 16 * 16, LQ = Dp + 8;
    bf16* sQ = reinterpret_cast<bf16*>(smem_attn);     // [MQ][LQ]
    constexpr int KT = KH * MK;                         // keys per step of the CTA: one 64-key tile per group of 4 warps
    bf16* sK0 = sQ + (size_t)MQ * LQ;                   // [2][KT][LQ]   (the second buffer only with VEC8)
    bf16* sV0 = sK0 + (size_t)(VEC8 ? NBUF : 1) * KT * LQ; // [2][KT][MLV]
    const int t0 = (gridDim.y - 1 - blockIdx.y) * MQ, h = blockIdx.x, c0 = blockIdx.z * MVW;
    const int g = h / (Hq / G);
    const int past = seq_past(pos, S);
    const int rows = min(MQ, S - t0);
    const int pf = past + t0, pl = pf + rows - 1;
    const int kbeg = first_key(pf, chunk, opt.window);       // the first row's first key: no later row starts earlier
    const int dvv = min(MVW, DV - c0), DVp = (dvv + 15) / 16 * 16;
    const int warp = (threadIdx.x >> 5) & 3, kh = threadIdx.x >> 7, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    // queries: fp32 -> bf16, zero padding
    for (int u = threadIdx.x; u < MQ * (Dp / 2); u += blockDim.x) {
        const int r = u / (Dp / 2), d = (u % (Dp / 2)) * 2;
        const float* qr = q + ((size_t)(t0 + r) * Hq + h) * D;
        const float v0 = (r < rows && d < D) ? qr[d] : 0.f, v1 = (r < rows && d + 1 < D) ? qr[d + 1] : 0.f;
        *reinterpret_cast<uint32_t*>(sQ + (size_t)r * LQ + d) = pack_bf16x2(v0, v1);
    }
    const int r_lo = warp * 16 + gq;                    // this thread's two rows of the tile: r_lo and r_lo + 8
    int p_row[2], lo_row[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        p_row[i] = pf + r_lo + 8 * i;
        lo_row[i] = first_key(p_row[i], chunk, opt.window);
    }
    const float sk = opt.no_sink ? kNoSinkMax : (sink ? sink[blockIdx.x] : 0.f);
    float m[2] = {sk, sk};
    // per-thread partial sums; the sink's 1 is counted once per row (by one thread of the first group of warps)
    const float l0 = (tq == 0 && kh == 0 && !opt.no_sink) ? 1.f : 0.f;
    float l[2] = {l0, l0};
    float o[16 * NV][4] = {};
    // VEC8: a tile's K and V rows arrive by 16-byte asynchronous copies (zero-filled past the last key and in the padding
    // columns), all in flight together, into the buffer the previous tile does not use, while that tile is computed
    auto issue = [&](int k0, int buf) {
        bf16* dK = sK0 + (size_t)buf * KT * LQ;
        bf16* dV = sV0 + (size_t)buf * KT * MLV;
        // a warp walks rows, its lanes walk a row's 16-byte pieces; page and slot advance without divisions
        const int kpr = Dp / 8, vpr = DVp / 8, nw = blockDim.x >> 5, wid = threadIdx.x >> 5;
        int pj = k0 + wid, pg = pj / page_size, slot = pj - pg * page_size;
        for (int r = wid; r < KT; r += nw) {
            const bool row_ok = pj <= pl;
            const size_t ro = row_ok ? ((size_t)page_table[pg] * G + g) * page_size + slot : 0;
            for (int cu = lane; cu < kpr + vpr; cu += 32) {
                if (cu < kpr) {
                    const int c = cu * 8;
                    const bool ok = row_ok && c < D;
                    cp_async16(dK + (size_t)r * LQ + c, ok ? k_pages + ro * D + c : k_pages, ok);
                } else {
                    const int c = (cu - kpr) * 8;
                    const bool ok = row_ok && c < dvv;
                    cp_async16(dV + (size_t)r * MLV + c, ok ? v_pages + ro * ld_v + c0 + c : v_pages, ok);
                }
            }
            pj += nw; slot += nw;
            while (slot >= page_size) { slot -= page_size; ++pg; }
        }
        cp_async_commit();
    };
    if (VEC8 && NBUF == 2) issue(kbeg, 0);
    int it = 0;
    for (int kc = kbeg; kc <= pl; kc += KT, ++it) {
        const int buf = (VEC8 && NBUF == 2) ? (it & 1) : 0;
        const int k0 = kc + kh * MK;                    // this group of warps' tile of the step
        const bf16* sK = sK0 + ((size_t)buf * KT + kh * MK) * LQ;
        const bf16* sV = sV0 + ((size_t)buf * KT + kh * MK) * MLV;
        if (VEC8 && NBUF == 1) {
            __syncthreads();       // every thread is done with the previous tile (and Q is staged)
            issue(kc, 0);
            cp_async_wait<0>();
            __syncthreads();
        } else if (VEC8) {
            cp_async_wait<0>();
            __syncthreads();       // this tile has landed for every thread, and every thread is done with the other buffer
            if (kc + KT <= pl) issue(kc + KT, buf ^ 1);
        } else {
            auto krow = [&](int r) -> const bf16* {
                const int pj = kc + r;
                return pj <= pl ? k_pages + (((size_t)page_table[pj / page_size] * G + g) * page_size + pj % page_size) * D : nullptr;
            };
            auto vrow = [&](int r) -> const bf16* {
                const int pj = kc + r;
                return pj <= pl ? v_pages + (((size_t)page_table[pj / page_size] * G + g) * page_size + pj % page_size) * ld_v + c0 : nullptr;
            };
            __syncthreads();
            stage_bf16_rows(sK0, LQ, Dp, D, krow);
            stage_bf16_rows(sV0, MLV, DVp, dvv, vrow);
            __syncthreads();
        }
        if (k0 > pl) continue;                          // no tile left for this group in the last step (barriers are above)
        float sc[8][4] = {};
        for (int ks = 0; ks < Dp; ks += 16) {
            uint32_t a[4];
            ldmatrix_x4(a[0], a[1], a[2], a[3], sQ + (size_t)(warp * 16 + (lane & 15)) * LQ + ks + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, sK + (size_t)(np * 16 + (lane & 7) + (lane >> 4) * 8) * LQ + ks + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(sc[2 * np], a, b0, b1);
                mma_bf16_16816(sc[2 * np + 1], a, b2, b3);
            }
        }
        // softmax on the fragments: elements 0, 1 belong to row r_lo, elements 2, 3 to row r_lo + 8; columns j * 8 + 2 tq (+1).
        // A tile every row of the CTA sees in full (at or after the last row's chunk start, wholly before the first row)
        // skips the mask. The exponentials are exp2 of pre-scaled arguments: their error (2^-22) is far below the bf16
        // rounding of the weights that follows.
        const bool full = k0 + MK - 1 <= pf && rows == MQ && k0 >= first_key(pl, chunk, opt.window);
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float v = sc[j][2 * i + e] * scale;
                    if (!full) {
                        const int pj = k0 + j * 8 + 2 * tq + e;
                        const bool ok = pj <= p_row[i] && pj >= lo_row[i] && r_lo + 8 * i < rows;
                        v = ok ? v : -INFINITY;
                    }
                    sc[j][2 * i + e] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m[i], mx);          // finite: m starts at the sink's score
            constexpr float kLog2e = 1.4426950408889634f;
            corr[i] = exp2f((m[i] - mn) * kLog2e);
            const float mn2 = mn * kLog2e;
            float rs = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pw = exp2f(fmaf(sc[j][2 * i + e], kLog2e, -mn2));
                    sc[j][2 * i + e] = pw;
                    rs += pw;
                }
            l[i] = fmaf(l[i], corr[i], rs);
            m[i] = mn;
        }
#pragma unroll
        for (int nt = 0; nt < 16 * NV; ++nt) { o[nt][0] *= corr[0]; o[nt][1] *= corr[0]; o[nt][2] *= corr[1]; o[nt][3] *= corr[1]; }
#pragma unroll
        for (int j2 = 0; j2 < 4; ++j2) {
            if (k0 + j2 * 16 > pl) break;              // uniform: the tile's remaining keys do not exist
            uint32_t a[4];
            a[0] = pack_bf16x2(sc[2 * j2][0], sc[2 * j2][1]);
            a[1] = pack_bf16x2(sc[2 * j2][2], sc[2 * j2][3]);
            a[2] = pack_bf16x2(sc[2 * j2 + 1][0], sc[2 * j2 + 1][1]);
            a[3] = pack_bf16x2(sc[2 * j2 + 1][2], sc[2 * j2 + 1][3]);
#pragma unroll
            for (int ntp = 0; ntp < 8 * NV; ++ntp) {
                if (ntp * 16 < DVp) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, sV + (size_t)(j2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * MLV + ntp * 16 + (lane >> 4) * 8);
                    mma_bf16_16816(o[2 * ntp], a, b0, b1);
                    mma_bf16_16816(o[2 * ntp + 1], a, b2, b3);
                }
            }
        }
    }
    static_assert(KH == 1 || NV == 1, "two groups of warps exchange one 128-channel tile");
    if (KH > 1 && NV == 1) {
        // the second group hands its (max, partial sum, unnormalised output) to the first through the tile buffers (K and V
        // buffers are contiguous; every asynchronous copy was waited for in the last step)
        float* xch = reinterpret_cast<float*>(sK0);
        const int tix = threadIdx.x & 127;
        __syncthreads();                                // every warp is done with the K/V buffers
        if (kh == 1) {
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) xch[(nt * 4 + e) * 128 + tix] = o[nt][e];
#pragma unroll
            for (int i = 0; i < 2; ++i) { xch[(64 + i) * 128 + tix] = m[i]; xch[(66 + i) * 128 + tix] = l[i]; }
        }
        __syncthreads();
        if (kh == 1) return;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float m1 = xch[(64 + i) * 128 + tix], l1 = xch[(66 + i) * 128 + tix];
            const float mn = fmaxf(m[i], m1);
            const float f0 = expf(m[i] - mn), f1 = expf(m1 - mn);
            l[i] = l[i] * f0 + l1 * f1;
            m[i] = mn;
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e)
                    o[nt][2 * i + e] = o[nt][2 * i + e] * f0 + xch[(nt * 4 + 2 * i + e) * 128 + tix] * f1;
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float lt = l[i];
        lt += __shfl_xor_sync(0xffffffffu, lt, 1);
        lt += __shfl_xor_sync(0xffffffffu, lt, 2);
        const int r = r_lo + 8 * i, t = t0 + r;
        if (r >= rows) continue;
        const float gh = (gate && !opt.gate_channel) ? gate_of(gate, ld_gate, t, h, 0, DV, false) : 1.f;
        const float f = gh / lt;
#pragma unroll
        for (int nt = 0; nt < 16 * NV; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int col = nt * 8 + 2 * tq + e;
                if (col < dvv) {
                    const float gv = (gate && opt.gate_channel) ? gate_of(gate, ld_gate, t, h, c0 + col, DV, true) : 1.f;
                    stf(out + (size_t)t * ld_out + (size_t)h * DV + c0 + col, o[nt][2 * i + e] * f * gv);
                }
            }
    }
}

int launch_attn_mma(const float* q, const void* k_pages, const void* v_pages, const int* page_table, int page_size,
                    const void* gate, int ld_gate, void* out, int ld_out, int S, int Hq, int G, int D, int DV, int chunk,
                    float scale, SeqPos pos, cudaStream_t s, const float* sink, int ld_v, AttnOpts opt) {
    static SmemAttrOnce once82, once82s, once81, once1, once81w, once1w;
    // two groups of warps: one K/V buffer and two CTAs per SM (default), or two buffers and one CTA (LIVECC_B200_SEQ_ATTN_NBUF=2)
    static const int nbuf2 = [] { const char* e = getenv("LIVECC_B200_SEQ_ATTN_NBUF"); return e ? atoi(e) : 1; }();
    const int Dp = (D + 15) / 16 * 16;
    // 16-byte copies need every K and V row (and the output-channel slice) to start on a 16-byte boundary
    const bool vec8 = (D % 8) == 0 && (DV % 8) == 0 && (ld_v % 8) == 0 && ((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0;
    // two groups of warps (two key tiles per step) when four tiles of K and V fit beside Q; the exchange area of the final
    // merge (68 floats per thread of a group, 34 KB) lies over the K and V buffers, whose V part alone is 68 KB
    // values wider than 128 channels: two output tiles per CTA against one pass over the scores (one group of warps)
    const bool wide = DV > 128;
    const bool two = vec8 && Dp <= 128 && !wide;
    const int nbuf = vec8 ? ((two && nbuf2 == 1) ? 1 : 2) : 1, kh = two ? 2 : 1, MVW = wide ? 256 : 128, MLV = MVW + 8;
    auto bytes = [&](int dp) { return ((size_t)MQ * (dp + 8) + (size_t)nbuf * kh * MK * (dp + 8 + MLV)) * sizeof(bf16); };
    const size_t smem = bytes(Dp), smem_max = bytes(two ? 128 : kAttnMmaMaxDim);
    dim3 grid(Hq, (S + MQ - 1) / MQ, (DV + MVW - 1) / MVW);
    count_launch();
#define LCC_ATTN_MMA(ONCE, VEC, KHN, NVN, ...)                                                                                  \
    do {                                                                                                                     \
        if (ensure_dyn_smem(ONCE, attn_chunk_sink_mma_kernel<VEC, KHN, NVN, ##__VA_ARGS__>, (int)smem_max)) return -100;          \
        attn_chunk_sink_mma_kernel<VEC, KHN, NVN, ##__VA_ARGS__><<<grid, 128 * KHN, smem, s>>>(q, (const bf16*)k_pages, (const bf16*)v_pages, page_table, \
                                                                           page_size, (const bf16*)gate, ld_gate, (bf16*)out, ld_out, \
                                                                           S, Hq, G, D, DV, chunk, scale, pos, sink, ld_v, opt);  \
    } while (0)
    if (two && nbuf == 1) LCC_ATTN_MMA(once82s, true, 2, 1, 1);
    else if (two) LCC_ATTN_MMA(once82, true, 2, 1);
    else if (wide && vec8) LCC_ATTN_MMA(once81w, true, 1, 2);
    else if (wide) LCC_ATTN_MMA(once1w, false, 1, 2);
    else if (vec8) LCC_ATTN_MMA(once81, true, 1, 1);
    else LCC_ATTN_MMA(once1, false, 1, 1);
#undef LCC_ATTN_MMA
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace

int qk_norm_kv_append(int dt, const void* proj, int ld, const float* qn_w, const float* kn_w, float eps, float* q_out,
                      void* k_pages, void* v_pages, const int* page_table, int page_size, int S, int Hq, int G, int D,
                      int DV, SeqPos pos, cudaStream_t s) {
    if (!proj || !qn_w || !kn_w || !q_out || !k_pages || !v_pages || !page_table || S < 1 || Hq < 1 || G < 1 || D < 1 ||
        DV < 1 || page_size < 1)
        return -2;
    count_launch();
    if (dt == DT_F32)
        qk_norm_kv_append_kernel<float><<<S, 256, 0, s>>>((const float*)proj, ld, qn_w, kn_w, eps, q_out, (float*)k_pages,
                                                          (float*)v_pages, page_table, page_size, S, Hq, G, D, DV, pos);
    else
        qk_norm_kv_append_kernel<bf16><<<S, 256, 0, s>>>((const bf16*)proj, ld, qn_w, kn_w, eps, q_out, (bf16*)k_pages,
                                                         (bf16*)v_pages, page_table, page_size, S, Hq, G, D, DV, pos);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

size_t attn_split_ws_floats(int rows, int Hq, int DV) {
    return (size_t)kSplitCounters + (size_t)rows * Hq * (DV + 2) * 32;
}

int attn_chunk_sink(int dt, const float* q, const void* k_pages, const void* v_pages, const int* page_table,
                    int page_size, const void* gate, int ld_gate, void* out, int ld_out, int S, int Hq, int G, int D,
                    int DV, int chunk, float scale, bool tensor_cores, SeqPos pos, cudaStream_t s, const float* sink, int ld_v,
                    float* split_ws, size_t split_ws_floats, int key_hint) {
    return attn_masked(dt, q, k_pages, v_pages, page_table, page_size, gate, ld_gate, out, ld_out, S, Hq, G, D, DV, chunk, scale,
                       tensor_cores, pos, s, AttnOpts{0, false, false}, sink, ld_v, split_ws, split_ws_floats, key_hint);
}

int qk_headnorm_rope_append(int dt, const void* proj, int ld, int v_col, const float* qn_w, const float* kn_w, float eps,
                            const float* inv_freq, float mag, int rot_dims, int rot_pairs, float* q_out, void* k_pages,
                            void* v_pages, const int* page_table, int page_size, int S, int Hq, int G, int D, int DV, SeqPos pos,
                            cudaStream_t s, const AppendOpts* opt) {
    if (!proj || !q_out || !k_pages || !v_pages || !page_table || S < 1 || Hq < 1 || G < 1 || D < 1 || DV < 1 || page_size < 1 ||
        rot_dims < 0 || (rot_dims & 1) || rot_dims > D || (rot_dims > 0 && !inv_freq) || v_col < 0 || v_col + G * DV > ld)
        return -2;
    const AppendOpts ao = opt ? *opt : AppendOpts{false, nullptr, nullptr, 0, 0.f, nullptr, 0};
    if ((ao.v_mix && ao.ld_mix < G * DV) || (ao.v_keep && ao.ld_keep < G * DV)) return -2;
    count_launch();
    // many rows: 8 warps walk a row's heads; few rows: 4-warp CTAs, one head per warp, so that a decode step fills more SMs
    const int threads = S >= 64 ? 256 : 128;
    const dim3 grid(S, S >= 64 ? 1 : (Hq + G + 3) / 4);
    const size_t es = dt == DT_F32 ? 4 : 2;
    const bool pairs = (rot_pairs || rot_dims == 0) && (D % 2) == 0 && (ld % 2) == 0 && ((uintptr_t)proj % (2 * es)) == 0 &&
                       ((uintptr_t)k_pages % (2 * es)) == 0 && ((uintptr_t)q_out % 8) == 0;
#define LCC_APPEND(T, P)                                                                                                      \
    qk_headnorm_rope_append_kernel<T, P><<<grid, threads, 0, s>>>((const T*)proj, ld, v_col, qn_w, kn_w, eps, inv_freq, mag, rot_dims,  \
                                                                  rot_pairs, q_out, (T*)k_pages, (T*)v_pages, page_table, page_size, S, Hq, \
                                                                  G, D, DV, pos, ao)
    if (dt == DT_F32) { if (pairs) LCC_APPEND(float, true); else LCC_APPEND(float, false); }
    else { if (pairs) LCC_APPEND(bf16, true); else LCC_APPEND(bf16, false); }
#undef LCC_APPEND
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int attn_masked(int dt, const float* q, const void* k_pages, const void* v_pages, const int* page_table, int page_size,
                const void* gate, int ld_gate, void* out, int ld_out, int S, int Hq, int G, int D, int DV, int chunk, float scale,
                bool tensor_cores, SeqPos pos, cudaStream_t s, const AttnOpts& opt, const float* sink, int ld_v, float* split_ws,
                size_t split_ws_floats, int key_hint) {
    if (!q || !k_pages || !v_pages || !page_table || !out || S < 1 || Hq < 1 || G < 1 || Hq % G || D < 1 || DV < 1)
        return -2;
    if (ld_v <= 0) ld_v = DV;
    if (ld_v < DV) return -2;
    const int window = opt.window > 0 ? opt.window : 0;
    // few rows without chunks over a long or device-known range of keys: key splits across CTAs
    int keys_est = pos.kv_len ? std::max(key_hint, pos.past + S) : pos.past + S;
    if (window) keys_est = std::min(keys_est, window + kSplitKeys);   // the window, plus the masked head of its first tile
    if (chunk <= 0 && S < kAttnTiledMin && split_ws && DV <= 128 * kSplitMaxOut && Hq <= kSplitMaxHeads &&
        ((pos.kv_len && !window) || keys_est > 2 * kSplitKeys)) {
        const size_t per = (size_t)S * Hq * (DV + 2), cnt = kSplitCounters;
        int nz = std::min(32, std::max(1, (keys_est + kSplitKeys - 1) / kSplitKeys));
        if (split_ws_floats > cnt) nz = (int)std::min<size_t>(nz, (split_ws_floats - cnt) / per);
        if (split_ws_floats > cnt && nz >= 1) {
            int* counters = reinterpret_cast<int*>(split_ws);           // zero when the workspace is bound; every launch leaves zeros
            float* part = split_ws + cnt;
            const size_t smem = sizeof(float) * ((size_t)D + kSplitKeys + 4 * (size_t)DV);
            dim3 grid(Hq, S, nz);
            count_launch();
#define LCC_SPLIT(T, VECB)                                                                                                   \
    attn_split_kernel<T, VECB><<<grid, 128, smem, s>>>(q, (const T*)k_pages, (const T*)v_pages, page_table, page_size, (const T*)gate,  \
                                                       ld_gate, (T*)out, ld_out, S, Hq, G, D, DV, scale, pos, sink, ld_v, part, counters, opt)
            if (smem > 48 * 1024) return -3;
            if (dt == DT_F32) {
                if (((D | DV | ld_v) % 4) == 0 && (((uintptr_t)k_pages | (uintptr_t)v_pages) % 16) == 0) LCC_SPLIT(float, true); else LCC_SPLIT(float, false);
            } else {
                if (((D | DV | ld_v) % 8) == 0 && (((uintptr_t)k_pages | (uintptr_t)v_pages) % 16) == 0) LCC_SPLIT(bf16, true); else LCC_SPLIT(bf16, false);
            }
#undef LCC_SPLIT
            return cudaGetLastError() == cudaSuccess ? 0 : -100;
        }
    }
    // The one-CTA-per-row kernel keeps one score per key of the longest range a row of this call can see in shared memory
    // (a chunk, a window, or everything cached when the host knows the length). Ranges that do not fit (or whose length only
    // the device knows, in a replayed step without chunks or window) go to the tiled kernels, which walk the keys in tiles
    // and take any row count.
    int max_keys = chunk > 0 ? chunk : -1;
    if (window) max_keys = max_keys > 0 ? std::min(max_keys, window) : window;
    if (!pos.kv_len) max_keys = max_keys > 0 ? std::min(max_keys, pos.past + S) : pos.past + S;
    const size_t smem = sizeof(float) * ((size_t)D + (size_t)std::max(max_keys, 0));
    static const bool force_tiled = [] { const char* e = getenv("LIVECC_B200_SEQ_ATTN_TILED"); return e && e[0] == '1'; }();
    if (S >= kAttnTiledMin || max_keys < 0 || smem > 160 * 1024 || force_tiled) {
        if (dt == DT_BF16 && tensor_cores && D <= kAttnMmaMaxDim)
            return launch_attn_mma(q, k_pages, v_pages, page_table, page_size, gate, ld_gate, out, ld_out, S, Hq, G, D, DV, chunk,
                                   scale, pos, s, sink, ld_v, opt);
        if (dt == DT_F32)
            return launch_attn_tiled<float>(q, k_pages, v_pages, page_table, page_size, gate, ld_gate, out, ld_out, S, Hq, G, D, DV,
                                            chunk, scale, pos, s, sink, ld_v, opt);
        return launch_attn_tiled<bf16>(q, k_pages, v_pages, page_table, page_size, gate, ld_gate, out, ld_out, S, Hq, G, D, DV, chunk,
                                       scale, pos, s, sink, ld_v, opt);
    }
    dim3 grid(S, Hq);
    count_launch();
    if (dt == DT_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attn_chunk_sink_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attn_chunk_sink_kernel<float><<<grid, 128, smem, s>>>(q, (const float*)k_pages, (const float*)v_pages, page_table,
                                                              page_size, (const float*)gate, ld_gate, (float*)out, ld_out, S, Hq,
                                                              G, D, DV, chunk, scale, pos, sink, ld_v, opt);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attn_chunk_sink_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attn_chunk_sink_kernel<bf16><<<grid, 128, smem, s>>>(q, (const bf16*)k_pages, (const bf16*)v_pages, page_table,
                                                             page_size, (const bf16*)gate, ld_gate, (bf16*)out, ld_out, S, Hq, G,
                                                             D, DV, chunk, scale, pos, sink, ld_v, opt);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace lcc
