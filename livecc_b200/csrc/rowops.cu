// Row-wise ops of the hybrid decoder models. The residual stream, every norm and every sum of squares is fp32; `xa` /
// `out` copies in the model's storage type feed the next linear layer.
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

__device__ __forceinline__ int seq_past(const SeqPos& p, int) { return p.kv_len ? *p.kv_len : p.past; }
__device__ __forceinline__ bool seq_done(const SeqPos& p) { return p.finished && *p.finished; }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

template <typename T>
__global__ void embed_sinusoid_kernel(const int64_t* __restrict__ ids, const int* __restrict__ seq_len, const T* __restrict__ table,
                                      int64_t vocab, float scale, const float* __restrict__ inv_freq, float* __restrict__ x32,
                                      T* __restrict__ xa, int S, int W, SeqPos pos, int copies) {
    if (seq_done(pos)) return;
    const int r = blockIdx.x;
    const int64_t id = seq_len ? ids[*seq_len - S + r] : ids[r];
    const float p = (float)(seq_past(pos, S) + r);
    const bool ok = id >= 0 && id < vocab;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float pe = 0.f;
        if (inv_freq) {
            const float ang = p * inv_freq[c >> 1];
            pe = (c & 1) ? cosf(ang) : sinf(ang);
        }
        const float v = (ok ? ldf(table + (size_t)id * W + c) * scale : 0.f) + pe;
        for (int k = 0; k < copies; ++k) x32[((size_t)r * copies + k) * W + c] = v;
        if (xa) stf(xa + (size_t)r * W + c, v);
    }
}

// One CTA per row. Rows of up to 256 * kRowCache elements are read once into registers (E per thread, every load in flight
// together); wider rows (E = 0) are re-read from L1/L2 in each of the three passes. Every form adds in the same order.
constexpr int kRowCache = 16;
template <typename T, int E>
__global__ void __launch_bounds__(256) postnorm_residual_kernel(float* __restrict__ x32, T* __restrict__ xa, const T* __restrict__ a,
                                                                int ld_a, const float* __restrict__ wa, const T* __restrict__ b,
                                                                int ld_b, const float* __restrict__ wb, const float* __restrict__ w,
                                                                float alpha, float eps, int W) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    float* x = x32 + (size_t)r * W;
    const T* ar = a + (size_t)r * ld_a;
    const T* br = b ? b + (size_t)r * ld_b : nullptr;
    constexpr bool CACHE = E > 0;
    constexpr int EN = E > 0 ? E : 1;
    float va[EN], vb[EN], vx[EN];
    if (CACHE) {
#pragma unroll
        for (int i = 0; i < EN; ++i) {
            const int c = threadIdx.x + i * 256;
            va[i] = c < W ? ldf(ar + c) : 0.f;
            vb[i] = (br && c < W) ? ldf(br + c) : 0.f;
            vx[i] = c < W ? x[c] : 0.f;
        }
    }
    float ra = 1.f, rb = 1.f;
    if (br) {
        float sa = 0.f, sb = 0.f;
        if (CACHE) {
#pragma unroll
            for (int i = 0; i < EN; ++i) { sa = fmaf(va[i], va[i], sa); sb = fmaf(vb[i], vb[i], sb); }
        } else {
            for (int c = threadIdx.x; c < W; c += blockDim.x) {
                const float ta = ldf(ar + c), tb = ldf(br + c);
                sa = fmaf(ta, ta, sa);
                sb = fmaf(tb, tb, sb);
            }
        }
        sa = block_sum(sa, red);
        sb = block_sum(sb, red);
        ra = 1.f / sqrtf(sa / (float)W + eps);
        rb = 1.f / sqrtf(sb / (float)W + eps);
    }
    float ss = 0.f;
    if (CACHE) {
#pragma unroll
        for (int i = 0; i < EN; ++i) {
            const int c = threadIdx.x + i * 256;
            if (c < W) {
                const float m = br ? 0.5f * (va[i] * ra * wa[c] + vb[i] * rb * wb[c]) : va[i];
                vx[i] = fmaf(alpha, vx[i], m);
                ss = fmaf(vx[i], vx[i], ss);
            }
        }
    } else {
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            const float m = br ? 0.5f * (ldf(ar + c) * ra * wa[c] + ldf(br + c) * rb * wb[c]) : ldf(ar + c);
            const float v = fmaf(alpha, x[c], m);
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    const float rn = 1.f / sqrtf(ss / (float)W + eps);
    if (CACHE) {
#pragma unroll
        for (int i = 0; i < EN; ++i) {
            const int c = threadIdx.x + i * 256;
            if (c < W) {
                const float v = vx[i] * rn * w[c];
                x[c] = v;
                stf(xa + (size_t)r * W + c, v);
            }
        }
    } else {
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            const float m = br ? 0.5f * (ldf(ar + c) * ra * wa[c] + ldf(br + c) * rb * wb[c]) : ldf(ar + c);
            const float v = fmaf(alpha, x[c], m) * rn * w[c];
            x[c] = v;
            stf(xa + (size_t)r * W + c, v);
        }
    }
}

// A team of TEAM threads (a warp, or a whole CTA for groups wider than 128 columns) per (row, group). Groups of up to
// TEAM * kRowCache columns are read once into registers (E per thread); wider ones (E = 0) are re-read in the second pass.
template <typename T, int TEAM, int E>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* __restrict__ y, int ld_y, const T* __restrict__ gate,
                                                               int ld_gate, const float* __restrict__ w, int w_len, T* __restrict__ out,
                                                               int ld_out, int S, int n, int group, int gate_first, float eps) {
    __shared__ float red[32];
    const int ngroups = n / group;
    const int wid = TEAM == 32 ? blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
    const int lane = TEAM == 32 ? (threadIdx.x & 31) : threadIdx.x;
    if (wid >= S * ngroups) return;
    const int r = wid / ngroups, c0 = (wid % ngroups) * group;
    const int wb = c0 % w_len;                 // weight index of the group's first column (one division per team)
    const float* yr = y + (size_t)r * ld_y + c0;
    const T* gr = gate + (size_t)r * ld_gate + c0;
    constexpr bool CACHE = E > 0;
    constexpr int EN = E > 0 ? E : 1;
    float vy[EN], vg[EN];
    float ss = 0.f;
    if (CACHE) {
#pragma unroll
        for (int i = 0; i < EN; ++i) {
            const int c = lane + i * TEAM;
            vy[i] = c < group ? yr[c] : 0.f;
            vg[i] = c < group ? ldf(gr + c) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < EN; ++i) {
            vg[i] = gate_first == 2 ? sigmoid_f(vg[i]) : silu_f(vg[i]);
            const float v = gate_first == 1 ? vy[i] * vg[i] : vy[i];
            ss = fmaf(v, v, ss);
        }
    } else {
        for (int c = lane; c < group; c += TEAM) {
            const float v = gate_first == 1 ? yr[c] * silu_f(ldf(gr + c)) : yr[c];
            ss = fmaf(v, v, ss);
        }
    }
    ss = TEAM == 32 ? warp_sum(ss) : block_sum(ss, red);
    const float rn = 1.f / sqrtf(ss / (float)group + eps);
    if (CACHE) {
#pragma unroll
        for (int i = 0; i < EN; ++i) {
            const int c = lane + i * TEAM;
            if (c < group) {
                const int wi = wb + c;
                const float wv = w[wi < w_len ? wi : wi % w_len];
                stf(out + (size_t)r * ld_out + c0 + c, gate_first == 1 ? vy[i] * vg[i] * rn * wv : vy[i] * rn * wv * vg[i]);
            }
        }
    } else {
        for (int c = lane; c < group; c += TEAM) {
            const float gsl = gate_first == 2 ? sigmoid_f(ldf(gr + c)) : silu_f(ldf(gr + c));
            const int wi = wb + c;
            const float wv = w[wi < w_len ? wi : wi % w_len];
            const float v = gate_first == 1 ? yr[c] * gsl * rn * wv : yr[c] * rn * wv * gsl;
            stf(out + (size_t)r * ld_out + c0 + c, v);
        }
    }
}

template <typename T>
__global__ void glu_gelu_tanh_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int ld_out, int S, int F) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)S * F) return;
    const int r = (int)(i / F), c = (int)(i % F);
    const float z = ldf(gu + (size_t)r * ld + c), u = ldf(gu + (size_t)r * ld + F + c);
    const float act = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    stf(out + (size_t)r * ld_out + c, act * u);
}

template <typename T>
__global__ void __launch_bounds__(256) gather_rmsnorm_kernel(const float* __restrict__ x32, const int* __restrict__ rows,
                                                             const float* __restrict__ w, float eps, T* __restrict__ out, int W) {
    __shared__ float red[32];
    const int i = blockIdx.x;
    const float* x = x32 + (size_t)rows[i] * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(x[c], x[c], ss);
    ss = block_sum(ss, red);
    const float rn = 1.f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) stf(out + (size_t)i * W + c, x[c] * rn * w[c]);
}

// out[r, :n] = rms(in[r, :n]) * w: one CTA per row of a slice in the storage type
template <typename T>
__global__ void __launch_bounds__(128) slice_rmsnorm_kernel(const T* __restrict__ in, int ld_in, const float* __restrict__ w, float eps,
                                                            T* __restrict__ out, int ld_out, int n) {
    __shared__ float red[32];
    const T* x = in + (size_t)blockIdx.x * ld_in;
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) { const float v = ldf(x + c); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float rn = 1.f / sqrtf(ss / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) stf(out + (size_t)blockIdx.x * ld_out + c, ldf(x + c) * rn * w[c]);
}

__global__ void softcap_kernel(float* __restrict__ x, int64_t n, float cap, float inv_cap, float scale) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = (cap > 0.f ? cap * tanhf(x[i] * inv_cap) : x[i]) * scale;
}

__device__ __forceinline__ float norm_apply(const NormSpec& n, float v, float rn, int c) {
    return n.kind == NORM_DYT ? fmaf(tanhf(n.alpha * v), n.w[c], n.b[c]) : v * rn * n.w[c];
}

template <typename T>
__global__ void __launch_bounds__(256) gather_norm_kernel(const float* __restrict__ x32, const int* __restrict__ rows, NormSpec n,
                                                          T* __restrict__ out, int W) {
    __shared__ float red[32];
    const int i = blockIdx.x;
    const float* x = x32 + (size_t)rows[i] * W;
    float rn = 1.f;
    if (n.kind == NORM_RMS) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(x[c], x[c], ss);
        ss = block_sum(ss, red);
        rn = 1.f / sqrtf(ss / (float)W + n.eps);
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) stf(out + (size_t)i * W + c, norm_apply(n, x[c], rn, c));
}

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
template <typename T> __device__ __forceinline__ void st4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void st4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void st4<bf16>(bf16* p, const float (&v)[4]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
}

// One CTA per row: pass 1 forms the new residual row (every addend read, also a row of xa that pass 2 rewrites) and, for a
// norm with a row statistic, its sum of squares; pass 2 writes the normed row. The places and weights of a routed row's
// choices are read once into shared memory, so that the expert rows' loads do not wait on them one by one. VEC: four
// columns per thread and step (every row start 16-byte aligned in fp32, 8-byte in bf16). Each column's sum is formed in the
// same order in both forms and does not depend on S.
constexpr int kCombineTop = 32;
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) residual_norm_kernel(float* __restrict__ x32, const T* __restrict__ a, int ld_a,
                                                            const T* __restrict__ b, int ld_b, bool has_mc, MoeCombine mc, NormSpec n,
                                                            T* __restrict__ xa, int W) {
    __shared__ float red[32];
    __shared__ int spos[kCombineTop];
    __shared__ float swt[kCombineTop];
    const int r = blockIdx.x;
    float* x = x32 + (size_t)r * W;
    float ss = 0.f;
    constexpr int V = VEC ? 4 : 1;
    if (a || b || has_mc) {
        const int top = has_mc ? mc.top : 0;
        const bool cached = top <= kCombineTop;
        if (has_mc && cached) {
            if (threadIdx.x < top) {
                spos[threadIdx.x] = mc.pos[(size_t)r * top + threadIdx.x];
                swt[threadIdx.x] = mc.weight[(size_t)r * top + threadIdx.x];
            }
            __syncthreads();
        }
        const float gs = (has_mc && mc.so) ? mc.gate[r] : 0.f;
        for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
            float y[V], t[V];
#pragma unroll
            for (int i = 0; i < V; ++i) y[i] = 0.f;
            if (has_mc) {
                for (int k = 0; k < top; ++k) {
                    const int p = cached ? spos[k] : mc.pos[(size_t)r * top + k];
                    if (p < 0) continue;
                    const float wk = cached ? swt[k] : mc.weight[(size_t)r * top + k];
                    const T* src = (const T*)mc.eo + (size_t)p * mc.ld_eo + c;
                    if (VEC) ld4(src, (float(&)[4])t); else t[0] = ldf(src);
#pragma unroll
                    for (int i = 0; i < V; ++i) y[i] = fmaf(wk, t[i], y[i]);
                }
                if (mc.so) {
                    const T* src = (const T*)mc.so + (size_t)r * mc.ld_so + c;
                    if (VEC) ld4(src, (float(&)[4])t); else t[0] = ldf(src);
#pragma unroll
                    for (int i = 0; i < V; ++i) y[i] = fmaf(gs, t[i], y[i]);
                }
            } else if (b) {
                const T* src = b + (size_t)r * ld_b + c;
                if (VEC) ld4(src, (float(&)[4])y); else y[0] = ldf(src);
            }
            if (a) {
                const T* src = a + (size_t)r * ld_a + c;
                if (VEC) ld4(src, (float(&)[4])t); else t[0] = ldf(src);
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] += t[i];       // the mixer's row + the feed-forward's row
            }
            float v[V];
            if (VEC) ld4(x + c, (float(&)[4])v); else v[0] = x[c];
#pragma unroll
            for (int i = 0; i < V; ++i) { v[i] += y[i]; ss = fmaf(v[i], v[i], ss); }
            if (VEC) st4(x + c, (const float(&)[4])v); else x[c] = v[0];
        }
    } else if (n.w && n.kind == NORM_RMS) {
        for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(x[c], x[c], ss);
    }
    if (!n.w) return;
    float rn = 1.f;
    if (n.kind == NORM_RMS) {
        ss = block_sum(ss, red);
        rn = 1.f / sqrtf(ss / (float)W + n.eps);
    }
    // (a thread rewrites in xa only the columns it read in pass 1: an xa row that served as an addend is safe)
    for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
        float v[V];
        if (VEC) ld4(x + c, (float(&)[4])v); else v[0] = x[c];
#pragma unroll
        for (int i = 0; i < V; ++i) v[i] = norm_apply(n, v[i], rn, c + i);
        if (VEC) st4(xa + (size_t)r * W + c, (const float(&)[4])v); else stf(xa + (size_t)r * W + c, v[0]);
    }
}

template <typename T>
__global__ void glu_clamp_swish_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int ld_out, int S, int F, float limit, bool il16,
                                       float alpha, float up_bias) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)S * F) return;
    const int r = (int)(i / F), c = (int)(i % F);
    const int gc = il16 ? ((c >> 4) << 5) + (c & 15) : c, uc = il16 ? gc + 16 : F + c;
    const float g = fminf(ldf(gu + (size_t)r * ld + gc), limit);
    const float u = fminf(fmaxf(ldf(gu + (size_t)r * ld + uc), -limit), limit);
    stf(out + (size_t)r * ld_out + c, g / (1.f + expf(-alpha * g)) * (u + up_bias));
}

// x <- x + rms(y) * w for one row per CTA, y = the sublayer's row or the routed feed-forward's weighted sum of expert rows. A
// thread keeps its E pieces of y in registers between the sum of squares and the update (E = 0: rows wider than 256 * 16
// pieces form y twice); a piece is one column, or with VEC four neighbouring ones (one 16-byte / 8-byte access). Each
// column's sum runs in the same order in both forms and for every S.
template <typename T, int E, bool VEC>
__global__ void __launch_bounds__(256) branch_norm_residual_kernel(float* __restrict__ x32, const T* __restrict__ a, int ld_a, bool has_mc,
                                                                   MoeCombine mc, const float* __restrict__ w, float eps,
                                                                   T* __restrict__ xa, int W) {
    __shared__ float red[32];
    __shared__ int spos[kCombineTop];
    __shared__ float swt[kCombineTop];
    constexpr int V = VEC ? 4 : 1;
    const int r = blockIdx.x;
    float* x = x32 + (size_t)r * W;
    const int top = has_mc ? mc.top : 0;
    const bool cached = top <= kCombineTop;
    if (has_mc && cached) {
        if (threadIdx.x < top) {
            spos[threadIdx.x] = mc.pos[(size_t)r * top + threadIdx.x];
            swt[threadIdx.x] = mc.weight[(size_t)r * top + threadIdx.x];
        }
        __syncthreads();
    }
    const float gs = (has_mc && mc.so) ? mc.gate[r] : 0.f;
    auto value = [&](int c, float (&y)[V]) {
        float t[V];
        if (!has_mc) {
            if (VEC) ld4(a + (size_t)r * ld_a + c, (float(&)[4])y); else y[0] = ldf(a + (size_t)r * ld_a + c);
            return;
        }
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = cached ? spos[k] : mc.pos[(size_t)r * top + k];
            if (p < 0) continue;
            const float wk = cached ? swt[k] : mc.weight[(size_t)r * top + k];
            const T* src = (const T*)mc.eo + (size_t)p * mc.ld_eo + c;
            if (VEC) ld4(src, (float(&)[4])t); else t[0] = ldf(src);
#pragma unroll
            for (int i = 0; i < V; ++i) y[i] = fmaf(wk, t[i], y[i]);
        }
        if (mc.so) {
            const T* src = (const T*)mc.so + (size_t)r * mc.ld_so + c;
            if (VEC) ld4(src, (float(&)[4])t); else t[0] = ldf(src);
#pragma unroll
            for (int i = 0; i < V; ++i) y[i] = fmaf(gs, t[i], y[i]);
        }
    };
    auto update = [&](int c, const float (&y)[V], float rn) {
        float v[V];
        if (VEC) ld4(x + c, (float(&)[4])v); else v[0] = x[c];
#pragma unroll
        for (int i = 0; i < V; ++i) v[i] = fmaf(y[i] * rn, w[c + i], v[i]);
        if (VEC) st4(x + c, (const float(&)[4])v); else x[c] = v[0];
        if (xa) { if (VEC) st4(xa + (size_t)r * W + c, (const float(&)[4])v); else stf(xa + (size_t)r * W + c, v[0]); }
    };
    constexpr int EN = E > 0 ? E : 1;
    float vy[EN][V];
    float ss = 0.f;
    if (E > 0) {
#pragma unroll
        for (int i = 0; i < EN; ++i) {
            const int c = (threadIdx.x + i * 256) * V;
#pragma unroll
            for (int u = 0; u < V; ++u) vy[i][u] = 0.f;
            if (c < W) value(c, vy[i]);
#pragma unroll
            for (int u = 0; u < V; ++u) ss = fmaf(vy[i][u], vy[i][u], ss);
        }
    } else {
        for (int c = threadIdx.x * V; c < W; c += 256 * V) {
            float y[V];
            value(c, y);
#pragma unroll
            for (int u = 0; u < V; ++u) ss = fmaf(y[u], y[u], ss);
        }
    }
    ss = block_sum(ss, red);
    const float rn = 1.f / sqrtf(ss / (float)W + eps);
    if (E > 0) {
#pragma unroll
        for (int i = 0; i < EN; ++i) {
            const int c = (threadIdx.x + i * 256) * V;
            if (c < W) update(c, vy[i], rn);
        }
    } else {
        for (int c = threadIdx.x * V; c < W; c += 256 * V) {
            float y[V];
            value(c, y);
            update(c, y, rn);
        }
    }
}

inline int done() { return cudaGetLastError() == cudaSuccess ? 0 : -100; }

}  // namespace

int embed_sinusoid(int dt, const int64_t* ids, const int* seq_len, const void* table, int64_t vocab, float scale,
                   const float* inv_freq, float* x32, void* xa, int S, int W, SeqPos pos, cudaStream_t s, int copies) {
    if (!ids || !table || !x32 || S < 1 || W < 1 || copies < 1) return -2;
    count_launch();
    if (dt == DT_F32)
        embed_sinusoid_kernel<float><<<S, 256, 0, s>>>(ids, seq_len, (const float*)table, vocab, scale, inv_freq, x32, (float*)xa, S, W, pos, copies);
    else
        embed_sinusoid_kernel<bf16><<<S, 256, 0, s>>>(ids, seq_len, (const bf16*)table, vocab, scale, inv_freq, x32, (bf16*)xa, S, W, pos, copies);
    return done();
}

int postnorm_residual(int dt, float* x32, void* xa, const void* a, int ld_a, const float* wa, const void* b, int ld_b,
                      const float* wb, const float* w, float alpha, float eps, int S, int W, cudaStream_t s) {
    if (!x32 || !xa || !a || !w || S < 1 || W < 1 || (b && (!wa || !wb))) return -2;
    count_launch();
#define LCC_PNR(E)                                                                                                          \
    do {                                                                                                                    \
        if (dt == DT_F32)                                                                                                   \
            postnorm_residual_kernel<float, E><<<S, 256, 0, s>>>(x32, (float*)xa, (const float*)a, ld_a, wa, (const float*)b, ld_b, wb, w, alpha, eps, W); \
        else                                                                                                                \
            postnorm_residual_kernel<bf16, E><<<S, 256, 0, s>>>(x32, (bf16*)xa, (const bf16*)a, ld_a, wa, (const bf16*)b, ld_b, wb, w, alpha, eps, W); \
    } while (0)
    const int per = (W + 255) / 256;
    if (per <= 2) LCC_PNR(2);
    else if (per <= 4) LCC_PNR(4);
    else if (per <= 8) LCC_PNR(8);
    else if (per <= kRowCache) LCC_PNR(16);
    else LCC_PNR(0);
#undef LCC_PNR
    return done();
}

int gated_group_norm(int dt, const float* y, int ld_y, const void* gate, int ld_gate, const float* w, int w_len,
                     void* out, int ld_out, int S, int n, int group, int gate_first, float eps, cudaStream_t s) {
    if (!y || !gate || !w || !out || S < 1 || n < 1 || group < 1 || n % group || w_len < 1) return -2;
    const int teams = S * (n / group);
    count_launch();
    // the team size depends on the group's width alone, so a row is summed in the same order in every batch and portion
#define LCC_GGN(TEAM, E, GRID)                                                                                            \
    do {                                                                                                                  \
        if (dt == DT_F32)                                                                                                 \
            gated_group_norm_kernel<float, TEAM, E><<<GRID, 256, 0, s>>>(y, ld_y, (const float*)gate, ld_gate, w, w_len, (float*)out, \
                                                                         ld_out, S, n, group, gate_first, eps);           \
        else                                                                                                              \
            gated_group_norm_kernel<bf16, TEAM, E><<<GRID, 256, 0, s>>>(y, ld_y, (const bf16*)gate, ld_gate, w, w_len, (bf16*)out,    \
                                                                        ld_out, S, n, group, gate_first, eps);            \
    } while (0)
    if (group <= 128) {
        LCC_GGN(32, 4, (teams + 7) / 8);
    } else {
        const int per = (group + 255) / 256;
        if (per <= 1) LCC_GGN(256, 1, teams);
        else if (per <= 2) LCC_GGN(256, 2, teams);
        else if (per <= 4) LCC_GGN(256, 4, teams);
        else if (per <= 8) LCC_GGN(256, 8, teams);
        else if (per <= kRowCache) LCC_GGN(256, 16, teams);
        else LCC_GGN(256, 0, teams);
    }
#undef LCC_GGN
    return done();
}

int glu_gelu_tanh(int dt, const void* gu, int ld, void* out, int ld_out, int S, int F, cudaStream_t s) {
    if (!gu || !out || S < 1 || F < 1) return -2;
    const int64_t n = (int64_t)S * F;
    count_launch();
    if (dt == DT_F32)
        glu_gelu_tanh_kernel<float><<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const float*)gu, ld, (float*)out, ld_out, S, F);
    else
        glu_gelu_tanh_kernel<bf16><<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const bf16*)gu, ld, (bf16*)out, ld_out, S, F);
    return done();
}

int gather_rmsnorm(int dt, const float* x32, const int* rows, const float* w, float eps, void* out, int n_rows, int W,
                   cudaStream_t s) {
    if (!x32 || !rows || !w || !out || n_rows < 1 || W < 1) return -2;
    count_launch();
    if (dt == DT_F32)
        gather_rmsnorm_kernel<float><<<n_rows, 256, 0, s>>>(x32, rows, w, eps, (float*)out, W);
    else
        gather_rmsnorm_kernel<bf16><<<n_rows, 256, 0, s>>>(x32, rows, w, eps, (bf16*)out, W);
    return done();
}

int slice_rmsnorm(int dt, const void* in, int ld_in, const float* w, float eps, void* out, int ld_out, int S, int n, cudaStream_t s) {
    if (!in || !w || !out || S < 1 || n < 1 || ld_in < n || ld_out < n) return -2;
    count_launch();
    if (dt == DT_F32)
        slice_rmsnorm_kernel<float><<<S, 128, 0, s>>>((const float*)in, ld_in, w, eps, (float*)out, ld_out, n);
    else
        slice_rmsnorm_kernel<bf16><<<S, 128, 0, s>>>((const bf16*)in, ld_in, w, eps, (bf16*)out, ld_out, n);
    return done();
}

int softcap(float* x, int64_t n, float cap, cudaStream_t s, float scale) {
    if (!x || n < 1) return -2;
    if (!(cap > 0.f) && scale == 1.f) return 0;
    count_launch();
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, n, cap > 0.f ? cap : 0.f, cap > 0.f ? 1.f / cap : 0.f, scale);
    return done();
}

int gather_norm(int dt, const float* x32, const int* rows, const NormSpec& n, void* out, int n_rows, int W, cudaStream_t s) {
    if (!x32 || !rows || !n.w || !out || n_rows < 1 || W < 1 || (n.kind == NORM_DYT && !n.b) || (n.kind != NORM_DYT && n.kind != NORM_RMS))
        return -2;
    count_launch();
    if (dt == DT_F32)
        gather_norm_kernel<float><<<n_rows, 256, 0, s>>>(x32, rows, n, (float*)out, W);
    else
        gather_norm_kernel<bf16><<<n_rows, 256, 0, s>>>(x32, rows, n, (bf16*)out, W);
    return done();
}

int residual_norm(int dt, float* x32, const void* a, int ld_a, const void* b, int ld_b, const MoeCombine* mc, const NormSpec& next,
                  void* xa, int S, int W, cudaStream_t s) {
    if (!x32 || S < 1 || W < 1 || (next.w && !xa) || (next.w && next.kind == NORM_DYT && !next.b) ||
        (next.kind != NORM_DYT && next.kind != NORM_RMS) || (mc && b))
        return -2;
    if (mc && (!mc->eo || !mc->pos || !mc->weight || mc->top < 1 || (mc->so && !mc->gate))) return -2;
    if (!a && !b && !mc && !next.w) return 0;
    count_launch();
    const MoeCombine m = mc ? *mc : MoeCombine{};
    const size_t es = dt == DT_F32 ? 4 : 2;
    auto ok4 = [&](const void* p, int ld) { return !p || ((ld % 4) == 0 && ((uintptr_t)p % (4 * es)) == 0); };
    const bool vec = (W % 4) == 0 && ((uintptr_t)x32 % 16) == 0 && ok4(a, ld_a) && ok4(b, ld_b) && ok4(xa, W) &&
                     (!mc || (ok4(m.eo, m.ld_eo) && ok4(m.so, m.ld_so)));
#define LCC_RN(T, VECB)                                                                                                      \
    residual_norm_kernel<T, VECB><<<S, 256, 0, s>>>(x32, (const T*)a, ld_a, (const T*)b, ld_b, mc != nullptr, m, next, (T*)xa, W)
    if (dt == DT_F32) { if (vec) LCC_RN(float, true); else LCC_RN(float, false); }
    else { if (vec) LCC_RN(bf16, true); else LCC_RN(bf16, false); }
#undef LCC_RN
    return done();
}

int branch_norm_residual(int dt, float* x32, const void* a, int ld_a, const MoeCombine* mc, const float* w, float eps, void* xa,
                         int S, int W, cudaStream_t s) {
    if (!x32 || !w || S < 1 || W < 1 || (!a && !mc) || (a && mc)) return -2;
    if (mc && (!mc->eo || !mc->pos || !mc->weight || mc->top < 1 || (mc->so && !mc->gate))) return -2;
    count_launch();
    const MoeCombine m = mc ? *mc : MoeCombine{};
    const size_t es = dt == DT_F32 ? 4 : 2;
    auto ok4 = [&](const void* p, int ld) { return !p || ((ld % 4) == 0 && ((uintptr_t)p % (4 * es)) == 0); };
    const bool vec = (W % 4) == 0 && ((uintptr_t)x32 % 16) == 0 && ((uintptr_t)w % 16) == 0 && ok4(a, ld_a) && ok4(xa, W) &&
                     (!mc || (ok4(m.eo, m.ld_eo) && ok4(m.so, m.ld_so)));
#define LCC_BNR2(E, VECB)                                                                                                      \
    do {                                                                                                                       \
        if (dt == DT_F32) branch_norm_residual_kernel<float, E, VECB><<<S, 256, 0, s>>>(x32, (const float*)a, ld_a, mc != nullptr, m, w, eps, (float*)xa, W); \
        else branch_norm_residual_kernel<bf16, E, VECB><<<S, 256, 0, s>>>(x32, (const bf16*)a, ld_a, mc != nullptr, m, w, eps, (bf16*)xa, W);                 \
    } while (0)
#define LCC_BNR(E) do { if (vec) LCC_BNR2(E, true); else LCC_BNR2(E, false); } while (0)
    const int per = (W / (vec ? 4 : 1) + 255) / 256;      // pieces per thread: the form depends on the row's width alone
    if (per <= 1) LCC_BNR(1);
    else if (per <= 2) LCC_BNR(2);
    else if (per <= 4) LCC_BNR(4);
    else if (per <= 8) LCC_BNR(8);
    else if (per <= kRowCache) LCC_BNR(16);
    else LCC_BNR(0);
#undef LCC_BNR
#undef LCC_BNR2
    return done();
}

int glu_clamp_swish(int dt, const void* gu, int ld, void* out, int ld_out, int S, int F, float limit, cudaStream_t s, bool il16,
                    float alpha, float up_bias) {
    if (!gu || !out || S < 1 || F < 1 || (il16 && (F % 16))) return -2;
    const int64_t n = (int64_t)S * F;
    count_launch();
    if (dt == DT_F32)
        glu_clamp_swish_kernel<float><<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const float*)gu, ld, (float*)out, ld_out, S, F, limit, il16, alpha, up_bias);
    else
        glu_clamp_swish_kernel<bf16><<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const bf16*)gu, ld, (bf16*)out, ld_out, S, F, limit, il16, alpha, up_bias);
    return done();
}

}  // namespace lcc
