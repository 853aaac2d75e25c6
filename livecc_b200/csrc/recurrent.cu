// Recurrent sequence mixers with state carried from call to call (prefill portions and decode steps run the same
// kernels): the short causal convolution of a state-space layer, its step sizes and decays, the per-channel decays of
// gated linear attention, the gated linear recurrence both share:
//     St <- diag(a_t) St + k_t (sc_t u_t)^T ,  y_t = St^T c_t + skip * u_t          (St: N x P per head, fp32)
// and the gated delta rule (a decay per key channel, then the write beta (v - St^T k) under the key k).
// Everything that enters the recurrence is fp32; the projections it reads are in the model's storage type.
#include <math.h>
#include <stdlib.h>

#include <algorithm>

#include "../../include/livecc_b200.h"
#include "common.cuh"
#include "mma.cuh"
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

__device__ __forceinline__ bool seq_done(const SeqPos& p) { return p.finished && *p.finished; }

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

// ---- causal convolution -----------------------------------------------------------------------------------------------
constexpr int kMaxTaps = 8;

// out[t, c] = silu(b[c] + sum_j w[c, j] * in[t - (taps-1) + j, c]); rows before 0 come from the carry. A thread owns one
// channel over kConvRows consecutive rows and slides the window through registers, so every input is read once. When the
// call has no more than kConvRows rows (a decode step), the same thread also writes the channel's new carry (carry_out),
// which it alone reads and writes; longer calls update the carry in a second launch, after every block has read it.
// TI / T: the input's and the output's element types (an fp32 residual stream may feed an output in the storage type); SILU: the
// activation; ADD: out = in + conv(in). b may be null.
constexpr int kConvRows = 8;
template <typename TI, typename T, bool SILU, bool ADD>
__global__ void causal_conv_kernel(const TI* __restrict__ in, int ld_in, T* __restrict__ out, int ld_out,
                                   const float* __restrict__ w, const float* __restrict__ b,
                                   const float* carry, float* carry_out, int S, int C, int taps, SeqPos pos) {
    if (seq_done(pos)) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t0 = blockIdx.y * kConvRows;
    if (c >= C) return;
    float wv[kMaxTaps], x[kMaxTaps + kConvRows - 1];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) wv[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
    // x[i] = input at row t0 - (taps-1) + i
#pragma unroll
    for (int i = 0; i < kMaxTaps + kConvRows - 1; ++i) {
        const int tt = t0 - (taps - 1) + i;
        float v = 0.f;
        if (i < taps - 1 + kConvRows && tt < S) v = tt >= 0 ? ldf(in + (size_t)tt * ld_in + c) : carry[(size_t)c * (taps - 1) + (taps - 1 + tt)];
        x[i] = v;
    }
    const float bias = b ? b[c] : 0.f;
#pragma unroll
    for (int r = 0; r < kConvRows; ++r) {
        float acc = bias;
#pragma unroll
        for (int j = 0; j < kMaxTaps; ++j)
            if (j < taps) acc = fmaf(wv[j], x[r + j], acc);
        if (ADD) {   // x[r + taps - 1] is the row's own input
            float own = 0.f;
#pragma unroll
            for (int j = 0; j < kMaxTaps; ++j)
                if (j == taps - 1) own = x[r + j];
            acc += own;
        }
        if (t0 + r < S) stf(out + (size_t)(t0 + r) * ld_out + c, SILU ? silu_f(acc) : acc);
    }
    if (carry_out) {
        // new carry[i] = input at row S - (taps-1) + i; an older carry entry when that row is negative: entry S + i, which lies
        // above every entry written so far (i ascending), so the update can run in place
        const int n = taps - 1;
        for (int i = 0; i < n; ++i) {
            const int tt = S - n + i;
            carry_out[(size_t)c * n + i] = tt >= 0 ? ldf(in + (size_t)tt * ld_in + c) : carry[(size_t)c * n + (n + tt)];
        }
    }
}

// carry[c, i] <- input at row S - (taps-1) + i (an older carry entry when that row is negative)
template <typename T>
__global__ void conv_carry_update_kernel(const T* __restrict__ in, int ld_in, float* __restrict__ carry, int S, int C,
                                         int taps, SeqPos pos) {
    if (seq_done(pos)) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int n = taps - 1;
    float nv[kMaxTaps];
    for (int i = 0; i < n; ++i) {
        const int tt = S - n + i;
        nv[i] = tt >= 0 ? ldf(in + (size_t)tt * ld_in + c) : carry[(size_t)c * n + (n + tt)];
    }
    for (int i = 0; i < n; ++i) carry[(size_t)c * n + i] = nv[i];
}

// ---- step sizes and decays ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void ssm_step_decay_kernel(const T* __restrict__ raw, int ld, const float* __restrict__ dt_bias,
                                      const float* __restrict__ a_log, float* __restrict__ dt_out,
                                      float* __restrict__ decay_out, int S, int heads) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= S * heads) return;
    const int t = i / heads, h = i % heads;
    const float dt = softplus_f(ldf(raw + (size_t)t * ld + h) + dt_bias[h]);
    dt_out[i] = dt;
    decay_out[i] = -expf(a_log[h]) * dt;
}

template <typename T>
__global__ void gla_decay_kernel(const T* __restrict__ z, int ld, const float* __restrict__ bias, float inv_tau,
                                 float* __restrict__ decay_out, int S, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= S * n) return;
    const int t = i / n, c = i % n;
    const float x = ldf(z + (size_t)t * ld + c) + (bias ? bias[c] : 0.f);
    // log(sigmoid(x)) = min(x, 0) - log1p(exp(-|x|)); the log decay is that over tau
    const float ls = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
    decay_out[i] = ls * inv_tau;
}

// ---- gated linear recurrence --------------------------------------------------------------------------------------------
// A thread keeps NT = 16 state entries St[n0..n0+15, p] of one value channel p in registers; JP (a power of two >= N / 16)
// neighbouring lanes share p and reduce y with shuffles. Tokens are staged through shared memory TT at a time so that the
// sequential loop over tokens reads only registers and shared memory and has no block barrier.
constexpr int NT = 16;
constexpr int TT = 16;
constexpr int kScanThreads = 128;

template <typename T, bool VEC>
__global__ void __launch_bounds__(kScanThreads) gated_scan_kernel(ScanArgs a, SeqPos pos) {
    if (seq_done(pos)) return;
    extern __shared__ float sm[];
    const int N = a.N, P = a.P, S = a.S;
    const int JP = blockDim.x;                 // lanes per value channel (x fastest: they sit in one warp)
    const int cols = blockDim.y;               // value channels per CTA
    const int h = blockIdx.x;
    const int col = threadIdx.y;
    const int p = blockIdx.y * cols + col;
    const int j = threadIdx.x;
    const int tid = threadIdx.y * JP + threadIdx.x, nthr = cols * JP;
    const int n0 = j * NT;
    const int g = h / a.heads_per_group;
    // shared: k[TT][N], c[TT][N], dec[TT][VEC ? N : 1], sc[TT], u[TT][cols]
    float* sk = sm;
    float* scv = sk + TT * N;
    float* sd = scv + TT * N;
    float* ssc = sd + TT * (VEC ? N : 1);
    float* su = ssc + TT;

    float st[NT];
    float* gstate = a.state + ((size_t)h * P + (p < P ? p : 0)) * N;
#pragma unroll
    for (int i = 0; i < NT; ++i) st[i] = (p < P && n0 + i < N) ? gstate[n0 + i] : 0.f;
    const float skip = a.skip ? a.skip[h] : 0.f;
    const T* gk = (const T*)a.k + (size_t)g * N;
    const T* gc = (const T*)a.c + (size_t)g * N;
    const T* gu = (const T*)a.u + (size_t)h * P + blockIdx.y * cols;

    for (int t0 = 0; t0 < S; t0 += TT) {
        const int nt = min(TT, S - t0);
        __syncthreads();
        for (int e = tid; e < nt * N; e += nthr) {
            const int t = e / N, n = e % N;
            sk[e] = ldf(gk + (size_t)(t0 + t) * a.ld_k + n);
            scv[e] = ldf(gc + (size_t)(t0 + t) * a.ld_c + n) * a.cs;
            if (VEC) sd[e] = expf(a.a[((size_t)(t0 + t) * a.heads + h) * N + n]);
        }
        for (int e = tid; e < nt; e += nthr) {
            if (!VEC) sd[e] = expf(a.a[(size_t)(t0 + e) * a.heads + h]);
            ssc[e] = a.sc ? a.sc[(size_t)(t0 + e) * a.heads + h] : 1.f;
        }
        for (int e = tid; e < nt * cols; e += nthr) {
            const int t = e / cols, c = e % cols;
            su[e] = (blockIdx.y * cols + c < P) ? ldf(gu + (size_t)(t0 + t) * a.ld_u + c) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float u = su[t * cols + col];
            const float su_t = ssc[t] * u;
            const float* kt = sk + t * N + n0;
            const float* ct = scv + t * N + n0;
            const float* dv = sd + (VEC ? t * N + n0 : t);
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                if (n0 + i < N) {
                    const float d = VEC ? dv[i] : dv[0];
                    st[i] = fmaf(d, st[i], kt[i] * su_t);
                    y = fmaf(st[i], ct[i], y);
                }
            }
            for (int o = JP >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);   // fixed butterfly order
            if (j == 0 && p < P) a.y[(size_t)(t0 + t) * a.ld_y + (size_t)h * P + p] = y + skip * u;
        }
    }
    if (p < P) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
            if (n0 + i < N) gstate[n0 + i] = st[i];
    }
}

// ---- delta rule ---------------------------------------------------------------------------------------------------------
// Everything the recurrence reads, prepared for all rows at once (one warp per (row, key head)) and laid out head by head, so
// that the operands of consecutive tokens of one head are contiguous: unit-length k and q (q also times q_scale) and their
// product k . q, the values as fp32, the decays exp(-exp(a_log[h]) * softplus(z + dt_bias)), and beta = sigmoid(b).
template <typename T>
__global__ void __launch_bounds__(128) delta_pack_kernel(DeltaPackArgs a) {
    const int wid = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (wid >= a.S * a.G) return;
    const int t = wid / a.G, g = wid % a.G, N = a.N, P = a.P, hpg = a.H / a.G;
    const size_t S = a.S;
    const DeltaOperands o = delta_operands(a.out, a.S, a.H, a.G, N, P);
    const T* row = (const T*)a.qkv + (size_t)t * a.ld;
    const T* qr = row + (size_t)g * N;
    const T* kr = row + a.col_k + (size_t)g * N;
    float sq = 0.f, sk = 0.f;
    for (int n = lane; n < N; n += 32) {
        const float q = ldf(qr + n), k = ldf(kr + n);
        sq = fmaf(q, q, sq); sk = fmaf(k, k, sk);
    }
    sq = warp_sum(sq); sk = warp_sum(sk);
    const float rq = (a.unit_eps > 0.f ? 1.f / sqrtf(sq + a.unit_eps) : 1.f) * a.q_scale;
    const float rk = a.unit_eps > 0.f ? 1.f / sqrtf(sk + a.unit_eps) : 1.f;
    float* ko = o.k + ((size_t)g * S + t) * N;
    float* qo = o.q + ((size_t)g * S + t) * N;
    float kq = 0.f;
    for (int n = lane; n < N; n += 32) {
        const float q = ldf(qr + n) * rq, k = ldf(kr + n) * rk;
        ko[n] = k;
        qo[n] = q;
        kq = fmaf(k, q, kq);
    }
    kq = warp_sum(kq);
    if (lane == 0) o.kq[(size_t)g * S + t] = kq;
    for (int h = g * hpg; h < (g + 1) * hpg; ++h) {
        const float rate = -expf(a.a_log[h]);
        const float* z = a.z + ((size_t)t * a.H + h) * N;
        float* d = a.dec + ((size_t)h * S + t) * N;
        for (int n = lane; n < N; n += 32) d[n] = expf(rate * softplus_f(z[n] + a.dt_bias[(size_t)h * N + n]));
        float* vo = o.v + ((size_t)h * S + t) * P;
        for (int p = lane; p < P; p += 32) vo[p] = ldf(row + a.col_v + (size_t)h * P + p);
        if (lane == 0) o.beta[(size_t)h * S + t] = 1.f / (1.f + expf(-ldf((const T*)a.b + (size_t)t * a.ld_b + h)));
    }
}

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}

// One state matrix per head; a thread keeps NT_ state entries of each of CPT value channels, JP lanes share those channels
// (lane j owns the 4-entry groups j, j + JP, ...: neighbouring lanes read neighbouring 16-byte pieces of shared memory). The
// prepared operands of TT tokens at a time are copied into one of two shared-memory buffers with cp.async while the tokens of
// the other buffer run, so the sequential loop reads only shared memory and registers; a thread's k, q and decay entries of
// a token are read once for its CPT channels (the kernel is bound by shared-memory reads: every channel needs the whole k, q
// and decay rows of every token). Per token: the state decays, the JP lanes reduce St^T k and St^T q together, the write
// w = beta (v - St^T k) lands, and the read-out is St^T q + (k . q) w: the same value as reading the state after the write,
// with one reduction pass instead of two. Shared rows are padded to JP * NT_ entries and the padding stays zero, so the inner
// loops need no bounds.
template <int NT_, int CPT>
__global__ void __launch_bounds__(kScanThreads) delta_scan_kernel(DeltaScanArgs a, SeqPos pos) {
    if (seq_done(pos)) return;
    extern __shared__ __align__(16) float sm[];
    const int N = a.N, P = a.P, S = a.S, TTn = a.TT;
    const int JP = blockDim.x, groups = blockDim.y, cols = groups * CPT;      // value channels per CTA
    const int h = blockIdx.x, j = threadIdx.x;
    const int p0 = blockIdx.y * cols, pc = threadIdx.y * CPT, p = p0 + pc;     // the thread's first channel
    const int tid = threadIdx.y * JP + threadIdx.x, nthr = groups * JP;
    const int NP = JP * NT_;
    const int g = h / (a.H / a.G);
    const DeltaOperands o = delta_operands(const_cast<float*>(a.ops), a.T, a.H, a.G, N, P);
    const float* gk = o.k + ((size_t)g * a.T + a.r0) * N;
    const float* gq = o.q + ((size_t)g * a.T + a.r0) * N;
    const float* gd = a.dec + ((size_t)h * a.T + a.r0) * N;
    const float* gv = o.v + ((size_t)h * a.T + a.r0) * P + p0;
    const float* gb = o.beta + (size_t)h * a.T + a.r0;
    const float* gkq = o.kq + (size_t)g * a.T + a.r0;
    // one buffer: k[TT][NP], q[TT][NP], d[TT][NP], u[TT][cols], beta[TT], kq[TT]
    const int buf_floats = TTn * (3 * NP + cols + 2);
    for (int e = tid; e < 2 * buf_floats; e += nthr) sm[e] = 0.f;
    __syncthreads();

    float2 st[CPT][NT_ / 2];          // entry i of the thread is key channel ((i / 4) * JP + j) * 4 + i % 4
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const float* gs = a.state + ((size_t)h * P + (p + c < P ? p + c : 0)) * N;
#pragma unroll
        for (int i = 0; i < NT_; ++i) {
            const int n = ((i >> 2) * JP + j) * 4 + (i & 3);
            const float v = (p + c < P && n < N) ? gs[n] : 0.f;
            if (i & 1) st[c][i >> 1].y = v; else st[c][i >> 1].x = v;
        }
    }

    auto fill = [&](int b, int t0) {
        float* sk = sm + b * buf_floats;
        float* sq = sk + TTn * NP;
        float* sd = sq + TTn * NP;
        float* su = sd + TTn * NP;
        float* sb = su + TTn * cols;
        float* skq = sb + TTn;
        const int nt = min(TTn, S - t0);
        if (a.async && NP == N) {               // whole rows: the stage's operands are three contiguous spans
            const float* ck = gk + (size_t)t0 * N;
            const float* cq = gq + (size_t)t0 * N;
            const float* cd = gd + (size_t)t0 * N;
            for (int e = tid * 4; e < nt * N; e += nthr * 4) {
                cp_async16(sk + e, ck + e, true);
                cp_async16(sq + e, cq + e, true);
                cp_async16(sd + e, cd + e, true);
            }
        } else if (a.async) {
            const int ch = N >> 2;
            for (int e = tid; e < nt * ch; e += nthr) {
                const int t = e / ch, c = (e % ch) << 2;
                cp_async16(sk + t * NP + c, gk + (size_t)(t0 + t) * N + c, true);
                cp_async16(sq + t * NP + c, gq + (size_t)(t0 + t) * N + c, true);
                cp_async16(sd + t * NP + c, gd + (size_t)(t0 + t) * N + c, true);
            }
        } else {
            for (int e = tid; e < nt * N; e += nthr) {
                const int t = e / N, n = e % N;
                sk[t * NP + n] = gk[(size_t)(t0 + t) * N + n];
                sq[t * NP + n] = gq[(size_t)(t0 + t) * N + n];
                sd[t * NP + n] = gd[(size_t)(t0 + t) * N + n];
            }
        }
        for (int e = tid; e < nt * cols; e += nthr) {
            const int t = e / cols, c = e % cols;
            if (p0 + c < P) cp_async4(su + e, gv + (size_t)(t0 + t) * P + c);
        }
        for (int t = tid; t < nt; t += nthr) {
            cp_async4(sb + t, gb + t0 + t);
            cp_async4(skq + t, gkq + t0 + t);
        }
        cp_async_commit();
    };

    fill(0, 0);
    int b = 0;
    for (int t0 = 0; t0 < S; t0 += TTn, b ^= 1) {
        cp_async_wait<0>();
        __syncthreads();            // buffer b is complete, and every thread has left buffer b ^ 1
        if (t0 + TTn < S) fill(b ^ 1, t0 + TTn);
        const float* sk = sm + b * buf_floats;
        const float* sq = sk + TTn * NP;
        const float* sd = sq + TTn * NP;
        const float* su = sd + TTn * NP + pc;
        const float* sb = sd + TTn * NP + TTn * cols;
        const float* skq = sb + TTn;
        const int nt = min(TTn, S - t0);
        float* yo = a.y + (size_t)t0 * a.ld_y + (size_t)h * P + p;
#pragma unroll 2
        for (int t = 0; t < nt; ++t) {
            const float4* k4 = reinterpret_cast<const float4*>(sk + t * NP) + j;
            const float4* q4 = reinterpret_cast<const float4*>(sq + t * NP) + j;
            const float4* d4 = reinterpret_cast<const float4*>(sd + t * NP) + j;
            // packed fp32 pairs (fma.rn.f32x2: each half rounds as a scalar fma does): half the arithmetic instructions
            float2 kv[NT_ / 2];
            float2 ks[CPT], qs[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) ks[c] = qs[c] = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < NT_ / 4; ++i) {
                const float4 kk = k4[i * JP], qq = q4[i * JP], dd = d4[i * JP];
                kv[2 * i] = make_float2(kk.x, kk.y); kv[2 * i + 1] = make_float2(kk.z, kk.w);
                const float2 d0 = make_float2(dd.x, dd.y), d1 = make_float2(dd.z, dd.w);
                const float2 q0 = make_float2(qq.x, qq.y), q1 = make_float2(qq.z, qq.w);
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    st[c][2 * i] = __fmul2_rn(st[c][2 * i], d0);
                    st[c][2 * i + 1] = __fmul2_rn(st[c][2 * i + 1], d1);
                    ks[c] = __ffma2_rn(st[c][2 * i], kv[2 * i], ks[c]);
                    qs[c] = __ffma2_rn(st[c][2 * i], q0, qs[c]);
                    ks[c] = __ffma2_rn(st[c][2 * i + 1], kv[2 * i + 1], ks[c]);
                    qs[c] = __ffma2_rn(st[c][2 * i + 1], q1, qs[c]);
                }
            }
            float ksum[CPT], qsum[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) { ksum[c] = ks[c].x + ks[c].y; qsum[c] = qs[c].x + qs[c].y; }
            for (int o2 = JP >> 1; o2 > 0; o2 >>= 1) {          // fixed butterfly order
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    ksum[c] += __shfl_xor_sync(0xffffffffu, ksum[c], o2);
                    qsum[c] += __shfl_xor_sync(0xffffffffu, qsum[c], o2);
                }
            }
            const float beta = sb[t], kq = skq[t];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const float w = beta * (su[t * cols + c] - ksum[c]);
                const float2 w2 = make_float2(w, w);
#pragma unroll
                for (int i = 0; i < NT_ / 2; ++i) st[c][i] = __ffma2_rn(kv[i], w2, st[c][i]);
                if (j == 0 && p + c < P) yo[(size_t)t * a.ld_y + c] = fmaf(kq, w, qsum[c]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        if (p + c >= P) continue;
        float* gs = a.state + ((size_t)h * P + p + c) * N;
#pragma unroll
        for (int i = 0; i < NT_; ++i) {
            const int n = ((i >> 2) * JP + j) * 4 + (i & 3);
            if (n < N) gs[n] = (i & 1) ? st[c][i >> 1].y : st[c][i >> 1].x;
        }
    }
}

}  // namespace

int causal_conv(int dt, const void* in, int ld_in, void* out, int ld_out, const float* w, const float* b, float* carry,
                int S, int C, int taps, SeqPos pos, cudaStream_t s, const ConvOpts& opt) {
    if (!in || !out || !w || S < 1 || C < 1 || taps < 1 || taps > kMaxTaps || (taps > 1 && !carry)) return -2;
    dim3 grid((C + 127) / 128, (S + kConvRows - 1) / kConvRows);
    const bool fused = taps > 1 && S <= kConvRows;
    float* carry_out = fused ? carry : nullptr;
    const bool in32 = opt.in_f32 || dt == DT_F32;
    count_launch();
#define LCC_CONV(TI, T, SL, AD) causal_conv_kernel<TI, T, SL, AD><<<grid, 128, 0, s>>>((const TI*)in, ld_in, (T*)out, ld_out, w, b, carry, carry_out, S, C, taps, pos)
#define LCC_CONV2(TI, T)                                                            \
    do {                                                                            \
        if (opt.silu && !opt.add_input) LCC_CONV(TI, T, true, false);               \
        else if (!opt.silu && opt.add_input) LCC_CONV(TI, T, false, true);          \
        else if (opt.silu) LCC_CONV(TI, T, true, true);                             \
        else LCC_CONV(TI, T, false, false);                                         \
    } while (0)
    if (dt == DT_F32) LCC_CONV2(float, float);
    else if (in32) LCC_CONV2(float, bf16);
    else LCC_CONV2(bf16, bf16);
#undef LCC_CONV2
#undef LCC_CONV
    if (taps > 1 && !fused) {
        count_launch();
        if (in32)
            conv_carry_update_kernel<float><<<(C + 127) / 128, 128, 0, s>>>((const float*)in, ld_in, carry, S, C, taps, pos);
        else
            conv_carry_update_kernel<bf16><<<(C + 127) / 128, 128, 0, s>>>((const bf16*)in, ld_in, carry, S, C, taps, pos);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int delta_pack(int dt, const DeltaPackArgs& a, cudaStream_t s) {
    if (!a.qkv || !a.z || !a.dt_bias || !a.a_log || !a.b || !a.out || !a.dec || a.S < 1 || a.H < 1 || a.G < 1 || a.H % a.G || a.N < 1 ||
        a.P < 1)
        return -2;
    const int warps = a.S * a.G;
    count_launch();
    if (dt == DT_F32) delta_pack_kernel<float><<<(warps + 3) / 4, 128, 0, s>>>(a);
    else delta_pack_kernel<bf16><<<(warps + 3) / 4, 128, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int delta_scan(const DeltaScanArgs& q, SeqPos pos, cudaStream_t s) {
    if (!q.ops || !q.dec || !q.state || !q.y || q.S < 1 || q.T < q.S || q.r0 < 0 || q.r0 + q.S > q.T || q.H < 1 || q.G < 1 || q.H % q.G ||
        q.N < 1 || q.N > 512 || q.P < 1)
        return -2;
    DeltaScanArgs a = q;
    // state entries per thread and value channel: 8 (16 lanes per channel at 128 key channels), 16 beyond 256 key channels, 4
    // for narrow heads so that a channel still spreads over lanes
    static int forced = -1;
    if (forced < 0) { const char* e = getenv("LIVECC_B200_DELTA_NT"); forced = e ? atoi(e) : 0; }
    int nt = a.N > 256 ? 16 : (a.N > 16 ? 8 : 4);
    if ((forced == 4 || forced == 8 || forced == 16) && forced * 32 >= a.N) nt = forced;
    int JP = 1;
    while (JP * nt < a.N) JP *= 2;
    // value channels per thread: 2 with 8 state entries each when the head has 16 value channels or more (half the
    // shared-memory reads per channel; measured best at 128 x 128 heads: 8 x 2 250 us, 16 x 1 310, 8 x 1 320, 16 x 2 375,
    // 8 x 4 420 per 1024 tokens); lane groups per CTA: whole warps, 16 channels per CTA at most
    static int forced_cpt = -1;
    if (forced_cpt < 0) { const char* e = getenv("LIVECC_B200_DELTA_CPT"); forced_cpt = e ? atoi(e) : 0; }
    int cpt = (nt == 8 && a.P >= 16) ? 2 : 1;
    if (forced_cpt == 1 || forced_cpt == 2 || (forced_cpt == 4 && nt <= 8)) cpt = forced_cpt;
    int groups = std::max(kScanThreads / JP / cpt, 32 / JP);
    while (groups * JP > 32 && (groups / 2) * cpt >= a.P) groups /= 2;   // narrow heads: fewer idle lanes, but always whole warps
    const int cols = groups * cpt;
    const int NP = JP * nt;
    a.TT = 16;
    while (a.TT > 2 && (size_t)2 * a.TT * (3 * NP + cols + 2) * sizeof(float) > 64 * 1024) a.TT /= 2;
    // 16-byte copies need 16-byte aligned rows in every operand block (each block starts at a multiple of 4 floats)
    a.async = (a.N % 4) == 0 && ((uintptr_t)a.ops % 16) == 0 && ((uintptr_t)a.dec % 16) == 0;
    const size_t smem = (size_t)2 * a.TT * (3 * NP + cols + 2) * sizeof(float);
    dim3 block(JP, groups), grid(a.H, (a.P + cols - 1) / cols);
    count_launch();
#define LCC_DSCAN(NTV, CPTV)                                                                                                    \
    do {                                                                                                                        \
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<NTV, CPTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        delta_scan_kernel<NTV, CPTV><<<grid, block, smem, s>>>(a, pos);                                                         \
    } while (0)
    if (nt == 4) { if (cpt == 4) LCC_DSCAN(4, 4); else if (cpt == 2) LCC_DSCAN(4, 2); else LCC_DSCAN(4, 1); }
    else if (nt == 8) { if (cpt == 4) LCC_DSCAN(8, 4); else if (cpt == 2) LCC_DSCAN(8, 2); else LCC_DSCAN(8, 1); }
    else { if (cpt == 2) LCC_DSCAN(16, 2); else LCC_DSCAN(16, 1); }
#undef LCC_DSCAN
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int causal_conv_silu(int dt, const void* in, int ld_in, void* out, int ld_out, const float* w, const float* b,
                     float* carry, int S, int C, int taps, SeqPos pos, cudaStream_t s) {
    if (!b || !carry) return -2;
    return causal_conv(dt, in, ld_in, out, ld_out, w, b, carry, S, C, taps, pos, s, ConvOpts{false, true, false});
}

int ssm_step_decay(int dt, const void* raw, int ld, const float* dt_bias, const float* a_log, float* dt_out,
                   float* decay_out, int S, int heads, cudaStream_t s) {
    if (!raw || !dt_bias || !a_log || !dt_out || !decay_out || S < 1 || heads < 1) return -2;
    const int n = S * heads;
    count_launch();
    if (dt == DT_F32)
        ssm_step_decay_kernel<float><<<(n + 255) / 256, 256, 0, s>>>((const float*)raw, ld, dt_bias, a_log, dt_out, decay_out, S, heads);
    else
        ssm_step_decay_kernel<bf16><<<(n + 255) / 256, 256, 0, s>>>((const bf16*)raw, ld, dt_bias, a_log, dt_out, decay_out, S, heads);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int gla_decay(int dt, const void* z, int ld, const float* bias, float tau, float* decay_out, int S, int n,
              cudaStream_t s) {
    if (!z || !decay_out || S < 1 || n < 1 || !(tau > 0.f)) return -2;
    const int tot = S * n;
    count_launch();
    if (dt == DT_F32)
        gla_decay_kernel<float><<<(tot + 255) / 256, 256, 0, s>>>((const float*)z, ld, bias, 1.f / tau, decay_out, S, n);
    else
        gla_decay_kernel<bf16><<<(tot + 255) / 256, 256, 0, s>>>((const bf16*)z, ld, bias, 1.f / tau, decay_out, S, n);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int gated_scan(const ScanArgs& a, SeqPos pos, cudaStream_t s) {
    if (!a.k || !a.c || !a.u || !a.a || !a.state || !a.y || a.S < 1 || a.heads < 1 || a.N < 1 || a.P < 1 ||
        a.heads_per_group < 1)
        return -2;
    if (a.ws && a.S >= kScanChunkedMin && !pos.kv_len) return gated_scan_chunked(a, pos, s);
    int JP = 1;
    while (JP * NT < a.N) JP *= 2;
    if (JP > 32) return -3;  // N <= 512
    int cols = kScanThreads / JP;
    while (cols * JP > 32 && cols / 2 >= a.P) cols /= 2;   // narrow heads: fewer idle lanes, but always whole warps
    dim3 block(JP, cols), grid(a.heads, (a.P + cols - 1) / cols);
    const size_t smem = sizeof(float) * ((size_t)TT * a.N * 2 + (size_t)TT * (a.vec_decay ? a.N : 1) + TT +
                                         (size_t)TT * cols);
    if (smem > 200 * 1024) return -3;
    count_launch();
#define LCC_SCAN(T, V)                                                                                            \
    do {                                                                                                          \
        if (smem > 48 * 1024) cudaFuncSetAttribute(gated_scan_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        gated_scan_kernel<T, V><<<grid, block, smem, s>>>(a, pos);                                                \
    } while (0)
    if (a.dt == DT_F32) {
        if (a.vec_decay) LCC_SCAN(float, true); else LCC_SCAN(float, false);
    } else {
        if (a.vec_decay) LCC_SCAN(bf16, true); else LCC_SCAN(bf16, false);
    }
#undef LCC_SCAN
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace lcc
