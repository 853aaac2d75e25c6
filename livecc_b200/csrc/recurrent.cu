// Recurrent sequence mixers with state carried from call to call (prefill portions and decode steps run the same
// kernels): the short causal convolution of a state-space layer, its step sizes and decays, the per-channel decays of
// gated linear attention, and the gated linear recurrence both share:
//     St <- diag(a_t) St + k_t (sc_t u_t)^T ,  y_t = St^T c_t + skip * u_t          (St: N x P per head, fp32)
// Everything that enters the recurrence is fp32; the projections it reads are in the model's storage type.
#include <math.h>

#include "../../include/livecc_b200.h"
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
// z -> log decay, b -> beta (see delta_gates)
template <typename T>
__global__ void delta_gates_kernel(float* __restrict__ z, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                   const T* __restrict__ b, int ld_b, float* __restrict__ beta_out, int S, int heads, int N) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int HN = heads * N;
    if (i < (int64_t)S * HN) {
        const int c = (int)(i % HN);
        z[i] = -expf(a_log[c / N]) * softplus_f(z[i] + dt_bias[c]);
    }
    if (i < (int64_t)S * heads) {
        const int t = (int)(i / heads), h = (int)(i % heads);
        beta_out[i] = 1.f / (1.f + expf(-ldf(b + (size_t)t * ld_b + h)));
    }
}

// The thread layout of gated_scan_kernel (NT state entries of one value channel per thread, JP lanes per channel). Per token:
// the state decays, the JP lanes reduce St^T k and St^T c together, the write w = beta (u - St^T k) lands, and the read-out is
// St^T c + (k . c) w: the same value as reading the state after the write, with one reduction round instead of two. With
// unit_eps the staged k and c rows are brought to unit length first (one warp per token), which also yields k . c.
template <typename T>
__global__ void __launch_bounds__(kScanThreads) delta_scan_kernel(ScanArgs a, SeqPos pos) {
    if (seq_done(pos)) return;
    extern __shared__ float sm[];
    const int N = a.N, P = a.P, S = a.S;
    const int JP = blockDim.x, cols = blockDim.y;
    const int h = blockIdx.x;
    const int col = threadIdx.y;
    const int p = blockIdx.y * cols + col;
    const int j = threadIdx.x;
    const int tid = threadIdx.y * JP + threadIdx.x, nthr = cols * JP;
    const int n0 = j * NT;
    const int g = h / a.heads_per_group;
    // shared: k[TT][N], c[TT][N], dec[TT][N], beta[TT], kc[TT], u[TT][cols]
    float* sk = sm;
    float* scv = sk + TT * N;
    float* sd = scv + TT * N;
    float* sb = sd + TT * N;
    float* skc = sb + TT;
    float* su = skc + TT;

    float st[NT];
    float* gstate = a.state + ((size_t)h * P + (p < P ? p : 0)) * N;
#pragma unroll
    for (int i = 0; i < NT; ++i) st[i] = (p < P && n0 + i < N) ? gstate[n0 + i] : 0.f;
    const T* gk = (const T*)a.k + (size_t)g * N;
    const T* gc = (const T*)a.c + (size_t)g * N;
    const T* gu = (const T*)a.u + (size_t)h * P + blockIdx.y * cols;

    for (int t0 = 0; t0 < S; t0 += TT) {
        const int nt = min(TT, S - t0);
        __syncthreads();
        for (int e = tid; e < nt * N; e += nthr) {
            const int t = e / N, n = e % N;
            sk[e] = ldf(gk + (size_t)(t0 + t) * a.ld_k + n);
            scv[e] = ldf(gc + (size_t)(t0 + t) * a.ld_c + n);
            sd[e] = expf(a.a[((size_t)(t0 + t) * a.heads + h) * N + n]);
        }
        for (int e = tid; e < nt; e += nthr) sb[e] = a.sc ? a.sc[(size_t)(t0 + e) * a.heads + h] : 1.f;
        for (int e = tid; e < nt * cols; e += nthr) {
            const int t = e / cols, c = e % cols;
            su[e] = (blockIdx.y * cols + c < P) ? ldf(gu + (size_t)(t0 + t) * a.ld_u + c) : 0.f;
        }
        __syncthreads();
        for (int t = tid >> 5; t < nt; t += nthr >> 5) {     // one warp per token: unit length, scale, k . c
            const int lane = tid & 31;
            float sk2 = 0.f, sc2 = 0.f;
            for (int n = lane; n < N; n += 32) { sk2 = fmaf(sk[t * N + n], sk[t * N + n], sk2); sc2 = fmaf(scv[t * N + n], scv[t * N + n], sc2); }
            sk2 = warp_sum(sk2); sc2 = warp_sum(sc2);
            const float rk = a.unit_eps > 0.f ? 1.f / sqrtf(sk2 + a.unit_eps) : 1.f;
            const float rc = (a.unit_eps > 0.f ? 1.f / sqrtf(sc2 + a.unit_eps) : 1.f) * a.cs;
            float kc = 0.f;
            for (int n = lane; n < N; n += 32) {
                const float kv = sk[t * N + n] * rk, cv = scv[t * N + n] * rc;
                sk[t * N + n] = kv; scv[t * N + n] = cv;
                kc = fmaf(kv, cv, kc);
            }
            kc = warp_sum(kc);
            if (lane == 0) skc[t] = kc;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float u = su[t * cols + col];
            const float* kt = sk + t * N + n0;
            const float* ct = scv + t * N + n0;
            const float* dv = sd + t * N + n0;
            float ks = 0.f, cs = 0.f;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                if (n0 + i < N) {
                    st[i] *= dv[i];
                    ks = fmaf(st[i], kt[i], ks);
                    cs = fmaf(st[i], ct[i], cs);
                }
            }
            for (int o = JP >> 1; o > 0; o >>= 1) {          // fixed butterfly order
                ks += __shfl_xor_sync(0xffffffffu, ks, o);
                cs += __shfl_xor_sync(0xffffffffu, cs, o);
            }
            const float w = sb[t] * (u - ks);
#pragma unroll
            for (int i = 0; i < NT; ++i)
                if (n0 + i < N) st[i] = fmaf(kt[i], w, st[i]);
            if (j == 0 && p < P) a.y[(size_t)(t0 + t) * a.ld_y + (size_t)h * P + p] = fmaf(skc[t], w, cs);
        }
    }
    if (p < P) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
            if (n0 + i < N) gstate[n0 + i] = st[i];
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

int delta_gates(int dt, float* z, const float* dt_bias, const float* a_log, const void* b, int ld_b, float* beta_out, int S,
                int heads, int N, cudaStream_t s) {
    if (!z || !dt_bias || !a_log || !b || !beta_out || S < 1 || heads < 1 || N < 1) return -2;
    const int64_t n = (int64_t)S * heads * N;
    count_launch();
    if (dt == DT_F32)
        delta_gates_kernel<float><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(z, dt_bias, a_log, (const float*)b, ld_b, beta_out, S, heads, N);
    else
        delta_gates_kernel<bf16><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(z, dt_bias, a_log, (const bf16*)b, ld_b, beta_out, S, heads, N);
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
    if (a.delta && (!a.vec_decay || a.skip)) return -2;
    if (!a.delta && a.ws && a.S >= kScanChunkedMin && !pos.kv_len) return gated_scan_chunked(a, pos, s);
    int JP = 1;
    while (JP * NT < a.N) JP *= 2;
    if (JP > 32) return -3;  // N <= 512
    int cols = kScanThreads / JP;
    while (cols * JP > 32 && cols / 2 >= a.P) cols /= 2;   // narrow heads: fewer idle lanes, but always whole warps
    dim3 block(JP, cols), grid(a.heads, (a.P + cols - 1) / cols);
    const size_t smem = sizeof(float) * ((size_t)TT * a.N * 2 + (size_t)TT * (a.vec_decay ? a.N : 1) + TT * (a.delta ? 2 : 1) +
                                         (size_t)TT * cols);
    if (smem > 200 * 1024) return -3;
    count_launch();
    if (a.delta) {
        if (a.dt == DT_F32) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            delta_scan_kernel<float><<<grid, block, smem, s>>>(a, pos);
        } else {
            if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            delta_scan_kernel<bf16><<<grid, block, smem, s>>>(a, pos);
        }
        return cudaGetLastError() == cudaSuccess ? 0 : -100;
    }
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
