// General-shape linear layers: C[M,N] = A[M,K] x W[N,K]^T (+ bias), fp32 accumulation, bf16 or fp32 storage.
// Two CUDA-core kernels cover every shape the tensor-core GEMM (gemm_tcgen05.cu) does not take: ragged N or K, fp32
// storage (true fp32 FMAs, no reduced-precision matrix mode), and the few-row case of a decode step, where the
// weight matrix is streamed once and every row of A is multiplied against it (HBM-bound).
#include <type_traits>
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

constexpr int BM = 64, BN = 64, BK = 16;

// One of several independent problems per blockIdx.z (plain calls: one group, no lists). With row_off the group's rows are
// row_off[z] .. row_off[z+1]-1 of C and of the row list a_rows (or of A itself).
struct Grp {
    int64_t a_stride, w_stride, c_stride;
    const int* row_off;
    const int* a_rows;
    int act;
    int compact;   // few-row kernel with lists: blockIdx.y counts the non-empty lists of `compact` groups (0: blockIdx.y is the group)
    int glu_F;     // few-row kernel, GLU form: a warp owns output column n = the gate row and the up row of that column
    int glu_il16;
    float glu_limit;
    float glu_alpha, glu_up_bias;   // g * sigmoid(alpha g) * (u + up_bias)
};
__device__ __forceinline__ float act_of(float v, int act) {
    if (act == ACT_RELU2) { v = fmaxf(v, 0.f); v *= v; }
    else if (act == ACT_GELU_TANH) v = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

// 64 x 64 output tile per CTA, 256 threads x (4 x 4) accumulators, k-slices of 16 staged in shared memory as fp32.
template <typename T, typename TC>
__global__ void __launch_bounds__(256) linear_tile_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int ldw,
                                                          const float* __restrict__ bias, TC* __restrict__ C, int ldc, int M,
                                                          int N, int K, Grp g) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    int row0 = 0;
    if (g.row_off) {
        row0 = g.row_off[blockIdx.z];
        M = g.row_off[blockIdx.z + 1] - row0;
        if (m0 >= M) return;
    }
    A += blockIdx.z * g.a_stride; W += blockIdx.z * g.w_stride; C += blockIdx.z * g.c_stride + (size_t)row0 * ldc;
    const int* arow = g.a_rows ? g.a_rows + row0 : nullptr;
    if (!arow) A += (size_t)row0 * lda;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread; consecutive threads read consecutive k (coalesced)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256, r = e / BK, k = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            As[k][r] = (gm < M && gk < K) ? ldf(A + (size_t)(arow ? arow[gm] : gm) * lda + gk) : 0.f;
            Ws[k][r] = (gn < N && gk < K) ? ldf(W + (size_t)gn * ldw + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][tm + i]; w[i] = Ws[k][tn + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + tm + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tn + j;
            if (gn < N) stf(C + (size_t)gm * ldc + gn, act_of(acc[i][j] + (bias ? bias[gn] : 0.f), g.act));
        }
    }
}

// Few rows (M <= 8), the shape of a decode step: the weight matrix is streamed once (HBM-bound). A warp owns WR output
// columns (2 for wide matrices; 1, in CTAs of 2 warps, when N is small, so that every SM still has enough loads in
// flight) and keeps WR x WU independent 16-byte non-allocating loads of their weight rows in flight per lane before it
// touches the activations (which stay in L1); lanes stride over k and keep one accumulator per (column, row of A), so
// the order of a column's sum does not depend on WR or M. Scalar loads when K or a row start is not 16-byte aligned.
constexpr int kRowsMax = 8;
constexpr int WU = 4;
template <typename T> struct Vec16;
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& u, float (&v)[8]) {
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
    }
};
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& u, float (&v)[4]) {
        v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
    }
};

template <typename T, typename TC, bool VEC, int WR, bool GLU = false>
__global__ void __launch_bounds__(256) linear_rows_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int ldw,
                                                          const float* __restrict__ bias, TC* __restrict__ C, int ldc, int M_all,
                                                          int N, int K, Grp g) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * (blockDim.x >> 5) + warp) * (GLU ? 1 : WR);
    if (n0 >= N) return;
    int row0 = 0, z = blockIdx.y;
    if (g.row_off) {
        if (g.compact) {
            // a decode step routes a handful of rows to a handful of lists: the grid has one y per possible non-empty list
            int seen = -1;
            for (z = 0; z < g.compact; ++z)
                if (g.row_off[z + 1] > g.row_off[z] && ++seen == (int)blockIdx.y) break;
            if (z == g.compact) return;
        }
        row0 = g.row_off[z];
        M_all = g.row_off[z + 1] - row0;
    }
    const T* A0 = A + z * g.a_stride;
    W += z * g.w_stride;
    TC* C0 = C + z * g.c_stride + (size_t)row0 * ldc;
    const int* arow = g.a_rows ? g.a_rows + row0 : nullptr;
    if (!arow) A0 += (size_t)row0 * lda;
    // a group with more than kRowsMax rows walks them in blocks (the weights come from L2 after the first block); a row's
    // sum is the same whatever block it falls into
    for (int mb = 0; mb < M_all; mb += kRowsMax) {
    const int M = min(kRowsMax, M_all - mb);
    const T* arp[kRowsMax];
#pragma unroll
    for (int m = 0; m < kRowsMax; ++m) arp[m] = A0 + (size_t)(m < M ? (arow ? arow[mb + m] : mb + m) : 0) * lda;
    C = C0 + (size_t)mb * ldc;
    float acc[WR][kRowsMax];
#pragma unroll
    for (int r = 0; r < WR; ++r)
#pragma unroll
        for (int m = 0; m < kRowsMax; ++m) acc[r][m] = 0.f;
    // the weight row behind accumulator r: output columns n0, n0 + 1, ...; in the GLU form (WR = 2) the gate row (r = 0) and
    // the up row (r = 1) of output column n0
    auto wrow = [&](int r) -> int {
        if (GLU) return g.glu_il16 ? ((n0 >> 4) << 5) + (n0 & 15) + 16 * r : n0 + r * g.glu_F;
        return min(n0 + r, N - 1);
    };
    if (VEC) {
        constexpr int V = Vec16<T>::N;
        const T* w[WR];
#pragma unroll
        for (int r = 0; r < WR; ++r) w[r] = W + (size_t)wrow(r) * ldw;
        for (int kb = lane * V; kb < K; kb += 32 * V * WU) {
            uint4 wq[WR][WU];
#pragma unroll
            for (int r = 0; r < WR; ++r)
#pragma unroll
                for (int u = 0; u < WU; ++u) {
                    const int k = kb + u * 32 * V;
                    wq[r][u] = k < K ? ld_stream16(w[r] + k) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
            for (int u = 0; u < WU; ++u) {
                const int k = min(kb + u * 32 * V, K - V);      // past the end the weights are zero; keep the address valid
                float wv[WR][V];
#pragma unroll
                for (int r = 0; r < WR; ++r) Vec16<T>::unpack(wq[r][u], wv[r]);
#pragma unroll
                for (int m = 0; m < kRowsMax; ++m) {
                    if (m < M) {
                        float av[V];
                        Vec16<T>::unpack(__ldg(reinterpret_cast<const uint4*>(arp[m] + k)), av);
#pragma unroll
                        for (int r = 0; r < WR; ++r)
#pragma unroll
                            for (int i = 0; i < V; ++i) acc[r][m] = fmaf(av[i], wv[r][i], acc[r][m]);
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
#pragma unroll
            for (int r = 0; r < WR; ++r) {
                const float wv = ldf(W + (size_t)wrow(r) * ldw + k);
#pragma unroll
                for (int m = 0; m < kRowsMax; ++m)
                    if (m < M) acc[r][m] = fmaf(ldf(arp[m] + k), wv, acc[r][m]);
            }
        }
    }
    if (GLU) {
#pragma unroll
        for (int m = 0; m < kRowsMax; ++m) {
            if (m < M) {
                const float gt = fminf(warp_sum(acc[0][m]), g.glu_limit);
                const float up = fminf(fmaxf(warp_sum(acc[WR - 1][m]), -g.glu_limit), g.glu_limit);
                if (lane == 0) stf(C + (size_t)m * ldc + n0, gt / (1.f + expf(-g.glu_alpha * gt)) * (up + g.glu_up_bias));
            }
        }
        continue;
    }
#pragma unroll
    for (int r = 0; r < WR; ++r) {
        const int n = n0 + r;
#pragma unroll
        for (int m = 0; m < kRowsMax; ++m) {
            if (m < M) {
                const float v = warp_sum(acc[r][m]);
                if (lane == 0 && n < N) stf(C + (size_t)m * ldc + n, act_of(v + (bias ? bias[n] : 0.f), g.act));
            }
        }
    }
    }
}

template <typename T, typename TC>
int launch_linear(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M, int N, int K,
                  cudaStream_t s, int groups = 1, Grp g = Grp{0, 0, 0, nullptr, nullptr, ACT_NONE, 0, 0, 0, 0.f}, int M_total = 0,
                  void* glu_tmp = nullptr, int ld_tmp = 0) {
    // GLU form: N = glu_F output columns from 2 * glu_F weight rows
    // lists: the row kernel while all groups together have few rows (a decode step routes `top` rows per sequence)
    if (g.row_off ? M_total <= 8 * kRowsMax : M <= kRowsMax) {
        constexpr int V = Vec16<T>::N;
        const bool vec = (K % V) == 0 && (lda % V) == 0 && (ldw % V) == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0 &&
                         (g.a_stride % V) == 0 && (g.w_stride % V) == 0;
        int grid_y = groups;
        if (g.row_off && M_total < groups) { g.compact = groups; grid_y = M_total; }
        count_launch();
        if (g.glu_F > 0) {
            if constexpr (std::is_same<T, TC>::value) {
                if (vec) linear_rows_kernel<T, TC, true, 2, true><<<dim3((N + 1) / 2, grid_y), 64, 0, s>>>((const T*)A, lda, (const T*)W, ldw, bias, (TC*)C, ldc, M, N, K, g);
                else linear_rows_kernel<T, TC, false, 2, true><<<dim3((N + 1) / 2, grid_y), 64, 0, s>>>((const T*)A, lda, (const T*)W, ldw, bias, (TC*)C, ldc, M, N, K, g);
                return cudaGetLastError() == cudaSuccess ? 0 : -100;
            } else {
                return -2;
            }
        }
#define LCC_ROWS(VECB, WRN, WARPS)                                                                                         \
    linear_rows_kernel<T, TC, VECB, WRN><<<dim3((N + WARPS * WRN - 1) / (WARPS * WRN), grid_y), WARPS * 32, 0, s>>>(            \
        (const T*)A, lda, (const T*)W, ldw, bias, (TC*)C, ldc, M, N, K, g)
        if (N >= 8192) {
            if (vec) LCC_ROWS(true, 2, 8); else LCC_ROWS(false, 2, 8);
        } else {
            if (vec) LCC_ROWS(true, 1, 2); else LCC_ROWS(false, 1, 2);
        }
#undef LCC_ROWS
    } else if (g.glu_F > 0) {
        // raw gate and up columns into the caller's scratch, then the activation as a row kernel
        if (!glu_tmp || ld_tmp < 2 * N || !std::is_same<T, TC>::value) return -2;
        Grp raw = g;
        raw.glu_F = 0;
        raw.c_stride = 0;
        dim3 grid((2 * N + BN - 1) / BN, (M + BM - 1) / BM, groups);
        count_launch();
        linear_tile_kernel<T, T><<<grid, 256, 0, s>>>((const T*)A, lda, (const T*)W, ldw, bias, (T*)glu_tmp, ld_tmp, M, 2 * N, K, raw);
        if (cudaGetLastError() != cudaSuccess) return -100;
        const int rows = g.row_off ? M_total : M;
        return glu_clamp_swish(sizeof(T) == 4 ? DT_F32 : DT_BF16, glu_tmp, ld_tmp, C, ldc, rows, N, g.glu_limit, s, g.glu_il16 != 0, g.glu_alpha, g.glu_up_bias);
    } else {
        dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, groups);
        count_launch();
        linear_tile_kernel<T, TC><<<grid, 256, 0, s>>>((const T*)A, lda, (const T*)W, ldw, bias, (TC*)C, ldc, M, N, K, g);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace

int linear_any(int dt, const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, bool c_f32,
               int M, int N, int K, cudaStream_t s) {
    if (!A || !W || !C || M < 1 || N < 1 || K < 1 || lda < K || ldw < K || ldc < N) return -2;
    if (dt == DT_F32) return launch_linear<float, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, s);
    if (c_f32) return launch_linear<bf16, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, s);
    return launch_linear<bf16, bf16>(A, lda, W, ldw, bias, C, ldc, M, N, K, s);
}

int linear_grouped(const GroupedLinear& q, cudaStream_t s) {
    if (!q.A || !q.W || !q.C || q.groups < 1 || q.groups > 65535 || q.M < 1 || q.N < 1 || q.K < 1 || q.lda < q.K || q.ldw < q.K ||
        q.ldc < q.N || (q.a_rows && !q.row_off))
        return -2;
    if (q.glu_F > 0 && (q.N != q.glu_F || q.act != ACT_NONE || q.c_f32 || (q.glu_il16 && (q.glu_F % 16)) || q.c_stride != 0 ||
                        (q.groups > 1 && !q.row_off)))
        return -2;
    const Grp g{q.a_stride, q.w_stride, q.c_stride, q.row_off, q.a_rows, q.act, 0, q.glu_F, q.glu_il16 ? 1 : 0, q.glu_limit, q.glu_alpha, q.glu_up_bias};
    const int mt = q.row_off ? (q.M_total > 0 ? q.M_total : q.M * q.groups) : 0;
    if (q.dt == DT_F32) return launch_linear<float, float>(q.A, q.lda, q.W, q.ldw, nullptr, q.C, q.ldc, q.M, q.N, q.K, s, q.groups, g, mt, q.glu_tmp, q.ld_tmp);
    if (q.c_f32) return launch_linear<bf16, float>(q.A, q.lda, q.W, q.ldw, nullptr, q.C, q.ldc, q.M, q.N, q.K, s, q.groups, g, mt);
    return launch_linear<bf16, bf16>(q.A, q.lda, q.W, q.ldw, nullptr, q.C, q.ldc, q.M, q.N, q.K, s, q.groups, g, mt, q.glu_tmp, q.ld_tmp);
}

}  // namespace lcc
