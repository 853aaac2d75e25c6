// Latent (low-rank) key/value cache. A token's cache row is [c: R channels | kr: DR channels]: c is the RMS-normed
// latent from which every head's unrotated keys and values are up-projections, kr one rotary key part shared by all
// heads. Attention runs in the absorbed form: head h's query against a cache row is (W_uk_h^T q_h) . c + rot(qr_h) . kr,
// so the cache serves as one key/value head of size R + DR whose values are the first R channels of the keys. This file
// holds the row kernel that fills the cache and the rotated query part; norm, positions, angles are fp32.
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

__device__ __forceinline__ int seq_past(const SeqPos& p) { return p.kv_len ? *p.kv_len : p.past; }
__device__ __forceinline__ bool seq_done(const SeqPos& p) { return p.finished && *p.finished; }

// gridDim.y CTAs per new row: all of them share the rotation of the query heads; the first one also norms the latent and
// fills the cache row.
template <typename T>
__global__ void __launch_bounds__(256) latent_kv_append_kernel(const T* __restrict__ proj, int ld, int has_kv,
                                                               const float* __restrict__ norm_w, float eps,
                                                               const float* __restrict__ inv_freq, float mag,
                                                               float* __restrict__ q_out, T* __restrict__ k_pages,
                                                               const int* __restrict__ page_table, int page_size, int H, int D,
                                                               int DR, int R, SeqPos pos, const T* __restrict__ qsrc, int ld_q) {
    if (seq_done(pos)) return;
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int pi = seq_past(pos) + t;
    const float p = (float)pi;
    const T* row = proj + (size_t)t * ld;
    const int half = DR / 2, QH = D + DR, nq = H * QH, KD = R + DR;
    // rotated query part of every head -> q_out[t, h, R + j]
    for (int i = threadIdx.x + blockIdx.y * blockDim.x; i < H * DR; i += blockDim.x * gridDim.y) {
        const int h = i / DR, r = i % DR;
        const int j = r < half ? r : r - half;
        const float ang = p * inv_freq[j];
        const float c = cosf(ang) * mag, s = sinf(ang) * mag;
        const T* qr = (qsrc ? qsrc + (size_t)t * ld_q : row) + (size_t)h * QH + D;
        const float v = ldf(qr + r), other = ldf(qr + (r < half ? r + half : r - half));
        q_out[((size_t)t * H + h) * KD + R + r] = r < half ? v * c - other * s : v * c + other * s;
    }
    if (!has_kv || blockIdx.y != 0) return;
    const T* lat = qsrc ? row : row + nq;      // queries of their own: the row starts with the latent
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = ldf(lat + i); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float rn = 1.f / sqrtf(ss / (float)R + eps);
    T* dst = k_pages + ((size_t)page_table[pi / page_size] * page_size + pi % page_size) * KD;
    for (int i = threadIdx.x; i < R; i += blockDim.x) stf(dst + i, ldf(lat + i) * rn * norm_w[i]);
    for (int r = threadIdx.x; r < DR; r += blockDim.x) {
        const int j = r < half ? r : r - half;
        const float ang = p * inv_freq[j];
        const float c = cosf(ang) * mag, s = sinf(ang) * mag;
        const float v = ldf(lat + R + r), other = ldf(lat + R + (r < half ? r + half : r - half));
        stf(dst + R + r, r < half ? v * c - other * s : v * c + other * s);
    }
}

}  // namespace

int latent_kv_append(int dt, const void* proj, int ld, int has_kv, const float* norm_w, float eps, const float* inv_freq,
                     float mag, float* q_out, void* k_pages, const int* page_table, int page_size, int S, int H, int D,
                     int DR, int R, SeqPos pos, cudaStream_t s, const void* q, int ld_q) {
    if (!proj || !inv_freq || !q_out || S < 1 || H < 1 || D < 0 || DR < 2 || (DR & 1) || R < 1) return -2;
    if (has_kv && (!norm_w || !k_pages || !page_table || page_size < 1)) return -2;
    count_launch();
    const dim3 S_grid(S, S < 32 ? 4 : 1);
    if (dt == DT_F32)
        latent_kv_append_kernel<float><<<S_grid, 256, 0, s>>>((const float*)proj, ld, has_kv, norm_w, eps, inv_freq, mag, q_out,
                                                         (float*)k_pages, page_table, page_size, H, D, DR, R, pos, (const float*)q, ld_q);
    else
        latent_kv_append_kernel<bf16><<<S_grid, 256, 0, s>>>((const bf16*)proj, ld, has_kv, norm_w, eps, inv_freq, mag, q_out,
                                                        (bf16*)k_pages, page_table, page_size, H, D, DR, R, pos, (const bf16*)q, ld_q);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace lcc
