// Native runtime of the hybrid sequence models: one C call runs a whole step (a prompt portion of any length, or one
// decode token per sequence) over every layer and produces the logits of the wanted rows. Prefill and decode use the
// same launch sequence; what differs is the row count and which kernel of an op the shape selects.
// A layer is a mixer (its output lands in one buffer), a feed-forward (dense or routed) and the block form around them
// (post-norm residual, pre-norm sublayers on several residual streams, a parallel block whose mixer and feed-forward read
// one normed row, or sublayers that read the residual stream itself and are normed on their way back into it); the three are
// chosen independently per model.
// The host (Python) owns every buffer; this file only sequences kernel launches.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "../../include/livecc_b200.h"
#include "cabi_common.h"
#include "gemm.h"
#include "launch.h"
#include "seqmix.h"

struct lcc_seq_model {
    lcc_ctx* ctx;
    lcc_seq_model_desc d;
    std::vector<lcc_seq_layer> layers;
    uint8_t* ws = nullptr;
    size_t ws_bytes = 0;
    int cap_tokens = 0, cap_want = 0;
    // few-row steps run the shared expert beside the router and the routed experts: a second stream, forked and joined by
    // events (inside a capture these become parallel branches of the graph)
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    bool use_tc = true;  // bf16: large 8-aligned linear layers go to the tcgen05 GEMM, prompt attention to the mma kernel (LIVECC_B200_SEQ_TC=0: never)
};

namespace {

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

struct Dims {
    int inner, conv_ch, s_proj;          // SSD
    int l_nq, l_nk, l_nv, l_proj, l_o;   // left
    int r_nk, r_nv, r_proj;              // right
    int t_nk, t_nv, t_proj, t_pack;      // retention: q and k columns, v columns, projection rows, fp32 pack [q | k | v]
    int a_nq, a_kv, a_kd, a_proj, a_gate, a_lat, a_o;   // latent attention: query columns, latent + key part, cache row, projection rows,
                                                        // gate column, absorbed-output columns, value columns
    int m_nq, m_nk, m_nv, m_vcol, m_gate, m_ngate, m_proj, m_o;   // masked attention: q, k, projected v columns, the values' first column,
                                                                  // the gate's first column and width, projection rows, output columns
    int a_qin;                                   // latent attention: the projection's leading query block (the heads, or their latent)
    int d_nk, d_nv, d_k, d_v, d_conv_ch, d_b, d_a1, d_g1, d_proj;   // delta rule: q / k columns, v columns, first columns of k, v, beta,
                                                                    // decay bottleneck, gate bottleneck (every block starts at a multiple of
                                                                    // 8 columns; q, k, v and their padding are the convolution's channels)
};
Dims dims_of(const lcc_seq_layer& L) {
    Dims z{};
    if (L.type == LCC_MIX_SSD) {
        z.inner = L.s_heads * L.s_vdim;
        z.conv_ch = z.inner + 2 * L.s_groups * L.s_state;
        z.s_proj = z.inner + z.conv_ch + L.s_heads;
    } else if (L.type == LCC_MIX_PARALLEL) {
        z.l_nq = L.l_heads * L.l_dim; z.l_nk = L.l_kv_heads * L.l_dim; z.l_nv = L.l_kv_heads * L.l_vdim;
        z.l_proj = z.l_nq + z.l_nk + z.l_nv + L.l_heads;
        z.l_o = L.l_heads * L.l_vdim;
        z.r_nk = L.r_heads * L.r_dim; z.r_nv = L.r_heads * L.r_vdim;
        z.r_proj = 2 * z.r_nk + 2 * z.r_nv + L.r_rank;
    } else if (L.type == LCC_MIX_RETENTION) {
        z.t_nk = L.t_heads * L.t_dim; z.t_nv = L.t_heads * L.t_vdim;
        z.t_proj = 2 * z.t_nk + 2 * z.t_nv;
        z.t_pack = 2 * z.t_nk + z.t_nv;
    } else if (L.type == LCC_MIX_LATENT) {
        z.a_nq = L.a_heads * (L.a_dim + L.a_rot_dim);
        z.a_kd = L.a_rank + L.a_rot_dim;
        z.a_kv = L.a_kv_from >= 0 ? 0 : z.a_kd;
        z.a_qin = L.a_q_rank > 0 ? L.a_q_rank : z.a_nq;
        z.a_gate = z.a_qin + z.a_kv;
        z.a_proj = z.a_gate + (L.a_gate ? L.a_heads : 0);
        z.a_lat = L.a_heads * L.a_rank;
        z.a_o = L.a_heads * L.a_vdim;
    } else if (L.type == LCC_MIX_ATTENTION) {
        z.m_nq = L.m_heads * L.m_dim; z.m_nk = L.m_kv_heads * L.m_dim;
        z.m_nv = L.m_value_keys ? 0 : L.m_kv_heads * L.m_vdim;
        z.m_vcol = L.m_value_keys ? z.m_nq : z.m_nq + z.m_nk;       // the values are the key columns as projected, or their own
        z.m_gate = z.m_nq + z.m_nk + z.m_nv;
        z.m_ngate = L.m_gate == LCC_GATE_CHANNEL ? L.m_heads * L.m_vdim : (L.m_gate == LCC_GATE_HEAD ? L.m_heads : 0);
        z.m_proj = z.m_gate + z.m_ngate;
        z.m_o = L.m_heads * L.m_vdim;
    } else if (L.type == LCC_MIX_DELTA) {
        auto up8 = [](int n) { return (n + 7) / 8 * 8; };
        z.d_nk = L.d_kv_heads * L.d_dim; z.d_nv = L.d_heads * L.d_vdim;
        z.d_k = up8(z.d_nk); z.d_v = z.d_k + up8(z.d_nk); z.d_conv_ch = z.d_v + up8(z.d_nv);
        z.d_b = z.d_conv_ch; z.d_a1 = z.d_b + up8(L.d_heads); z.d_g1 = z.d_a1 + up8(L.d_rank_a);
        z.d_proj = z.d_g1 + up8(L.d_rank_g);
    }
    return z;
}

// Row strides of activation buffers are rounded up to 8 elements so that every buffer a tensor-core GEMM may read or
// write has 16-byte aligned rows.
inline int ld8(int n) { return (n + 7) / 8 * 8; }

constexpr int kMoeTile = 128;        // row tile of the grouped tensor-core GEMM: expert lists are padded to it on that route
constexpr int kMoeTcMinRows = 256;   // routed rows (tokens x top) from which the experts run on the tensor cores
constexpr int kForkMaxRows = 32;     // rows up to which the shared expert runs on the second stream

struct WsLayout {
    size_t x32, xa, proj, proj2, mid, mid2, y32, q32, f1, f2, o1, o2, xf, vkeep, scan, scan_floats, xsum, moe_f, moe_i, moe_x, moe_h, moe_g, moe_o, split, split_floats, total;
    int moe_rows;         // rows of the expert-sorted buffers: top per token, every list padded to a whole 128-row tile
    int w_proj, w_proj2, w_mid, w_y, w_q, w_f;
    int moe_e, moe_top;   // largest expert count and top-k of any layer (0: no routed feed-forward)
    int w_vkeep;          // widest value row that a layer keeps for later layers of the step (0: none)
};

WsLayout make_layout(const lcc_seq_model* m, int NT, int NW) {
    WsLayout L{};
    const size_t es = lcc::dt_size(m->d.dtype);
    const size_t nt = NT > 0 ? NT : 1, nw = NW > 0 ? NW : 1;
    int wp = 8, wp2 = 8, wm = 8, wy = 8, wq = 8, wf = 8;
    size_t scan_floats = 0;
    int moe_e = 0, moe_top = 0, moe_ff = 0, moe_rows = 0, moe_glu = 0;   // moe_glu: widest hidden row of a gated expert
    size_t split_floats = 0;   // key-split partials of few-row plain causal attention
    int wvk = 0;
    size_t delta_floats = 0;   // the delta rule's prepared operands (head by head, fp32) share the fp32 query buffer
    for (const lcc_seq_layer& l : m->layers) {
        const Dims z = dims_of(l);
        if (l.type == LCC_MIX_DELTA) {
            wp = std::max(wp, z.d_proj); wm = std::max(wm, std::max(z.d_conv_ch, ld8(z.d_nv))); wp2 = std::max(wp2, ld8(z.d_nv));
            wy = std::max(wy, z.d_nv); wf = std::max(wf, l.d_heads * l.d_dim);
            delta_floats = std::max(delta_floats, lcc::delta_operand_floats((int)nt, l.d_heads, l.d_kv_heads, l.d_dim, l.d_vdim));
        }
        if (l.type == LCC_MIX_LATENT && l.a_q_rank > 0) { wp2 = std::max(wp2, ld8(z.a_nq)); wm = std::max(wm, ld8(l.a_q_rank)); }
        if (l.type == LCC_MIX_ATTENTION && l.m_vmix_role == 1) wvk = std::max(wvk, ld8(z.m_nv));
        if (l.type == LCC_MIX_SSD) {
            wp = std::max(wp, ld8(z.s_proj)); wm = std::max(wm, ld8(std::max(z.conv_ch, z.inner)));
            wy = std::max(wy, z.inner); wf = std::max(wf, l.s_heads);
            scan_floats = std::max(scan_floats, lcc::gated_scan_ws_floats(NT, l.s_heads, l.s_state, l.s_vdim));
        } else if (l.type == LCC_MIX_PARALLEL) {
            wp = std::max(wp, ld8(std::max(z.l_proj, z.r_proj))); wp2 = std::max(wp2, ld8(z.r_nk));
            wm = std::max(wm, ld8(std::max(z.l_o, z.r_nv)));
            wy = std::max(wy, z.r_nv); wq = std::max(wq, z.l_nq); wf = std::max(wf, z.r_nk);
            scan_floats = std::max(scan_floats, lcc::gated_scan_ws_floats(NT, l.r_heads, l.r_dim, l.r_vdim));
        } else if (l.type == LCC_MIX_RETENTION) {
            wp = std::max(wp, ld8(z.t_proj)); wm = std::max(wm, ld8(z.t_nv));
            wy = std::max(wy, z.t_nv); wq = std::max(wq, z.t_pack); wf = std::max(wf, l.t_heads);
            scan_floats = std::max(scan_floats, lcc::gated_scan_ws_floats(NT, l.t_heads, l.t_dim, l.t_vdim));
        } else if (l.type == LCC_MIX_LATENT) {
            wp = std::max(wp, ld8(z.a_proj)); wm = std::max(wm, ld8(std::max(z.a_lat, z.a_o)));
            wq = std::max(wq, l.a_heads * z.a_kd);
            split_floats = std::max(split_floats, lcc::attn_split_ws_floats(lcc::kAttnTiledMin - 1, l.a_heads, l.a_rank));
        }
        if (l.type == LCC_MIX_PARALLEL && l.l_chunk <= 0)
            split_floats = std::max(split_floats, lcc::attn_split_ws_floats(lcc::kAttnTiledMin - 1, l.l_heads, l.l_vdim));
        if (l.type == LCC_MIX_ATTENTION) {
            wp = std::max(wp, ld8(z.m_proj)); wm = std::max(wm, ld8(z.m_o)); wq = std::max(wq, z.m_nq);
            if (l.m_chunk <= 0)
                split_floats = std::max(split_floats, lcc::attn_split_ws_floats(lcc::kAttnTiledMin - 1, l.m_heads, l.m_vdim));
        }
        if (l.ff_kind == LCC_FF_MOE) {
            const bool glu = l.e_act == LCC_EXPERT_CLAMP_GLU || l.e_act == LCC_EXPERT_SILU_GLU;
            wm = std::max(wm, ld8(l.e_shared_ff));            // the shared expert's hidden row
            // logits row: every router output (real + identity experts), then the shared expert's gate
            moe_e = std::max(moe_e, l.e_experts + l.e_identity); moe_top = std::max(moe_top, l.e_top);
            moe_ff = std::max(moe_ff, ld8(glu ? 2 * l.e_ff : l.e_ff));
            if (glu) moe_glu = std::max(moe_glu, ld8(l.e_ff));
            moe_rows = std::max(moe_rows, (int)nt * l.e_top + (l.e_experts + 1) * kMoeTile);
        } else if (l.ff_kind == LCC_FF_MLP && l.ff > 0) { wm = std::max(wm, ld8(l.ff)); }
        else if (l.ff > 0) { wp = std::max(wp, ld8(2 * l.ff)); wm = std::max(wm, ld8(l.ff)); }
    }
    L.moe_e = moe_e; L.moe_top = moe_top; L.moe_rows = moe_rows;
    L.w_proj = wp; L.w_proj2 = wp2; L.w_mid = wm; L.w_y = wy; L.w_q = wq; L.w_f = wf; L.w_vkeep = wvk;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes); return o; };
    const int W = m->d.width;
    L.x32 = take(nt * W * 4 * (m->d.block == LCC_BLOCK_PRENORM_HC ? m->d.streams : 1));
    L.xsum = take(m->d.block == LCC_BLOCK_PRENORM_HC ? nt * W * 4 : 0);
    // routed feed-forward: fp32 [logits: E+1 | weights: top | shared gate: 1] per row; int32 [sel, rank, pos: top each |
    // src_row: top] per row, then [counts: E | row_off: E+1]
    L.moe_f = take(moe_e ? nt * (size_t)(ld8(moe_e + 1) + 1 + moe_top) * 4 : 0);
    L.moe_i = take(moe_e ? (nt * (size_t)(3 * moe_top) + (size_t)moe_rows + moe_rows / kMoeTile + 1 + 2 * moe_e + 1) * 4 : 0);
    // expert-sorted rows: the gathered inputs (tensor-core route only), the hidden rows, the expert outputs
    L.moe_x = take(moe_e && m->use_tc && m->d.dtype == LCC_DT_BF16 ? (size_t)moe_rows * ld8(W) * es : 0);
    L.moe_h = take((size_t)moe_rows * moe_ff * es);
    L.moe_g = take((size_t)moe_rows * moe_glu * es);
    L.moe_o = take((size_t)moe_rows * (moe_e ? ld8(W) : 0) * es);
    L.xa = take(nt * ld8(W) * es);
    L.proj = take(nt * wp * es);
    L.proj2 = take(nt * wp2 * es);
    L.mid = take(nt * wm * es);
    L.mid2 = take(nt * wm * es);
    L.y32 = take(nt * wy * 4);
    L.q32 = take(std::max(nt * wq, delta_floats) * 4);
    L.f1 = take(nt * wf * 4);
    L.f2 = take(nt * wf * 4);
    L.o1 = take(nt * ld8(W) * es);
    L.o2 = take(nt * ld8(W) * es);
    L.xf = take(nw * ld8(W) * es);
    L.vkeep = take(nt * wvk * es);
    L.scan_floats = NT >= lcc::kScanChunkedMin ? scan_floats : 0;   // a decode-only workspace has no use for it
    L.scan = take(L.scan_floats * 4);
    L.split_floats = split_floats;
    L.split = take(split_floats * 4);
    L.total = off;
    return L;
}

#define STEP(expr, what)                                                                      \
    do {                                                                                      \
        int rc__ = (expr);                                                                    \
        if (rc__) LCC_FAIL(m->ctx, rc__, "%s failed (code %d)", what, rc__);                  \
    } while (0)

// y[M, N] = x[M, K] W^T (+ bias). Large bf16 products with 8-aligned shapes run on the tensor cores; everything else on
// the CUDA-core kernels. bias is fp32; the tensor-core epilogue takes a copy in the storage type (bias_st; without one a
// biased product stays on the CUDA cores). A ragged N runs on the tensor cores when the matrix rows are padded to 8.
int linear(const lcc_seq_model* m, const void* x, int ldx, const void* W, const float* bias, void* y, int ldy,
           bool y_f32, int M, int N, int K, cudaStream_t s, const void* bias_st = nullptr, int act = lcc::ACT_NONE) {
    const int Np = m->d.rows_padded8 ? ld8(N) : N;
    if (act != lcc::ACT_NONE && bias) return -2;
    if (m->use_tc && m->d.dtype == LCC_DT_BF16 && (!y_f32 || (!bias && act == lcc::ACT_NONE)) && (!bias || bias_st) && M >= 16 &&
        (Np >= 32 || y_f32) && K >= 64 && (K % 8) == 0 && (Np % 8) == 0 && ldy >= Np && (ldx % 8) == 0 && (ldy % 8) == 0 &&
        ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0) {   // (a slice of a wider row may start anywhere)
        lcc::GemmArgs a;
        a.c_f32 = y_f32;
        a.A = x; a.B = W; a.C = y; a.M = M; a.N = Np; a.K = K; a.lda = ldx; a.ldb = K; a.ldc = ldy;
        a.bias = bias ? bias_st : nullptr; a.residual = nullptr; a.ldr = 0; a.block_n = 0;
        a.epi = act == lcc::ACT_RELU2 ? lcc::EPI_RELU2 : (act == lcc::ACT_GELU_TANH ? lcc::EPI_GELU_TANH : (bias ? lcc::EPI_BIAS : lcc::EPI_NONE));
        return lcc::gemm_bf16_tn(a, m->ctx->num_sms, s);
    }
    if (act != lcc::ACT_NONE) {   // the activation rides in the store of the CUDA-core kernels too
        lcc::GroupedLinear g{};
        g.dt = m->d.dtype; g.A = x; g.lda = ldx; g.W = W; g.ldw = K; g.C = y; g.ldc = ldy; g.c_f32 = y_f32;
        g.groups = 1; g.M = M; g.N = N; g.K = K; g.act = act;
        return lcc::linear_grouped(g, s);
    }
    return lcc::linear_any(m->d.dtype, x, ldx, W, K, bias, y, ldy, y_f32, M, N, K, s);
}

// Per-head products: head h multiplies columns h * a_stride .. of x with the h-th [N, K] matrix of W and writes columns
// h * c_stride .. of y. One batched tensor-core GEMM when the shapes allow it, else the grouped CUDA-core kernels.
int linear_heads(const lcc_seq_model* m, const void* x, int ldx, int a_stride, const void* W, void* y, int ldy, int c_stride,
                 bool y_f32, int heads, int M, int N, int K, cudaStream_t s) {
    if (m->use_tc && m->d.dtype == LCC_DT_BF16 && M >= 16 && N >= 32 && (K % 64) == 0 && (N % 8) == 0 && (ldx % 8) == 0 &&
        (ldy % 8) == 0 && (a_stride % 8) == 0 && (c_stride % 8) == 0) {
        lcc::GemmArgs a;
        a.A = x; a.B = W; a.C = y; a.M = M; a.N = N; a.K = K; a.lda = ldx; a.ldb = K; a.ldc = ldy;
        a.bias = nullptr; a.residual = nullptr; a.ldr = 0; a.epi = lcc::EPI_NONE; a.block_n = 0;
        a.batch = heads; a.a_col_stride = a_stride; a.c_col_stride = c_stride; a.c_f32 = y_f32;
        return lcc::gemm_bf16_tn(a, m->ctx->num_sms, s);
    }
    lcc::GroupedLinear g{};
    g.dt = m->d.dtype; g.A = x; g.lda = ldx; g.a_stride = a_stride;
    g.W = W; g.ldw = K; g.w_stride = (int64_t)N * K;
    g.C = y; g.ldc = ldy; g.c_stride = c_stride; g.c_f32 = y_f32;
    g.groups = heads; g.M = M; g.N = N; g.K = K;
    return lcc::linear_grouped(g, s);
}

}  // namespace

extern "C" {

lcc_seq_model* lcc_seq_model_create(lcc_ctx* ctx, const lcc_seq_model_desc* desc) {
    if (!ctx || !desc || !desc->layers) return nullptr;
    auto fail = [&](const char* msg) -> lcc_seq_model* { snprintf(ctx->err, sizeof(ctx->err), "lcc_seq_model_create: %s", msg); return nullptr; };
    if (desc->width < 1 || desc->vocab < 1 || desc->n_layers < 1) return fail("bad sizes");
    if (desc->dtype != LCC_DT_BF16 && desc->dtype != LCC_DT_F32) return fail("unknown storage type");
    if (!desc->embed || !desc->final_norm_f32 || !desc->head) return fail("missing weights");
    const bool hc = desc->block == LCC_BLOCK_PRENORM_HC, par = desc->block == LCC_BLOCK_PARALLEL, bn = desc->block == LCC_BLOCK_BRANCHNORM;
    const bool dyt = desc->norm_kind == LCC_NORM_DYT;
    if (desc->block != LCC_BLOCK_POSTNORM && !hc && !par && !bn) return fail("unknown block form");
    if (bn && (desc->canon_taps < 0 || desc->canon_taps > 8)) return fail("at most 8 taps in the convolution in front of a mixer");
    bool vkeep_seen = false;
    int vkeep_cols = 0;
    if (desc->norm_kind != LCC_NORM_RMS && !dyt) return fail("unknown norm kind");
    if (dyt && (!par || !desc->final_norm_bias_f32)) return fail("the Dynamic-Tanh norm is served in parallel blocks and needs its bias");
    if (hc && (desc->streams < 1 || desc->streams > 8)) return fail("1 to 8 residual streams");
    for (int i = 0; i < desc->n_layers; ++i) {
        const lcc_seq_layer& l = desc->layers[i];
        if (l.ff_kind == LCC_FF_MOE) {
            if (l.e_experts < 1 || l.e_experts > 512 || l.e_top < 1 || l.e_top > l.e_experts + std::max(l.e_identity, 0) || l.e_ff < 1 || l.e_shared_ff < 0)
                return fail("routed feed-forward: unsupported sizes");
            if ((!par && !l.norm2_f32) || !l.e_router || (!l.e_correction_f32 && l.e_router_kind != LCC_ROUTER_TOPK_SOFTMAX) || !l.e_up || !l.e_down || (l.e_shared_ff > 0 && (!l.e_shared_up || !l.e_shared_down)))
                return fail("routed feed-forward: missing weights");
            const int outs = l.e_experts + l.e_identity;
            if (l.e_identity < 0 || outs > 512 || l.e_top > outs || (l.e_identity > 0 && (l.e_shared_ff > 0 || !par)))
                return fail("routed feed-forward: identity experts are served in parallel blocks, without a shared expert");
            if (l.e_groups < 0 || (l.e_groups > 0 && (outs % l.e_groups || l.e_keep < 1 || l.e_keep > l.e_groups || l.e_keep * (outs / l.e_groups) < l.e_top)))
                return fail("routed feed-forward: the kept groups must be equal groups that hold at least `top` experts");
            if (l.e_router_kind != LCC_ROUTER_SIGMOID && l.e_router_kind != LCC_ROUTER_SOFTMAX && l.e_router_kind != LCC_ROUTER_TOPK_SOFTMAX) return fail("unknown router kind");
            if (l.e_router_kind == LCC_ROUTER_TOPK_SOFTMAX && (l.e_identity > 0 || l.e_groups > 0 || l.e_shared_ff > 0))
                return fail("routed feed-forward: weights over the chosen logits combine with neither identity experts, groups nor a shared expert");
            if (l.e_act != LCC_EXPERT_RELU2 && l.e_act != LCC_EXPERT_CLAMP_GLU && l.e_act != LCC_EXPERT_SILU_GLU) return fail("unknown expert activation");
            if (l.e_up_il16 && (l.e_act == LCC_EXPERT_RELU2 || l.e_ff % 16)) return fail("interleaved gate / up rows need a gated expert width that is a multiple of 16");
        } else if (l.ff_kind != LCC_FF_GLU && l.ff_kind != LCC_FF_MLP) {
            return fail("unknown feed-forward kind");
        }
        if (bn && l.canon_w_f32 && desc->canon_taps < 1) return fail("a convolution in front of the mixer needs its tap count");
        if (!l.norm1_f32 || (l.ff > 0 && ((!par && !l.norm2_f32) || !l.ff_in || !l.ff_out))) return fail("missing norm / feed-forward weights");
        if (dyt && !l.norm1_bias_f32) return fail("missing norm bias");
        if (par && l.type != LCC_MIX_ATTENTION) return fail("a parallel block takes the attention mixer");
        if (!par && !bn && l.type == LCC_MIX_ATTENTION) return fail("the attention mixer is served in parallel blocks and in blocks normed on the sublayer's output");
        if (bn && l.type == LCC_MIX_PARALLEL) return fail("the parallel mixer merges its branches in a post-norm block");
        if (hc && (!l.hc1_f32 || ((l.ff > 0 || l.ff_kind == LCC_FF_MOE) && !l.hc2_f32))) return fail("missing stream weights");
        if (hc && l.type == LCC_MIX_PARALLEL) return fail("the parallel mixer merges its branches in a post-norm block");
        if (l.type == LCC_MIX_SSD) {
            if (l.s_heads < 1 || l.s_vdim < 1 || l.s_state < 1 || l.s_state > 512 || l.s_groups < 1 || l.s_heads % l.s_groups ||
                l.s_conv < 1 || l.s_conv > 8 || l.s_norm_groups < 1 || (l.s_heads * l.s_vdim) % l.s_norm_groups)
                return fail("state-space layer: unsupported sizes");
            if (!l.s_in || !l.s_conv_w_f32 || !l.s_conv_b_f32 || !l.s_dt_bias_f32 || !l.s_a_log_f32 || !l.s_skip_f32 || !l.s_norm_f32 || !l.s_out)
                return fail("state-space layer: missing weights");
        } else if (l.type == LCC_MIX_PARALLEL) {
            if (l.l_heads < 1 || l.l_kv_heads < 1 || l.l_heads % l.l_kv_heads || l.l_dim < 1 || l.l_vdim < 1 || l.r_heads < 1 ||
                l.r_dim < 1 || l.r_dim > 512 || l.r_vdim < 1 || l.r_rank < 1 || !(l.r_tau > 0.f))
                return fail("parallel layer: unsupported sizes");
            if (!l.l_in || !l.l_in_bias_f32 || !l.l_qnorm_f32 || !l.l_knorm_f32 || !l.l_out || !l.l_branch_norm_f32 || !l.r_in ||
                !l.r_decay_up || !l.r_decay_bias_f32 || !l.r_norm_f32 || !l.r_out || !l.r_branch_norm_f32)
                return fail("parallel layer: missing weights");
        } else if (l.type == LCC_MIX_RETENTION) {
            if (l.t_heads < 1 || l.t_dim < 1 || l.t_dim > 512 || l.t_vdim < 1 || l.t_rot_dims < 0 || (l.t_rot_dims & 1) || l.t_rot_dims > l.t_dim)
                return fail("retention layer: unsupported sizes");
            if (!l.t_in || !l.t_log_decay_f32 || !l.t_norm_f32 || !l.t_out || (l.t_rot_dims > 0 && !l.rot_inv_freq_f32))
                return fail("retention layer: missing weights");
        } else if (l.type == LCC_MIX_LATENT) {
            if (l.a_heads < 1 || l.a_dim < 1 || l.a_rot_dim < 2 || (l.a_rot_dim & 1) || l.a_vdim < 1 || l.a_rank < 1)
                return fail("latent attention layer: unsupported sizes");
            if (l.a_kv_from >= 0) {
                if (l.a_kv_from >= i) return fail("latent attention layer: the shared cache must belong to an earlier layer");
                const lcc_seq_layer& o = desc->layers[l.a_kv_from];
                if (o.type != LCC_MIX_LATENT || o.a_kv_from >= 0 || o.a_rank != l.a_rank || o.a_rot_dim != l.a_rot_dim)
                    return fail("latent attention layer: the shared cache has another geometry");
            } else if (!l.a_latent_norm_f32) {
                return fail("latent attention layer: missing weights");
            }
            if (!l.a_in || !l.a_uk_t || !l.a_uv || !l.a_out || !l.rot_inv_freq_f32 || (l.a_q_rank > 0 && (!l.a_uq || !l.a_q_norm_f32)))
                return fail("latent attention layer: missing weights");
            if (l.a_q_rank < 0 || l.a_window < 0) return fail("latent attention layer: unsupported sizes");
        } else if (l.type == LCC_MIX_ATTENTION) {
            if (l.m_heads < 1 || l.m_kv_heads < 1 || l.m_heads % l.m_kv_heads || l.m_dim < 1 || l.m_vdim < 1 || l.m_rot_dims < 0 ||
                (l.m_rot_dims & 1) || l.m_rot_dims > l.m_dim || (l.m_value_keys && l.m_vdim != l.m_dim) || l.m_gate < LCC_GATE_NONE ||
                l.m_gate > LCC_GATE_CHANNEL)
                return fail("attention layer: unsupported sizes");
            if (!l.m_in || (!l.m_unit_norm && (!l.m_qnorm_f32 || !l.m_knorm_f32)) || !l.m_out || (l.m_rot_dims > 0 && !l.rot_inv_freq_f32))
                return fail("attention layer: missing weights");
            if (l.m_vmix_role < 0 || l.m_vmix_role > 2 || (l.m_vmix_role && l.m_value_keys)) return fail("attention layer: values are mixed across layers only when they are projected");
            if (l.m_vmix_role == 1) {
                if (vkeep_seen) return fail("attention layer: one layer keeps its values for the later ones");
                vkeep_seen = true; vkeep_cols = l.m_kv_heads * l.m_vdim;
            }
            if (l.m_vmix_role == 2 && (!vkeep_seen || vkeep_cols != l.m_kv_heads * l.m_vdim))
                return fail("attention layer: mixed values need an earlier layer that keeps values of the same shape");
        } else if (l.type == LCC_MIX_DELTA) {
            if (l.d_heads < 1 || l.d_kv_heads < 1 || l.d_heads % l.d_kv_heads || l.d_dim < 1 || l.d_dim > 512 || l.d_vdim < 1 || l.d_conv < 1 ||
                l.d_conv > 8 || l.d_rank_a < 1 || l.d_rank_g < 1)
                return fail("delta-rule layer: unsupported sizes");
            if (!l.d_in || !l.d_conv_w_f32 || !l.d_a_up || !l.d_dt_bias_f32 || !l.d_a_log_f32 || !l.d_g_up || !l.d_norm_f32 || !l.d_out)
                return fail("delta-rule layer: missing weights");
        } else {
            return fail("unknown mixer type");
        }
    }
    lcc_seq_model* m = new lcc_seq_model();
    m->ctx = ctx;
    m->d = *desc;
    m->layers.assign(desc->layers, desc->layers + desc->n_layers);
    m->d.layers = m->layers.data();
    const char* e = getenv("LIVECC_B200_SEQ_TC");
    m->use_tc = !(e && e[0] == '0');
    const char* f = getenv("LIVECC_B200_SEQ_FORK");
    if (!(f && f[0] == '0')) {
        if (cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            m->side = nullptr;      // no second stream: everything stays on the caller's
        }
    }
    return m;
}

void lcc_seq_model_destroy(lcc_seq_model* m) {
    if (!m) return;
    if (m->ev_fork) cudaEventDestroy(m->ev_fork);
    if (m->ev_join) cudaEventDestroy(m->ev_join);
    if (m->side) cudaStreamDestroy(m->side);
    delete m;
}

size_t lcc_seq_workspace_bytes(const lcc_seq_model* m, int max_tokens, int max_want) {
    return m ? make_layout(m, max_tokens, max_want).total : 0;
}

int lcc_seq_bind_workspace(lcc_seq_model* m, void* ws, size_t ws_bytes, int max_tokens, int max_want) {
    if (!m || !ws) return -1;
    if (ws_bytes < make_layout(m, max_tokens, max_want).total) LCC_FAIL(m->ctx, -2, "lcc_seq_bind_workspace: buffer too small");
    m->ws = (uint8_t*)ws; m->ws_bytes = ws_bytes; m->cap_tokens = max_tokens; m->cap_want = max_want;
    // the arrival counters at the head of the key-split area start at zero; every launch leaves them at zero
    const WsLayout L = make_layout(m, max_tokens, max_want);
    if (L.split_floats && cudaMemset(m->ws + L.split, 0, L.split_floats * 4) != cudaSuccess) LCC_FAIL(m->ctx, -100, "lcc_seq_bind_workspace: memset failed");
    return 0;
}

size_t lcc_seq_struct_bytes(int which) {
    return which == 0 ? sizeof(lcc_seq_layer) : (which == 1 ? sizeof(lcc_seq_model_desc) : (which == 2 ? sizeof(lcc_seq_entry) : 0));
}

int64_t lcc_seq_layer_state_floats(const lcc_seq_model* m, int layer) {
    if (!m || layer < 0 || layer >= (int)m->layers.size()) return -1;
    const lcc_seq_layer& l = m->layers[layer];
    const Dims z = dims_of(l);
    // in a block whose mixer sits behind a convolution over time, every layer's slot starts with that convolution's last inputs
    const int64_t canon = (m->d.block == LCC_BLOCK_BRANCHNORM && l.canon_w_f32) ? (int64_t)m->d.width * (m->d.canon_taps - 1) : 0;
    if (l.type == LCC_MIX_SSD) return canon + (int64_t)z.conv_ch * (l.s_conv - 1) + (int64_t)l.s_heads * l.s_vdim * l.s_state;
    if (l.type == LCC_MIX_RETENTION) return canon + (int64_t)l.t_heads * l.t_vdim * l.t_dim;
    if (l.type == LCC_MIX_LATENT || l.type == LCC_MIX_ATTENTION) return canon;
    if (l.type == LCC_MIX_DELTA) return canon + (int64_t)z.d_conv_ch * (l.d_conv - 1) + (int64_t)l.d_heads * l.d_vdim * l.d_dim;
    return canon + (int64_t)l.r_heads * l.r_vdim * l.r_dim;
}

int lcc_seq_forward(lcc_seq_model* m, const lcc_seq_entry* entries, int n_entries, int page_size, const int32_t* want_rows,
                    int n_want, float* logits, float* logits_copy, float* layer_dump, lcc_stream_t stream) {
    if (!m || !entries || n_entries < 1) return -1;
    if (!m->ws) LCC_FAIL(m->ctx, -3, "lcc_seq_forward: no workspace bound");
    int T = 0;
    for (int e = 0; e < n_entries; ++e) {
        if (entries[e].n_new < 1 || !entries[e].ids || !entries[e].layer_state) LCC_FAIL(m->ctx, -2, "lcc_seq_forward: bad entry %d", e);
        T += entries[e].n_new;
    }
    if (T > m->cap_tokens || n_want > m->cap_want) LCC_FAIL(m->ctx, -4, "lcc_seq_forward: %d rows / %d wanted exceed the bound workspace (%d / %d)", T, n_want, m->cap_tokens, m->cap_want);
    if (n_want > 0 && (!want_rows || !logits)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const lcc_seq_model_desc& d = m->d;
    const int dt = d.dtype, W = d.width;
    const size_t es = lcc::dt_size(dt);
    const WsLayout L = make_layout(m, m->cap_tokens, m->cap_want);
    uint8_t* ws = m->ws;
    float* x32 = (float*)(ws + L.x32);
    uint8_t* xa = ws + L.xa;
    uint8_t* proj = ws + L.proj; uint8_t* proj2 = ws + L.proj2; uint8_t* mid = ws + L.mid; uint8_t* mid2 = ws + L.mid2;
    float* y32 = (float*)(ws + L.y32); float* q32 = (float*)(ws + L.q32);
    float* f1 = (float*)(ws + L.f1); float* f2 = (float*)(ws + L.f2);
    uint8_t* o1 = ws + L.o1; uint8_t* o2 = ws + L.o2; uint8_t* xf = ws + L.xf;
    float* scan_ws = L.scan_floats ? (float*)(ws + L.scan) : nullptr;
    float* split_ws = L.split_floats ? (float*)(ws + L.split) : nullptr;
    const bool hc = d.block == LCC_BLOCK_PRENORM_HC, par = d.block == LCC_BLOCK_PARALLEL, bn = d.block == LCC_BLOCK_BRANCHNORM;
    const int NS = hc ? d.streams : 1;
    uint8_t* vkeep = ws + L.vkeep;
    // blocks normed on the sublayer's output: does layer i read the residual stream through a convolution over time?
    auto canon_of = [&](int i) { return bn && i < d.n_layers && m->layers[i].canon_w_f32 != nullptr; };
    // parallel blocks: the norm that opens layer i (none past the last layer)
    auto norm_of = [&](int i) {
        if (i >= d.n_layers) return lcc::NormSpec{d.norm_kind, nullptr, nullptr, 0.f, d.eps};
        const lcc_seq_layer& n = m->layers[i];
        return lcc::NormSpec{d.norm_kind, n.norm1_f32, n.norm1_bias_f32, n.norm1_alpha, d.eps};
    };
    float* xsum = (float*)(ws + L.xsum);
    // pre-norm blocks: the sublayer output that the next boundary kernel folds into the streams
    const float* pend_hc = nullptr;
    lcc::MoeCombine pend_mc{};      // set when that sublayer was a routed feed-forward: its combine runs inside the boundary
    bool pend_is_mc = false;
    // boundary between sublayers of a pre-norm block: fold the finished sublayer's output (o1) into the streams, read and
    // norm for the next one (next_hc / next_w; null at the end of the model), optionally emit the sum of the streams
    auto boundary = [&](const float* next_hc, const float* next_w, float* sum_out) -> int {
        const int rc = lcc::hyper_boundary(dt, x32, NS, (pend_hc && !pend_is_mc) ? ws + L.o1 : nullptr, W, pend_hc, next_hc, next_w, d.eps, xa,
                                           sum_out, T, W, s, (pend_hc && pend_is_mc) ? &pend_mc : nullptr);
        pend_hc = nullptr;
        pend_is_mc = false;
        return rc;
    };
    auto pos_of = [&](const lcc_seq_entry& e) {
        lcc::SeqPos p{e.past, nullptr, nullptr};
        if (e.scalars) { p.kv_len = e.scalars + LCC_SC_KV_LEN; p.finished = e.scalars + LCC_SC_FINISHED; }
        return p;
    };
    // ---- embedding + positions ----
    {
        int r0 = 0;
        for (int e = 0; e < n_entries; ++e) {
            const lcc_seq_entry& en = entries[e];
            STEP(lcc::embed_sinusoid(dt, en.ids, en.scalars ? en.scalars + LCC_SC_SEQ_LEN : nullptr, d.embed, d.vocab, d.embed_scale,
                                     d.inv_freq_f32, x32 + (size_t)r0 * W * NS, (hc || canon_of(0)) ? nullptr : xa + (size_t)r0 * W * es, en.n_new, W,
                                     pos_of(en), s, NS), "embedding");
            r0 += en.n_new;
        }
        if (par) STEP(lcc::residual_norm(dt, x32, nullptr, 0, nullptr, 0, nullptr, norm_of(0), xa, T, W, s), "first norm");
    }
    for (int li = 0; li < d.n_layers; ++li) {
        const lcc_seq_layer& l = m->layers[li];
        const Dims z = dims_of(l);
        const bool has_ff = l.ff > 0 || l.ff_kind == LCC_FF_MOE;
        // parallel block, few rows (every kernel latency-bound): the feed-forward depends on the normed row only and runs on
        // the second stream beside the mixer (inside a capture: two branches of the graph), joined before the residual sum
        const bool fork_ff = par && has_ff && m->side && T <= kForkMaxRows && (l.ff_kind == LCC_FF_MOE || l.ff_kind == LCC_FF_MLP);
        if (fork_ff && (cudaEventRecord(m->ev_fork, s) != cudaSuccess || cudaStreamWaitEvent(m->side, m->ev_fork, 0) != cudaSuccess))
            LCC_FAIL(m->ctx, -100, "stream fork failed");
        cudaStream_t fs = fork_ff ? m->side : s;
        if (hc) STEP(boundary(l.hc1_f32, l.norm1_f32, (layer_dump && li > 0) ? layer_dump + (size_t)(li - 1) * T * W : nullptr), "stream boundary");
        // what precedes the mixer's own state in the layer's slot
        const size_t st_off = canon_of(li) ? (size_t)W * (d.canon_taps - 1) : 0;
        if (canon_of(li)) {
            // the mixer reads x + conv(x): fp32 rows of the residual stream in, rows in the storage type out; the convolution's last
            // inputs are the head of the layer's state slot
            int r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                float* st = en.layer_state[li];
                if (!st && d.canon_taps > 1) LCC_FAIL(m->ctx, -2, "lcc_seq_forward: entry %d has no state for layer %d", e, li);
                STEP(lcc::causal_conv(dt, x32 + (size_t)r0 * W, W, xa + (size_t)r0 * W * es, W, l.canon_w_f32, nullptr, st, en.n_new, W,
                                      d.canon_taps, pos_of(en), s, lcc::ConvOpts{true, false, true}), "input convolution");
                r0 += en.n_new;
            }
        }
        if (l.type == LCC_MIX_DELTA) {
            // [q | k | v | beta | decay-down | gate-down] -> causal convolution + silu on q, k, v -> decay-up (fp32) -> the
            // recurrence's operands in fp32 (unit q and k, decays, beta) -> delta rule -> gate-up -> unit-rms heads x weight x
            // sigmoid(gate) -> out-proj
            const int ldp = z.d_proj, ldm = z.d_conv_ch, H = l.d_heads, HN = H * l.d_dim, ldv = ld8(z.d_nv);
            STEP(linear(m, xa, W, l.d_in, nullptr, proj, ldp, false, T, z.d_proj, W, s), "delta-rule in-proj");
            STEP(linear(m, proj + (size_t)z.d_a1 * es, ldp, l.d_a_up, nullptr, f1, HN, true, T, HN, l.d_rank_a, s), "decay projection");
            STEP(linear(m, proj + (size_t)z.d_g1 * es, ldp, l.d_g_up, nullptr, proj2, ldv, false, T, z.d_nv, l.d_rank_g, s), "gate projection");
            int r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                float* st = en.layer_state[li];
                if (!st) LCC_FAIL(m->ctx, -2, "lcc_seq_forward: entry %d has no state for layer %d", e, li);
                STEP(lcc::causal_conv(dt, proj + (size_t)r0 * ldp * es, ldp, mid + (size_t)r0 * ldm * es, ldm, l.d_conv_w_f32, nullptr, st + st_off,
                                      en.n_new, z.d_conv_ch, l.d_conv, pos_of(en), s, lcc::ConvOpts{false, true, false}), "causal convolution");
                r0 += en.n_new;
            }
            // unit q and k, k . q, fp32 values, decays and write strengths of all rows, head by head (operands in q32, decays in f2)
            lcc::DeltaPackArgs pa{mid, ldm, z.d_k, z.d_v, f1, l.d_dt_bias_f32, l.d_a_log_f32, proj + (size_t)z.d_b * es, ldp, q32, f2,
                                  T, H, l.d_kv_heads, l.d_dim, l.d_vdim, 1e-6f, 1.f / sqrtf((float)l.d_dim)};
            STEP(lcc::delta_pack(dt, pa, s), "delta-rule operands");
            r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                lcc::DeltaScanArgs a{};
                a.ops = q32; a.dec = f2; a.T = T; a.r0 = r0;
                a.state = en.layer_state[li] + st_off + (size_t)z.d_conv_ch * (l.d_conv - 1);
                a.y = y32 + (size_t)r0 * z.d_nv; a.ld_y = z.d_nv;
                a.S = en.n_new; a.H = H; a.G = l.d_kv_heads; a.N = l.d_dim; a.P = l.d_vdim;
                STEP(lcc::delta_scan(a, pos_of(en), s), "delta-rule recurrence");
                r0 += en.n_new;
            }
            STEP(lcc::gated_group_norm(dt, y32, z.d_nv, proj2, ldv, l.d_norm_f32, l.d_vdim, mid2, ldv, T, z.d_nv, l.d_vdim, 2, d.eps, s),
                 "head norm + gate");
            STEP(linear(m, mid2, ldv, l.d_out, nullptr, o1, W, false, T, W, z.d_nv, s), "delta-rule out-proj");
        } else if (l.type == LCC_MIX_RETENTION) {
            // [q | k | v | gate] -> rotary q, k (k scaled), everything that enters the recurrence packed as fp32 -> recurrence
            // with one constant decay per head -> unit-rms heads x silu(gate) -> out-proj
            const int ldp = ld8(z.t_proj), ldv = ld8(z.t_nv), H = l.t_heads;
            STEP(linear(m, xa, W, l.t_in, nullptr, proj, ldp, false, T, z.t_proj, W, s), "retention in-proj");
            int r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                float* st = en.layer_state[li];
                if (!st) LCC_FAIL(m->ctx, -2, "lcc_seq_forward: entry %d has no state for layer %d", e, li);
                st += st_off;
                const lcc::SeqPos pos = pos_of(en);
                float* pk = q32 + (size_t)r0 * z.t_pack;
                const lcc::RotarySegment seg[3] = {
                    {0, 0, H, l.t_dim, 0, l.t_rot_dims, 1.f},
                    {z.t_nk, z.t_nk, H, l.t_dim, 0, l.t_rot_dims, 1.f / sqrtf((float)l.t_dim)},
                    {2 * z.t_nk, 2 * z.t_nk, H, l.t_vdim, 0, 0, 1.f}};
                STEP(lcc::rotary_pack_f32(dt, proj + (size_t)r0 * ldp * es, ldp, pk, z.t_pack, seg, 3, l.rot_inv_freq_f32, l.rot_mag,
                                          l.t_log_decay_f32, f1 + (size_t)r0 * H, H, en.n_new, pos, s), "rotary positions");
                lcc::ScanArgs a{};
                a.dt = LCC_DT_F32;      // the packed operands are fp32 in both storage types
                a.k = pk + z.t_nk; a.ld_k = z.t_pack;
                a.c = pk; a.ld_c = z.t_pack;
                a.u = pk + 2 * z.t_nk; a.ld_u = z.t_pack;
                a.a = f1 + (size_t)r0 * H; a.vec_decay = 0;
                a.sc = nullptr; a.skip = nullptr; a.cs = 1.f;
                a.state = st;
                a.y = y32 + (size_t)r0 * z.t_nv; a.ld_y = z.t_nv;
                a.S = en.n_new; a.heads = H; a.heads_per_group = 1; a.N = l.t_dim; a.P = l.t_vdim;
                a.ws = scan_ws; a.ws_floats = L.scan_floats;
                STEP(lcc::gated_scan(a, pos, s), "retention recurrence");
                r0 += en.n_new;
            }
            STEP(lcc::gated_group_norm(dt, y32, z.t_nv, proj + (size_t)(2 * z.t_nk + z.t_nv) * es, ldp, l.t_norm_f32, l.t_vdim, mid2, ldv, T,
                                       z.t_nv, l.t_vdim, 0, d.eps, s), "head norm + gate");
            STEP(linear(m, mid2, ldv, l.t_out, nullptr, o1, W, false, T, W, z.t_nv, s), "retention out-proj");
        } else if (l.type == LCC_MIX_LATENT) {
            // [q | latent, key part | gate] -> cache append + rotary query part -> unrotated query part absorbed through
            // W_uk^T per head -> attention over the cache rows (one key/value head, values = the latent channels) ->
            // per-head W_uv -> out-proj
            const int ldp = ld8(z.a_proj), ldl = ld8(z.a_lat), ldo = ld8(z.a_o), H = l.a_heads, QH = l.a_dim + l.a_rot_dim;
            const int src = l.a_kv_from >= 0 ? l.a_kv_from : li;
            STEP(linear(m, xa, W, l.a_in, nullptr, proj, ldp, false, T, z.a_proj, W, s), "latent attention in-proj");
            // queries through a latent of their own: RMS norm of the projection's first block, then the up-projection to the heads
            const uint8_t* qsrc = proj; int ldq = ldp;
            if (l.a_q_rank > 0) {
                const int ldc = ld8(l.a_q_rank);
                STEP(lcc::slice_rmsnorm(dt, proj, ldp, l.a_q_norm_f32, d.eps, mid2, ldc, T, l.a_q_rank, s), "query latent norm");
                STEP(linear(m, mid2, ldc, l.a_uq, nullptr, proj2, ld8(z.a_nq), false, T, z.a_nq, l.a_q_rank, s), "query up-projection");
                qsrc = proj2; ldq = ld8(z.a_nq);
            }
            const bool own_q = l.a_q_rank > 0;
            const lcc::AttnOpts lo{l.a_window, l.a_sink_f32 == nullptr, false};
            int r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                if (!en.k_pages || !en.k_pages[src] || !en.page_table)
                    LCC_FAIL(m->ctx, -2, "lcc_seq_forward: entry %d has no pages for layer %d", e, src);
                STEP(lcc::latent_kv_append(dt, proj + ((size_t)r0 * ldp + (own_q ? z.a_qin : 0)) * es, ldp, l.a_kv_from < 0, l.a_latent_norm_f32, d.eps,
                                           l.rot_inv_freq_f32, l.rot_mag, q32 + (size_t)r0 * H * z.a_kd, en.k_pages[src], en.page_table,
                                           page_size, en.n_new, H, l.a_dim, l.a_rot_dim, l.a_rank, pos_of(en), s,
                                           own_q ? qsrc + (size_t)r0 * ldq * es : nullptr, ldq), "latent cache append");
                r0 += en.n_new;
            }
            STEP(linear_heads(m, qsrc, ldq, QH, l.a_uk_t, q32, H * z.a_kd, z.a_kd, true, H, T, l.a_rank, l.a_dim, s), "query absorption");
            r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                STEP(lcc::attn_masked(dt, q32 + (size_t)r0 * H * z.a_kd, en.k_pages[src], en.k_pages[src], en.page_table, page_size,
                                      l.a_gate ? proj + ((size_t)r0 * ldp + z.a_gate) * es : nullptr, ldp, mid + (size_t)r0 * ldl * es, ldl, en.n_new, H, 1,
                                      z.a_kd, l.a_rank, 0, l.a_scale, m->use_tc, pos_of(en), s, lo, l.a_sink_f32, z.a_kd, split_ws, L.split_floats,
                                      en.past + en.n_new), "latent attention");
                r0 += en.n_new;
            }
            STEP(linear_heads(m, mid, ldl, l.a_rank, l.a_uv, mid2, ldo, l.a_vdim, false, H, T, l.a_vdim, l.a_rank, s), "value up-projection");
            STEP(linear(m, mid2, ldo, l.a_out, nullptr, o1, W, false, T, W, z.a_o, s), "latent attention out-proj");
        } else if (l.type == LCC_MIX_ATTENTION) {
            // [q | k | (v) | gate] -> per-head q/k norm + rotary positions, k and the values (the key columns as projected, or
            // their own) into the pages -> attention inside the window -> sigmoid gate (in the attention kernel's store) -> out-proj
            const int ldp = ld8(z.m_proj), ldo = ld8(z.m_o);
            STEP(linear(m, xa, W, l.m_in, nullptr, proj, ldp, false, T, z.m_proj, W, s), "attention in-proj");
            const lcc::AttnOpts ao{l.m_window, !l.m_sink, l.m_gate == LCC_GATE_CHANNEL};
            int r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                if (!en.k_pages || !en.v_pages || !en.k_pages[li] || !en.v_pages[li] || !en.page_table)
                    LCC_FAIL(m->ctx, -2, "lcc_seq_forward: entry %d has no pages for layer %d", e, li);
                const lcc::SeqPos pos = pos_of(en);
                uint8_t* pr = proj + (size_t)r0 * ldp * es;
                float* q = q32 + (size_t)r0 * z.m_nq;
                // values mixed across layers: the first such layer keeps its rows as projected, later ones cache a blend with them
                const int ldk = ld8(z.m_nv);
                const lcc::AppendOpts apo{l.m_unit_norm != 0, l.m_temp_f32,
                                          l.m_vmix_role == 2 ? vkeep + (size_t)r0 * ldk * es : nullptr, ldk, l.m_vmix,
                                          l.m_vmix_role == 1 ? vkeep + (size_t)r0 * ldk * es : nullptr, ldk};
                STEP(lcc::qk_headnorm_rope_append(dt, pr, ldp, z.m_vcol, l.m_qnorm_f32, l.m_knorm_f32, d.eps, l.rot_inv_freq_f32, l.rot_mag,
                                                  l.m_rot_dims, l.m_rot_pairs, q, en.k_pages[li], en.v_pages[li], en.page_table, page_size,
                                                  en.n_new, l.m_heads, l.m_kv_heads, l.m_dim, l.m_vdim, pos, s, &apo), "q/k norm + rotary + cache append");
                STEP(lcc::attn_masked(dt, q, en.k_pages[li], en.v_pages[li], en.page_table, page_size,
                                      z.m_ngate ? pr + (size_t)z.m_gate * es : nullptr, ldp, mid + (size_t)r0 * ldo * es, ldo, en.n_new,
                                      l.m_heads, l.m_kv_heads, l.m_dim, l.m_vdim, l.m_chunk, l.m_scale, m->use_tc, pos, s, ao, nullptr, 0,
                                      split_ws, L.split_floats, en.past + en.n_new), "window attention");
                r0 += en.n_new;
            }
            STEP(linear(m, mid, ldo, l.m_out, nullptr, o1, W, false, T, W, z.m_o, s), "attention out-proj");
        } else if (l.type == LCC_MIX_SSD) {
            const int ldp = ld8(z.s_proj), ldm = ld8(z.conv_ch), GN = l.s_groups * l.s_state;
            STEP(linear(m, xa, W, l.s_in, nullptr, proj, ldp, false, T, z.s_proj, W, s), "state-space in-proj");
            STEP(lcc::ssm_step_decay(dt, proj + (size_t)(z.inner + z.conv_ch) * es, ldp, l.s_dt_bias_f32, l.s_a_log_f32, f1, f2, T,
                                     l.s_heads, s), "step sizes");
            int r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                float* st = en.layer_state[li];
                if (!st) LCC_FAIL(m->ctx, -2, "lcc_seq_forward: entry %d has no state for layer %d", e, li);
                st += st_off;
                const lcc::SeqPos pos = pos_of(en);
                uint8_t* pr = proj + (size_t)r0 * ldp * es;
                uint8_t* xbc = mid + (size_t)r0 * ldm * es;
                STEP(lcc::causal_conv_silu(dt, pr + (size_t)z.inner * es, ldp, xbc, ldm, l.s_conv_w_f32, l.s_conv_b_f32, st, en.n_new,
                                           z.conv_ch, l.s_conv, pos, s), "causal convolution");
                lcc::ScanArgs a{};
                a.dt = dt;
                a.k = xbc + (size_t)z.inner * es; a.ld_k = ldm;
                a.c = xbc + (size_t)(z.inner + GN) * es; a.ld_c = ldm;
                a.u = xbc; a.ld_u = ldm;
                a.a = f2 + (size_t)r0 * l.s_heads; a.vec_decay = 0;
                a.sc = f1 + (size_t)r0 * l.s_heads;
                a.skip = l.s_skip_f32; a.cs = 1.f;
                a.state = st + (size_t)z.conv_ch * (l.s_conv - 1);
                a.y = y32 + (size_t)r0 * z.inner; a.ld_y = z.inner;
                a.S = en.n_new; a.heads = l.s_heads; a.heads_per_group = l.s_heads / l.s_groups; a.N = l.s_state; a.P = l.s_vdim;
                a.ws = scan_ws; a.ws_floats = L.scan_floats;
                STEP(lcc::gated_scan(a, pos, s), "state-space recurrence");
                r0 += en.n_new;
            }
            const int ldi = ld8(z.inner);
            STEP(lcc::gated_group_norm(dt, y32, z.inner, proj, ldp, l.s_norm_f32, z.inner, mid2, ldi, T, z.inner,
                                       z.inner / l.s_norm_groups, 1, d.eps, s), "gated norm");
            STEP(linear(m, mid2, ldi, l.s_out, nullptr, o1, W, false, T, W, z.inner, s), "state-space out-proj");
        } else {
            // left: chunk-local attention with a sink
            const int ldl = ld8(z.l_proj), ldo = ld8(z.l_o);
            STEP(linear(m, xa, W, l.l_in, l.l_in_bias_f32, proj, ldl, false, T, z.l_proj, W, s, l.l_in_bias), "attention in-proj");
            int r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                if (!en.k_pages || !en.v_pages || !en.k_pages[li] || !en.v_pages[li] || !en.page_table)
                    LCC_FAIL(m->ctx, -2, "lcc_seq_forward: entry %d has no pages for layer %d", e, li);
                const lcc::SeqPos pos = pos_of(en);
                uint8_t* pr = proj + (size_t)r0 * ldl * es;
                float* q = q32 + (size_t)r0 * z.l_nq;
                STEP(lcc::qk_norm_kv_append(dt, pr, ldl, l.l_qnorm_f32, l.l_knorm_f32, d.eps, q, en.k_pages[li], en.v_pages[li],
                                            en.page_table, page_size, en.n_new, l.l_heads, l.l_kv_heads, l.l_dim, l.l_vdim, pos, s),
                     "q/k norm + cache append");
                STEP(lcc::attn_chunk_sink(dt, q, en.k_pages[li], en.v_pages[li], en.page_table, page_size,
                                          pr + (size_t)(z.l_nq + z.l_nk + z.l_nv) * es, ldl, mid + (size_t)r0 * ldo * es, ldo, en.n_new,
                                          l.l_heads, l.l_kv_heads, l.l_dim, l.l_vdim, l.l_chunk, l.l_scale, m->use_tc, pos, s, nullptr, 0, split_ws,
                                          L.split_floats, en.past + en.n_new), "chunk attention");
                r0 += en.n_new;
            }
            STEP(linear(m, mid, ldo, l.l_out, nullptr, o1, W, false, T, W, z.l_o, s), "attention out-proj");
            // right: gated linear attention
            const int ldr = ld8(z.r_proj), ldz = ld8(z.r_nk), ldv = ld8(z.r_nv);
            STEP(linear(m, xa, W, l.r_in, nullptr, proj, ldr, false, T, z.r_proj, W, s), "linear-attention in-proj");
            STEP(linear(m, proj + (size_t)(2 * z.r_nk + 2 * z.r_nv) * es, ldr, l.r_decay_up, l.r_decay_bias_f32, proj2, ldz, false, T, z.r_nk, l.r_rank, s), "decay projection");
            STEP(lcc::gla_decay(dt, proj2, ldz, nullptr, l.r_tau, f1, T, z.r_nk, s), "decays");
            r0 = 0;
            for (int e = 0; e < n_entries; ++e) {
                const lcc_seq_entry& en = entries[e];
                float* st = en.layer_state[li];
                if (!st) LCC_FAIL(m->ctx, -2, "lcc_seq_forward: entry %d has no state for layer %d", e, li);
                uint8_t* pr = proj + (size_t)r0 * ldr * es;
                lcc::ScanArgs a{};
                a.dt = dt;
                a.k = pr + (size_t)z.r_nk * es; a.ld_k = ldr;
                a.c = pr; a.ld_c = ldr;
                a.u = pr + (size_t)(2 * z.r_nk) * es; a.ld_u = ldr;
                a.a = f1 + (size_t)r0 * z.r_nk; a.vec_decay = 1;
                a.sc = nullptr; a.skip = nullptr; a.cs = 1.f / sqrtf((float)l.r_dim);
                a.state = st;
                a.y = y32 + (size_t)r0 * z.r_nv; a.ld_y = z.r_nv;
                a.S = en.n_new; a.heads = l.r_heads; a.heads_per_group = 1; a.N = l.r_dim; a.P = l.r_vdim;
                a.ws = scan_ws; a.ws_floats = L.scan_floats;
                STEP(lcc::gated_scan(a, pos_of(en), s), "linear-attention recurrence");
                r0 += en.n_new;
            }
            STEP(lcc::gated_group_norm(dt, y32, z.r_nv, proj + (size_t)(2 * z.r_nk + z.r_nv) * es, ldr, l.r_norm_f32, l.r_vdim, mid2, ldv, T,
                                       z.r_nv, l.r_vdim, 0, d.eps, s), "head norm + gate");
            STEP(linear(m, mid2, ldv, l.r_out, nullptr, o2, W, false, T, W, z.r_nv, s), "linear-attention out-proj");
            STEP(lcc::postnorm_residual(dt, x32, xa, o1, W, l.l_branch_norm_f32, o2, W, l.r_branch_norm_f32, l.norm1_f32, d.alpha, d.eps,
                                        T, W, s), "branch merge + norm1");
        }
        // ---- the mixer's output is in o1 ----
        if (hc) pend_hc = l.hc1_f32;
        else if (par) {}   // the feed-forward reads the same normed row; the residual sum closes the layer
        else if (bn)       // x <- x + norm1(mixer); the feed-forward (or a next layer without a convolution) reads the new row
            STEP(lcc::branch_norm_residual(dt, x32, o1, W, nullptr, l.norm1_f32, d.eps, (has_ff || (li + 1 < d.n_layers && !canon_of(li + 1))) ? xa : nullptr,
                                           T, W, s), "norm1 + residual");
        else if (l.type != LCC_MIX_PARALLEL)
            STEP(lcc::postnorm_residual(dt, x32, xa, o1, W, nullptr, nullptr, 0, nullptr, l.norm1_f32, d.alpha, d.eps, T, W, s), "norm1");
        if (has_ff && hc) STEP(boundary(l.hc2_f32, l.norm2_f32, nullptr), "stream boundary");
        lcc::MoeCombine par_mc{};       // parallel block and output-normed block: the routed feed-forward's row is formed by the layer's residual kernel
        bool par_is_mc = false;
        if (l.ff_kind == LCC_FF_MOE) {
            // E real experts own row lists; the router has EO = E + identity outputs
            const bool glu = l.e_act == LCC_EXPERT_CLAMP_GLU || l.e_act == LCC_EXPERT_SILU_GLU;
            // the gated activation g * sigmoid(alpha g) * (u + up_bias) with its clamp: the plain silu form has no clamp
            const bool silu_glu = l.e_act == LCC_EXPERT_SILU_GLU;
            const float glu_limit = silu_glu ? INFINITY : l.e_limit, glu_alpha = silu_glu ? 1.f : 1.702f, glu_up_bias = silu_glu ? 0.f : 1.f;
            const int E = l.e_experts, EO = E + l.e_identity, K = l.e_top, lde = ld8(EO + 1), NH = glu ? 2 * l.e_ff : l.e_ff, ldh = ld8(NH),
                      ldg = ld8(l.e_ff), ldw8 = ld8(W), lds = ld8(l.e_shared_ff);
            const lcc::MoeRouterOpts ro{l.e_router_kind == LCC_ROUTER_SOFTMAX, l.e_identity, l.e_groups, l.e_keep, l.e_router_kind == LCC_ROUTER_TOPK_SOFTMAX};
            const int up_act = glu ? lcc::ACT_NONE : lcc::ACT_RELU2;
            float* mf = (float*)(ws + L.moe_f);
            float* logit = mf; float* wsel = mf + (size_t)T * lde; float* sgate = wsel + (size_t)T * K;
            int* mi = (int*)(ws + L.moe_i);
            int* sel = mi; int* rank = sel + (size_t)T * K; int* posn = rank + (size_t)T * K; int* src_row = posn + (size_t)T * K;
            int* tile_group = src_row + L.moe_rows; int* counts = tile_group + L.moe_rows / kMoeTile + 1; int* row_off = counts + E;
            uint8_t* ex = ws + L.moe_x; uint8_t* eh = ws + L.moe_h; uint8_t* eg = ws + L.moe_g; uint8_t* eo = ws + L.moe_o;
            const bool shared = l.e_shared_ff > 0, ident = l.e_identity > 0;
            float* gate_out = (shared || ident) ? sgate : nullptr;   // the shared expert's gate, or the chosen identity experts' weights
            // experts on the tensor cores: bf16, enough routed rows, 8-aligned shapes; lists are then padded to whole tiles
            const bool tc = m->use_tc && dt == LCC_DT_BF16 && T * K >= kMoeTcMinRows && (W % 8) == 0 && (l.e_ff % 8) == 0 && W >= 64 && l.e_ff >= 64;
            const int rows_max = T * K + E * (kMoeTile - 1), n_tiles = (rows_max + kMoeTile - 1) / kMoeTile;
            // the shared expert depends on the normed row only: in few-row steps, where every kernel is latency-bound, it runs on
            // the second stream beside the router and the routed experts
            const bool fork = shared && m->side && T <= kForkMaxRows && !fork_ff;
            if (fork && (cudaEventRecord(m->ev_fork, fs) != cudaSuccess || cudaStreamWaitEvent(m->side, m->ev_fork, 0) != cudaSuccess))
                LCC_FAIL(m->ctx, -100, "stream fork failed");
            if (shared) {
                cudaStream_t ss = fork ? m->side : fs;
                STEP(linear(m, xa, W, l.e_shared_up, nullptr, mid2, lds, false, T, l.e_shared_ff, W, ss, nullptr, lcc::ACT_RELU2), "shared expert up");
                STEP(linear(m, mid2, lds, l.e_shared_down, nullptr, o2, W, false, T, W, l.e_shared_ff, ss), "shared expert down");
            }
            // router logits (and the shared expert's gate logit) accumulate in fp32 from the normed row
            STEP(linear(m, xa, W, l.e_router, nullptr, logit, lde, true, T, EO + (shared ? 1 : 0), W, fs), "router");
            if (!tc && T * K <= 256 && EO <= 512) {
                STEP(lcc::moe_route_small(logit, lde, l.e_correction_f32, EO, K, l.e_scale, sel, wsel, gate_out, row_off, posn,
                                          src_row, T, fs, &ro), "expert choice + row lists");
            } else {
                if (cudaMemsetAsync(counts, 0, sizeof(int) * E, fs) != cudaSuccess) LCC_FAIL(m->ctx, -100, "router counters");
                if (tc && cudaMemsetAsync(src_row, 0xff, sizeof(int) * (size_t)n_tiles * kMoeTile, fs) != cudaSuccess) LCC_FAIL(m->ctx, -100, "row lists");
                STEP(lcc::moe_route(logit, lde, l.e_correction_f32, EO, K, l.e_scale, sel, wsel, gate_out, counts, rank, T, fs, &ro), "expert choice");
                STEP(lcc::moe_index(sel, rank, counts, E, K, tc ? kMoeTile : 1, row_off, posn, src_row, tc ? tile_group : nullptr, n_tiles, T, fs), "expert row lists");
            }
            if (tc) {
                STEP(lcc::moe_gather_rows(dt, xa, W, src_row, ex, ldw8, n_tiles * kMoeTile, W, fs), "expert row gather");
                lcc::GemmArgs a;
                // gated experts with interleaved rows: the activation is the up product's epilogue and the hidden rows land in eg
                const bool epi_glu = glu && l.e_up_il16;
                a.A = ex; a.B = l.e_up; a.C = epi_glu ? eg : eh; a.M = n_tiles * kMoeTile; a.N = NH; a.K = W; a.lda = ldw8; a.ldb = W;
                a.ldc = epi_glu ? ldg : ldh;
                a.bias = nullptr; a.residual = nullptr; a.ldr = 0; a.block_n = 0;
                a.epi = epi_glu ? lcc::EPI_CLAMP_GLU : (glu ? lcc::EPI_NONE : lcc::EPI_RELU2);
                a.epi_param = glu_limit; a.epi_alpha = glu_alpha; a.epi_up_bias = glu_up_bias;
                a.tile_group = tile_group; a.groups = E;
                STEP(lcc::gemm_bf16_tn(a, m->ctx->num_sms, fs), "experts up");
                if (glu && !epi_glu) STEP(lcc::glu_clamp_swish(dt, eh, ldh, eg, ldg, n_tiles * kMoeTile, l.e_ff, glu_limit, fs, false, glu_alpha, glu_up_bias), "expert activation");
                a.A = glu ? eg : eh; a.B = l.e_down; a.C = eo; a.N = W; a.K = l.e_ff; a.lda = glu ? ldg : ldh; a.ldb = l.e_ff; a.ldc = ldw8; a.epi = lcc::EPI_NONE;
                STEP(lcc::gemm_bf16_tn(a, m->ctx->num_sms, fs), "experts down");
            } else {
                lcc::GroupedLinear g{};
                g.dt = dt; g.A = xa; g.lda = W; g.a_stride = 0; g.a_rows = src_row; g.row_off = row_off; g.M_total = T * K;
                g.W = l.e_up; g.ldw = W; g.w_stride = (int64_t)NH * W;
                g.C = glu ? eg : eh; g.ldc = glu ? ldg : ldh; g.c_stride = 0; g.c_f32 = false;
                g.groups = E; g.M = T; g.N = l.e_ff; g.K = W; g.act = up_act;
                if (glu) {
                    g.glu_F = l.e_ff; g.glu_il16 = l.e_up_il16 != 0; g.glu_limit = glu_limit; g.glu_tmp = eh; g.ld_tmp = ldh;
                    g.glu_alpha = glu_alpha; g.glu_up_bias = glu_up_bias;
                }
                STEP(lcc::linear_grouped(g, fs), "experts up");
                g.glu_F = 0; g.glu_tmp = nullptr;
                g.A = glu ? eg : eh; g.lda = glu ? ldg : ldh; g.a_rows = nullptr;
                g.W = l.e_down; g.ldw = l.e_ff; g.w_stride = (int64_t)W * l.e_ff;
                g.C = eo; g.ldc = ldw8; g.N = W; g.K = l.e_ff; g.act = lcc::ACT_NONE;
                STEP(lcc::linear_grouped(g, fs), "experts down");
            }
            if (fork && (cudaEventRecord(m->ev_join, m->side) != cudaSuccess || cudaStreamWaitEvent(fs, m->ev_join, 0) != cudaSuccess))
                LCC_FAIL(m->ctx, -100, "stream join failed");
            if (hc) {   // the weighted sum of the experts' rows is formed by the boundary kernel that folds it into the streams
                pend_mc = lcc::MoeCombine{eo, ldw8, posn, wsel, K, shared ? o2 : nullptr, W, sgate};
                pend_is_mc = true;
            } else if (par || bn) {   // ... or by the residual kernel that closes the layer; identity experts return the normed row
                par_mc = lcc::MoeCombine{eo, ldw8, posn, wsel, K, shared ? (const void*)o2 : (ident ? (const void*)xa : nullptr), W, sgate};
                par_is_mc = true;
            } else {
                STEP(lcc::moe_combine(dt, eo, ldw8, posn, wsel, K, shared ? o2 : nullptr, W, sgate, o1, W, T, W, fs), "expert combine");
            }
        } else if (l.ff > 0 && l.ff_kind == LCC_FF_MLP) {
            const int ldf = ld8(l.ff);
            // (its hidden rows in mid2: in a parallel block the mixer's rows in mid may still be in use on the other stream)
            STEP(linear(m, xa, W, l.ff_in, nullptr, mid2, ldf, false, T, l.ff, W, fs, nullptr, lcc::ACT_GELU_TANH), "feed-forward up + gelu");
            STEP(linear(m, mid2, ldf, l.ff_out, nullptr, par ? o2 : o1, W, false, T, W, l.ff, fs), "feed-forward down");
        } else if (l.ff > 0) {
            const int ldg = ld8(2 * l.ff), ldf = ld8(l.ff);
            STEP(linear(m, xa, W, l.ff_in, nullptr, proj, ldg, false, T, 2 * l.ff, W, fs), "feed-forward in");
            STEP(lcc::glu_gelu_tanh(dt, proj, ldg, mid, ldf, T, l.ff, fs), "gated gelu");
            STEP(linear(m, mid, ldf, l.ff_out, nullptr, par ? o2 : o1, W, false, T, W, l.ff, fs), "feed-forward out");
        }
        if (fork_ff && (cudaEventRecord(m->ev_join, m->side) != cudaSuccess || cudaStreamWaitEvent(s, m->ev_join, 0) != cudaSuccess))
            LCC_FAIL(m->ctx, -100, "stream join failed");
        if (par) {
            // x <- x + (mixer + feed-forward), then the next layer's norm of the new row
            STEP(lcc::residual_norm(dt, x32, o1, W, (has_ff && !par_is_mc) ? o2 : nullptr, W, par_is_mc ? &par_mc : nullptr, norm_of(li + 1),
                                    xa, T, W, s), "residual sum + next norm");
        } else if (has_ff && bn) {
            // x <- x + norm2(feed-forward); a next layer without a convolution in front of its mixer reads the new row
            STEP(lcc::branch_norm_residual(dt, x32, par_is_mc ? nullptr : o1, W, par_is_mc ? &par_mc : nullptr, l.norm2_f32, d.eps,
                                           (li + 1 < d.n_layers && !canon_of(li + 1)) ? xa : nullptr, T, W, s), "norm2 + residual");
        } else if (has_ff) {
            if (hc) pend_hc = l.hc2_f32;
            else STEP(lcc::postnorm_residual(dt, x32, xa, o1, W, nullptr, nullptr, 0, nullptr, l.norm2_f32, d.alpha, d.eps, T, W, s), "norm2");
        }
        if (layer_dump && !hc) {
            if (cudaMemcpyAsync(layer_dump + (size_t)li * T * W, x32, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
                LCC_FAIL(m->ctx, -100, "layer dump copy failed");
        }
    }
    if (hc) {
        STEP(boundary(nullptr, nullptr, xsum), "stream sum");
        if (layer_dump && cudaMemcpyAsync(layer_dump + (size_t)(d.n_layers - 1) * T * W, xsum, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
            LCC_FAIL(m->ctx, -100, "layer dump copy failed");
    }
    if (n_want > 0) {
        const lcc::NormSpec fn{d.norm_kind, d.final_norm_f32, d.final_norm_bias_f32, d.final_norm_alpha, d.eps};
        STEP(lcc::gather_norm(dt, hc ? xsum : x32, want_rows, fn, xf, n_want, W, s), "final norm");
        STEP(lcc::linear_any(dt, xf, W, d.head, W, nullptr, logits, d.vocab, true, n_want, d.vocab, W, s), "output head");
        STEP(lcc::softcap(logits, (int64_t)n_want * d.vocab, d.logit_softcap, s, d.logit_scale != 0.f ? d.logit_scale : 1.f), "logit soft cap / scale");
        if (logits_copy &&
            cudaMemcpyAsync(logits_copy, logits, (size_t)n_want * d.vocab * 4, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
            LCC_FAIL(m->ctx, -100, "logits copy failed");
    }
    LCC_CHECK_LAUNCH(m->ctx, "lcc_seq_forward");
    return 0;
}

}  // extern "C"
