// Internal launch interfaces of the sequence-mixing ops used by the hybrid decoder models (state-space layers, gated
// linear attention, chunk-local attention with a softmax sink, post-norm residual blocks):
//   linear_any.cu   general-shape linear layers (any M, N, K; bf16 or fp32 storage, fp32 accumulation)
//   recurrent.cu    short causal convolution with carried inputs, gated linear recurrences and the gated delta rule with carried fp32 state
//   attn_local.cu   whole-projection q/k norm + paged K/V append, chunk-local attention with a sink term
//   rowops.cu       embedding + sinusoidal positions, post-norm / parallel / output-normed residual rows, grouped gated RMS norm, GLU, soft cap
//   rotary.cu       rotate-half rotary positions on slices of a projection, packed to fp32 for a recurrence
//   attn_latent.cu  latent (low-rank) K/V cache: latent norm + shared rotary key part -> pages, rotary query part
//   hyper.cu        pre-norm blocks on several residual streams (hyper-connections)
//   moe.cu          sigmoid, softmax or chosen-logit-softmax top-k router (groups of experts, identity experts), expert row lists, weighted combine
// Every op exists for two storage types (DT_BF16: bf16 storage, fp32 arithmetic where the model asks for it;
// DT_F32: everything fp32). All return 0 on success, negative on invalid arguments; launches are asynchronous on `s`.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lcc {

enum { DT_BF16 = 0, DT_F32 = 1 };
inline size_t dt_size(int dt) { return dt == DT_F32 ? 4 : 2; }

// A sequence position source: `past` tokens precede row 0 of this call. When `kv_len` is non-null the kernels read
// past = *kv_len from the device instead (CUDA-graph replay of decode steps), and do nothing when `*finished` is set.
struct SeqPos {
    int past;
    const int* kv_len;
    const int* finished;
};

// The row a routed feed-forward contributes, formed inside the kernel that consumes it (hyper_boundary, residual_norm):
//   y[r] = sum_k weight[r, k] * eo[pos[r, k]] + gate[r] * so[r]   (fp32; choices with pos < 0 are skipped)
struct MoeCombine {
    const void* eo; int ld_eo; const int* pos; const float* weight; int top;
    const void* so; int ld_so; const float* gate;      // so null: no shared expert
};

// ---- linear_any.cu ------------------------------------------------------------------------------------------------------
// C[M,N] = A[M,K] x W[N,K]^T (+ bias[N], fp32). A and W have storage type dt; C has storage type dt, or fp32 when
// c_f32. Any M, N, K >= 1; leading dimensions in elements.
int linear_any(int dt, const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, bool c_f32,
               int M, int N, int K, cudaStream_t s);

// The same product for `groups` independent problems in one launch (per-head projections, routed experts). Group z reads
// A + z * a_stride, W + z * w_stride and writes C + z * c_stride (strides in elements). Without row_off every group has M
// rows. With row_off (device int32[groups + 1]) group z owns rows row_off[z] .. row_off[z+1]-1 of A and C, M is an upper
// bound of any group's row count and M_total of their sum; a_rows (optional, device int32) then names the row of A that
// feeds each of those rows (a gather), while C rows stay in list order. act: 0 none, 1 relu(x)^2 before the store.
struct GroupedLinear {
    int dt;
    const void* A; int lda; int64_t a_stride;
    const void* W; int ldw; int64_t w_stride;
    void* C; int ldc; int64_t c_stride; bool c_f32;
    int groups, M, N, K;
    const int* row_off; const int* a_rows; int M_total;
    int act;
    // Gated experts (glu_F > 0): W holds 2 * glu_F rows per group, gate and up rows either [gate: F | up: F] or, with glu_il16,
    // interleaved in groups of 16 (16 gate rows, then the 16 matching up rows); N = glu_F and C receives
    // g * sigmoid(1.702 g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit). The few-row kernel forms it in its
    // store; the tile kernel writes the 2 * glu_F raw columns to glu_tmp (leading dimension ld_tmp, storage dt, the rows of C)
    // and a row kernel follows.
    int glu_F; bool glu_il16; float glu_limit; void* glu_tmp; int ld_tmp;
    // the general gated activation g * sigmoid(alpha g) * (u + up_bias) with g = min(gate, limit), u = clamp(up, -limit, limit):
    // the defaults are the clamped form above; alpha 1, up_bias 0 and an infinite limit give silu(gate) * up
    float glu_alpha = 1.702f, glu_up_bias = 1.f;
};
enum { ACT_NONE = 0, ACT_RELU2 = 1, ACT_GELU_TANH = 2 };   // 2: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
int linear_grouped(const GroupedLinear& g, cudaStream_t s);

// ---- recurrent.cu -------------------------------------------------------------------------------------------------------
// Causal per-channel convolution over `taps` inputs followed by silu. in/out: [S, C] slices (storage dt, leading
// dimensions ld_in / ld_out); w: fp32 [C, taps] (last column multiplies the current token); b: fp32 [C];
// carry: fp32 [C, taps-1] = the last taps-1 inputs before row 0 (zeros at the start of a sequence), updated to the last
// taps-1 inputs of this call.
int causal_conv_silu(int dt, const void* in, int ld_in, void* out, int ld_out, const float* w, const float* b,
                     float* carry, int S, int C, int taps, SeqPos pos, cudaStream_t s);
// The same convolution with its parts as options: in_f32: `in` is fp32 whatever dt says (a residual stream); silu: the
// activation; add_input: out = in + conv(in) (a convolution on a skip path). b may be null (no bias). out has storage dt.
struct ConvOpts { bool in_f32; bool silu; bool add_input; };
int causal_conv(int dt, const void* in, int ld_in, void* out, int ld_out, const float* w, const float* b, float* carry,
                int S, int C, int taps, SeqPos pos, cudaStream_t s, const ConvOpts& opt);

// Step sizes and log decays of a scalar-decay state-space layer: dt = softplus(raw + dt_bias[h]),
// log decay = -exp(a_log[h]) * dt. raw: [S, heads] slice (storage dt, leading dimension ld); dt_out / decay_out: fp32 [S, heads].
int ssm_step_decay(int dt, const void* raw, int ld, const float* dt_bias, const float* a_log, float* dt_out,
                   float* decay_out, int S, int heads, cudaStream_t s);
// Per-channel log decays of gated linear attention: log(sigmoid(z + bias)) / tau; z: [S, n] slice (storage dt).
int gla_decay(int dt, const void* z, int ld, const float* bias, float tau, float* decay_out, int S, int n,
              cudaStream_t s);
// Gated delta rule with a decay per head and key channel, one state matrix St[n, p] per head (H value heads of P channels over
// G key heads of N channels, head h reads key head h / (H / G)):
//     St <- diag(d_t) St;  w = beta_t (v_t - St^T k_t);  St <- St + k_t w^T;  y_t = St^T q_t
// in two steps. delta_pack prepares all S rows of a step at once: qkv [S, ld] (storage dt) holds q at column 0, k at col_k and
// v at col_v; k and q are divided by sqrt(sum(x^2) + unit_eps) per key head (unit_eps <= 0: left as they are), q also times
// q_scale. The prepared operands are fp32 and laid out head by head (the rows of one head contiguous):
//     out: k [G][S][N] | q [G][S][N] | v [H][S][P] | k . q [G][S] | beta [H][S]   (every block padded to a multiple of 4 floats)
//     dec: [H][S][N] = exp(-exp(a_log[h]) * softplus(z + dt_bias[h*N + n])), z: fp32 [S, H*N]
// beta = sigmoid(b), b: [S, H] slice (storage dt).
struct DeltaOperands { float *k, *q, *v, *kq, *beta; };
__host__ __device__ inline size_t delta_pad4(size_t n) { return (n + 3) / 4 * 4; }
__host__ __device__ inline DeltaOperands delta_operands(float* base, int S, int H, int G, int N, int P) {
    DeltaOperands o;
    o.k = base;
    o.q = o.k + delta_pad4((size_t)G * S * N);
    o.v = o.q + delta_pad4((size_t)G * S * N);
    o.kq = o.v + delta_pad4((size_t)H * S * P);
    o.beta = o.kq + delta_pad4((size_t)G * S);
    return o;
}
inline size_t delta_operand_floats(int S, int H, int G, int N, int P) {
    return 2 * delta_pad4((size_t)G * S * N) + delta_pad4((size_t)H * S * P) + delta_pad4((size_t)G * S) + delta_pad4((size_t)H * S);
}
struct DeltaPackArgs {
    const void* qkv; int ld, col_k, col_v;
    const float* z; const float* dt_bias; const float* a_log;
    const void* b; int ld_b;
    float* out; float* dec;
    int S, H, G, N, P;
    float unit_eps, q_scale;
};
int delta_pack(int dt, const DeltaPackArgs& a, cudaStream_t s);
// delta_scan runs the recurrence token by token over one sequence's S rows (prompt portions and decode steps alike): rows
// r0 .. r0 + S - 1 of the T rows that delta_pack prepared (ops = its `out`). state: fp32 [H, P, N] (n fastest), read at the start
// and written back at the end; y: fp32 [S, H*P]. TT and async are chosen by the launcher.
struct DeltaScanArgs {
    const float* ops; const float* dec;
    int T, r0;
    float* state; float* y; int ld_y;
    int S, H, G, N, P;
    int TT; bool async;
};
int delta_scan(const DeltaScanArgs& a, SeqPos pos, cudaStream_t s);

// Gated linear recurrence, one state matrix St[n, p] (n < N key channels, p < P value channels) per head:
//     St <- diag(a_t) St + k_t (sc_t * u_t)^T ,   y_t = St^T (cs * c_t) + skip[h] * u_t
// k, c: [S, *] slices with head-group stride (head h reads columns (h / heads_per_group) * N + n); u: [S, heads*P] slice;
// a: fp32 log decays (log a_t <= 0), either [S, heads] (vec_decay = 0) or [S, heads*N]; sc: fp32 [S, heads] or null (= 1);
// skip: fp32 [heads] or null. state: fp32 [heads, P, N] (n fastest), read at the start and written back at the end.
// y: fp32 [S, heads*P]. Two forms compute it: a token-by-token kernel (decode steps and short portions), and, for portions
// of kScanChunkedMin rows or more when a workspace is given, a sequence-parallel form over blocks of 64 rows
// (recurrent_chunked.cu), which overwrites `a` with block-local cumulative sums.
struct ScanArgs {
    int dt;
    const void* k; int ld_k;
    const void* c; int ld_c;
    const void* u; int ld_u;
    float* a; int vec_decay;
    const float* sc;
    const float* skip;
    float cs;
    float* state;
    float* y; int ld_y;
    int S, heads, heads_per_group, N, P;
    float* ws; size_t ws_floats;   // workspace of the sequence-parallel form (null: token by token)
};
constexpr int kScanChunkedMin = 32;     // rows from which the sequence-parallel form runs
constexpr int kScanMaxBlocks = 64;      // blocks of 64 rows per pass of the sequence-parallel form (bounds its workspace)
int gated_scan(const ScanArgs& a, SeqPos pos, cudaStream_t s);
int gated_scan_chunked(const ScanArgs& a, SeqPos pos, cudaStream_t s);
// fp32 elements of workspace that let a call of S rows run in the fewest passes
size_t gated_scan_ws_floats(int S, int heads, int N, int P);

// ---- attn_local.cu ------------------------------------------------------------------------------------------------------
// RMS norm of the whole q projection and of the whole k projection of each row (weights qn_w [Hq*D], kn_w [G*D], fp32),
// then: normalised q -> q_out fp32 [S, Hq*D]; normalised k and raw v -> the paged cache at positions past..past+S-1.
// proj: [S, ld] rows laid out [q: Hq*D | k: G*D | v: G*DV | ...] (storage dt). K pages: [page][G][page_size][D],
// V pages: [page][G][page_size][DV] (storage dt).
int qk_norm_kv_append(int dt, const void* proj, int ld, const float* qn_w, const float* kn_w, float eps, float* q_out,
                      void* k_pages, void* v_pages, const int* page_table, int page_size, int S, int Hq, int G, int D,
                      int DV, SeqPos pos, cudaStream_t s);
// Attention of S new rows over the cached keys of the same chunk: row at position i sees j <= i with
// floor(j / chunk) == floor(i / chunk); weights exp(s_j) / (1 + sum_j exp(s_j)) (a sink with score 0 and no value);
// head h's output is multiplied by sigmoid(gate[h]). q: fp32 [S, Hq*D]; gate: [S, Hq] slice (storage dt, leading dim
// ld_gate) or null; out: [S, Hq*DV] (storage dt). chunk <= 0 means one chunk (plain causal attention).
// Three kernels: one CTA per (row, head) for decode steps and portions of fewer than kAttnTiledMin rows; a tiled fp32
// CUDA-core kernel for longer portions; and, for bf16 storage with head size <= kAttnMmaMaxDim when tensor_cores is set,
// the same tiling with both products on the tensor cores (bf16 operands, fp32 accumulation, fp32 softmax).
constexpr int kAttnTiledMin = 16;
constexpr int kAttnMmaMaxDim = 256;
// sink: fp32 [Hq] sink logits (null: 0 for every head); the sink adds exp(sink[h]) to the denominator and nothing else.
// ld_v: elements between consecutive V rows of a (page, group); DV for V pages of their own, and the K row length when the
// values are the first DV channels of the key rows (v_pages = k_pages), as in a latent cache.
int attn_chunk_sink(int dt, const float* q, const void* k_pages, const void* v_pages, const int* page_table,
                    int page_size, const void* gate, int ld_gate, void* out, int ld_out, int S, int Hq, int G, int D,
                    int DV, int chunk, float scale, bool tensor_cores, SeqPos pos, cudaStream_t s,
                    const float* sink = nullptr, int ld_v = 0, float* split_ws = nullptr, size_t split_ws_floats = 0,
                    int key_hint = 0);
// split_ws (optional, fp32, zero-filled once by the owner; attn_split_ws_floats(rows, Hq, DV) elements let every call of
// up to `rows` rows use all its key splits): with it, calls of fewer than kAttnTiledMin rows of plain causal attention
// (chunk <= 0) over long windows, or windows whose length only the device knows, run one CTA per (row, head, key split)
// and merge the splits in the last CTA to arrive. key_hint: the host's estimate of the window (sets the number of splits
// only; any length is computed correctly).
size_t attn_split_ws_floats(int rows, int Hq, int DV);
// Further options of attn_chunk_sink (null: chunks only, a zero-logit sink, one gate per head). window > 0: a row at position
// i sees only j with i - j < window (inside its chunk, when there are chunks too). no_sink: ordinary softmax over the visible
// keys. gate_channel: the gate slice is [S, Hq*DV], one sigmoid gate per output element.
struct AttnOpts { int window; bool no_sink; bool gate_channel; };
// Options of qk_headnorm_rope_append (null: none). unit_norm: q and k heads are divided by their rms without a weight (qn_w, kn_w
// null; the rotation keeps every pair's length, so norming before it equals norming after it). q_head_scale: fp32 [Hq], one factor
// per query head on q_out (a temperature on the scores). v_mix: [S, ld_mix] slice (storage dt) of G*DV columns: the cached values
// are (1 - mix) * v + mix * v_mix in fp32. v_keep: [S, ld_keep] (storage dt) receives the values as projected.
struct AppendOpts { bool unit_norm; const float* q_head_scale; const void* v_mix; int ld_mix; float mix; void* v_keep; int ld_keep; };
int attn_masked(int dt, const float* q, const void* k_pages, const void* v_pages, const int* page_table, int page_size,
                const void* gate, int ld_gate, void* out, int ld_out, int S, int Hq, int G, int D, int DV, int chunk, float scale,
                bool tensor_cores, SeqPos pos, cudaStream_t s, const AttnOpts& opt, const float* sink = nullptr, int ld_v = 0,
                float* split_ws = nullptr, size_t split_ws_floats = 0, int key_hint = 0);
// Per-head RMS norm of q and k (weights qn_w, kn_w: fp32 [D], shared by the heads), then rotary positions on the first
// rot_dims channels of every q and k head (rot_pairs: channel 2i turns with 2i+1, else i with i + rot_dims/2; angle =
// position * inv_freq[i] in fp32, cos and sin times mag), then: q -> q_out fp32 [S, Hq*D]; k -> K pages; the values -> V
// pages, read from columns [v_col, v_col + G*DV) of the row as projected (v_col = Hq*D: the values are the un-normed,
// unrotated keys). proj: [S, ld] rows laid out [q: Hq*D | k: G*D | ...] (storage dt). Page layout as qk_norm_kv_append.
int qk_headnorm_rope_append(int dt, const void* proj, int ld, int v_col, const float* qn_w, const float* kn_w, float eps,
                            const float* inv_freq, float mag, int rot_dims, int rot_pairs, float* q_out, void* k_pages,
                            void* v_pages, const int* page_table, int page_size, int S, int Hq, int G, int D, int DV, SeqPos pos,
                            cudaStream_t s, const AppendOpts* opt = nullptr);

// ---- rotary.cu ----------------------------------------------------------------------------------------------------------
// Rotary positions in the rotate-half layout: inside a head, channel i < dims/2 of the rotated block pairs with channel
// i + dims/2; the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a) * mag, a = p * inv_freq[i]
// (fp32 position, angle, cos and sin). A segment is `heads` heads of `dim` channels starting at column `col_in` of a row
// of `in` (storage dt); the rotated block is channels [rot_off, rot_off + rot_dims) of each head, the rest pass; every
// output is multiplied by `scale` and written as fp32 at column col_out of `out` with the same head layout.
struct RotarySegment { int col_in, col_out, heads, dim, rot_off, rot_dims; float scale; };
// Up to 4 segments of one row in one launch. fill: optional fp32 [fill_n] row that is copied to fill_out [S, fill_n] for
// every row (per-head constants a recurrence wants per token, e.g. log decays).
int rotary_pack_f32(int dt, const void* in, int ld_in, float* out, int ld_out, const RotarySegment* seg, int n_seg,
                    const float* inv_freq, float mag, const float* fill, float* fill_out, int fill_n, int S, SeqPos pos,
                    cudaStream_t s);

// ---- attn_latent.cu -----------------------------------------------------------------------------------------------------
// Rows of `proj` (storage dt) are laid out [q: H x (D + DR) | latent: R, key part: DR | ...]; has_kv = 0: no middle block.
// With has_kv: c = rms(latent) * norm_w (fp32) and the rotated key part go to the K pages [page][1][page_size][R + DR]
// at positions past .. past+S-1. Always: the rotated part of each head's query goes to q_out fp32 [S, H, R + DR] at
// channels R .. R+DR-1 (channels 0 .. R-1 are left for the absorbed unrotated part: W_uk_h^T q_h).
// q (optional): the query heads [S, ld_q] (storage dt) when they are not the first columns of proj (queries that come through
// a latent of their own); proj then starts with the latent.
int latent_kv_append(int dt, const void* proj, int ld, int has_kv, const float* norm_w, float eps, const float* inv_freq,
                     float mag, float* q_out, void* k_pages, const int* page_table, int page_size, int S, int H, int D,
                     int DR, int R, SeqPos pos, cudaStream_t s, const void* q = nullptr, int ld_q = 0);

// ---- hyper.cu -----------------------------------------------------------------------------------------------------------
// One boundary between two sublayers of a pre-norm block on n residual streams xs fp32 [S, n, W]:
//   (1) if y: x_t <- sum_s mix[s * n + t] x_s + out[t] * y            (all streams at once from the old ones; y storage dt)
//   (2) if w:  u = sum_s in[s] x_s;  xa = u / sqrt(mean(u^2) + eps) * w   (storage dt; w is the full weight)
//   (3) if sum_out: sum_out = sum_s x_s  (fp32 [S, W])
// prev: fp32 [in: n | out: n | mix: n*n] of the sublayer that produced y; next: the same block of the sublayer that reads xa.
// mc (instead of y): the finished sublayer is a routed feed-forward whose output row is formed here,
//   y[r] = sum_k weight[r, k] * eo[pos[r, k]] + gate[r] * so[r]   (in fp32; moe_combine as part of the boundary).
int hyper_boundary(int dt, float* xs, int n, const void* y, int ld_y, const float* prev, const float* next, const float* w,
                   float eps, void* xa, float* sum_out, int S, int W, cudaStream_t s, const MoeCombine* mc = nullptr);

// ---- moe.cu -------------------------------------------------------------------------------------------------------------
// Router of a mixture of experts. logits fp32 [S, ld] (E expert logits, then optionally the shared expert's gate logit at
// column E). score = sigmoid(logit); the `top` experts with the largest score + correction[e] are chosen (ties: the lower
// index), weight = score * scale (no renormalisation). Outputs: sel int32 [S, top], weight fp32 [S, top],
// shared_gate fp32 [S] = sigmoid(logit[E]) (when shared_gate is non-null); counts int32 [E] must be zero on entry and
// receives the number of rows per expert; rank int32 [S, top] = the row's arrival number inside its expert.
// opt (null: a sigmoid score per expert, no identity experts, no groups): softmax: score = softmax over all E router outputs;
// identity: the last `identity` of the E outputs stand for experts that return their input: they enter no list (rank and pos
// are -1, counts / row_off cover the E - identity real experts) and the sum of their weights goes to shared_gate[r] (which
// must then be given; the logits have no shared-gate column); groups > 0: the E outputs form that many equal groups of
// neighbours, a group scores as its largest choice score and only members of the `keep` best groups can be chosen.
// topk_softmax: the choice is by logit (+ correction) and the weights are the softmax over the chosen logits only (times scale);
// it combines with neither identity experts nor groups. correction may be null (zeros).
struct MoeRouterOpts { bool softmax; int identity; int groups; int keep; bool topk_softmax = false; };
int moe_route(const float* logits, int ld, const float* correction, int E, int top, float scale, int* sel, float* weight,
              float* shared_gate, int* counts, int* rank, int S, cudaStream_t s, const MoeRouterOpts* opt = nullptr);
// moe_route and moe_index (dense lists) in one launch of one CTA, for calls of up to kMoeSmallItems (row, choice) pairs; it
// needs no counters.
constexpr int kMoeSmallItems = 1024;
int moe_route_small(const float* logits, int ld, const float* correction, int E, int top, float scale, int* sel, float* weight,
                    float* shared_gate, int* row_off, int* pos, int* src_row, int S, cudaStream_t s, const MoeRouterOpts* opt = nullptr);
// Expert-sorted row lists. Each list is padded to a multiple of `pad` rows (1: dense). row_off int32 [E+1] = start of every
// list (row_off[E] = total); pos[r, k] = row_off[sel] + rank = the row's place; src_row[pos] = r (entries of padding rows
// are not written: fill src_row with -1 first when pad > 1). tile_group (optional, int32 [n_tiles]): the list that owns
// rows [i * pad, (i + 1) * pad), -1 past the end: the tile table of a grouped tensor-core GEMM.
int moe_index(const int* sel, const int* rank, const int* counts, int E, int top, int pad, int* row_off, int* pos, int* src_row,
              int* tile_group, int n_tiles, int S, cudaStream_t s);
// out[i, :] = in[src_row[i], :] for rows with src_row[i] >= 0 (storage dt; W, leading dimensions and bases 16-byte aligned)
int moe_gather_rows(int dt, const void* in, int ld_in, const int* src_row, void* out, int ld_out, int rows, int W, cudaStream_t s);
// out[r, :] = sum_k weight[r, k] * eo[pos[r, k], :] (+ shared_gate[r] * so[r, :])   (eo, so, out: storage dt); choices with
// pos < 0 (identity experts) are skipped: their share is the so term
int moe_combine(int dt, const void* eo, int ld_eo, const int* pos, const float* weight, int top, const void* so, int ld_so,
                const float* shared_gate, void* out, int ld_out, int S, int W, cudaStream_t s);

// ---- rowops.cu ----------------------------------------------------------------------------------------------------------
// x[r, :] = table[id_r, :] * scale + sinusoid(past + r): entry 2i = sin(p * inv_freq[i]), 2i+1 = cos of the same
// (inv_freq null: no position term). ids: device int64; when seq_len is non-null, row r reads ids[*seq_len - S + r].
// x32: fp32 [S, copies, W], every copy the same; xa: copy in storage dt [S, W], or null.
int embed_sinusoid(int dt, const int64_t* ids, const int* seq_len, const void* table, int64_t vocab, float scale,
                   const float* inv_freq, float* x32, void* xa, int S, int W, SeqPos pos, cudaStream_t s, int copies = 1);
// Post-norm residual block: m = a, or (two branches) m = (rms(a) * wa + rms(b) * wb) / 2; x <- rms(alpha * x + m) * w.
// a, b: [S, W] (storage dt); wa, wb, w: fp32 [W]; x32 updated in place, xa = copy in storage dt.
int postnorm_residual(int dt, float* x32, void* xa, const void* a, int ld_a, const float* wa, const void* b, int ld_b,
                      const float* wb, const float* w, float alpha, float eps, int S, int W, cudaStream_t s);
// Grouped RMS norm with a multiplicative silu gate: y: fp32 [S, n]; gate: [S, n] slice (storage dt). Groups of `group`
// consecutive columns; weight w[c % w_len]. gate_first 1: out = rms(y * silu(g)) * w; 0: out = rms(y) * w * silu(g);
// 2: out = rms(y) * w * sigmoid(g).
int gated_group_norm(int dt, const float* y, int ld_y, const void* gate, int ld_gate, const float* w, int w_len,
                     void* out, int ld_out, int S, int n, int group, int gate_first, float eps, cudaStream_t s);
// out[r, c] = gelu_tanh(gu[r, c]) * gu[r, F + c]
int glu_gelu_tanh(int dt, const void* gu, int ld, void* out, int ld_out, int S, int F, cudaStream_t s);
// out[i, :] = rms(x32[rows[i], :]) * w  (storage dt)
int gather_rmsnorm(int dt, const float* x32, const int* rows, const float* w, float eps, void* out, int n_rows, int W,
                   cudaStream_t s);
// out[r, :n] = rms(in[r, :n]) * w for a slice of rows in the storage type (in, out: leading dimensions in elements; w: fp32 [n])
int slice_rmsnorm(int dt, const void* in, int ld_in, const float* w, float eps, void* out, int ld_out, int S, int n, cudaStream_t s);
// A row norm: NORM_RMS x / sqrt(mean(x^2) + eps) * w; NORM_DYT tanh(alpha * x) * w + b (no statistics of the row).
enum { NORM_RMS = 0, NORM_DYT = 1 };
struct NormSpec { int kind; const float* w; const float* b; float alpha; float eps; };
// out[i, :] = norm(x32[rows[i], :])  (storage dt)
int gather_norm(int dt, const float* x32, const int* rows, const NormSpec& n, void* out, int n_rows, int W, cudaStream_t s);
// End of a parallel block (both sublayers read the same normed row) fused with the next block's norm:
//   x32 <- x32 + (a + b)  in fp32 (a, b: [S, W] storage dt, either may be null; mc instead of b: the routed feed-forward's row
//   sum_k weight[r, k] * eo[pos[r, k]] + gate[r] * so[r] is formed here in fp32), then, if next.w, xa = next(x32) (storage dt).
// mc->so may be xa itself (identity experts return the block's normed input): every element is read before it is rewritten.
int residual_norm(int dt, float* x32, const void* a, int ld_a, const void* b, int ld_b, const MoeCombine* mc, const NormSpec& next,
                  void* xa, int S, int W, cudaStream_t s);
// out[r, c] = g * sigmoid(alpha g) * (u + up_bias), g = min(gate, limit), u = clamp(up, -limit, limit); gate = gu[r, c] and
// up = gu[r, F + c], or with il16 (columns interleaved in groups of 16) gate = gu[r, (c / 16) * 32 + c % 16], up 16 further
int glu_clamp_swish(int dt, const void* gu, int ld, void* out, int ld_out, int S, int F, float limit, cudaStream_t s, bool il16 = false,
                    float alpha = 1.702f, float up_bias = 1.f);
// A block whose norm sits on the sublayer's output: x32 <- x32 + rms(y) * w in fp32, y = the sublayer's row a [S, ld_a] (storage
// dt) or, with mc, the routed feed-forward's row formed here as in residual_norm. w: fp32 [W]. xa (optional): the new row in
// storage dt, what the next sublayer reads.
int branch_norm_residual(int dt, float* x32, const void* a, int ld_a, const MoeCombine* mc, const float* w, float eps, void* xa,
                         int S, int W, cudaStream_t s);
// x <- cap * tanh(x / cap) in place (fp32; cap <= 0: unchanged), then x <- x * scale
int softcap(float* x, int64_t n, float cap, cudaStream_t s, float scale = 1.f);

}  // namespace lcc
