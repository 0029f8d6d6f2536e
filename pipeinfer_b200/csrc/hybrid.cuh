// hybrid.cuh -- layer-list models: every layer names its own mixer and its own feed-forward.
//   mixers:        windowed latent attention with a sink; the gated linear recurrence HGRN2; windowed softmax attention over cached
//                  key / value heads (grouped queries, short convolutions on q / k / v, per-head query / key norms, value mixing with
//                  an earlier layer); RWKV-style time mixing (token shift, per-channel decay, bonus for the current token); the gated
//                  delta rule; the selective state-space scan (Mamba); a two-branch mixer -- softmax attention over chunks with a sink,
//                  rotated and unit-normed queries / keys, values that are the unrotated keys and a gate per head, beside a linear
//                  attention with a constant decay per head ("lightning attention") -- whose outputs are summed with two constants
//   feed-forwards: dense with a PolyNorm or an xIELU activation; routed mixtures of experts with a shared expert (softmax or sigmoid router,
//                  weights renormalised or not, on the experts' outputs or inputs, relu^2 or clamped gated experts)
//   layer forms:   sequential with LayerNorm on the sublayers' outputs; parallel with two RMS norms of the same input; sequential
//                  pre-norm (RMS norm with ONE number as its weight) with a token shift in front of every mixer
//                  hyper-connections: several residual streams; a sublayer reads a weighted sum of them through a LayerNorm with weight
//                  and bias, and every stream becomes a mix of the old streams plus its own multiple of the sublayer's output
//   layer runs:    a run of layers may be walked several times with the same weights, each walk with a cache and state of its own and
//                  (optionally) opened by a projection of [stream ; embedding] plus a learned vector per walk
//   more mixers:   Mamba-2 (state-space duality: one decay per head and token, keys / queries shared by groups of heads, gate before a
//                  grouped RMS norm); differential attention (two softmax maps per head over the same values, subtracted, per-head unit
//                  RMS; biases, partial rotation with YaRN-scaled frequencies); latent attention without a query latent or sink, rotated
//                  in adjacent pairs
//   more feed-forwards: dense clamped gated (the experts' activation of the mixtures above as one dense block)
// Designs built from these parts: "Rapisun", "Fabivik", "Lulenex", "Putazen".  The parts take their sizes and constants as parameters so that another
// layer-list design can name them too.
//
// What such a model adds to the runtime, beside what llama / falcon graphs use:
//   * dense weights (bfloat16 or float32 rows, pib_weight with type PIB_TYPE_BF16 / PIB_TYPE_F32) and the matmul for them (dense_mm.cu);
//   * a per-sequence STATE SLOT (SeqSlots, kv_meta.cuh): the recurrent matrices, the tails of the short convolutions and the
//     position -> cell table of the sequence.  A slot is taken at a sequence's first token and given back by llama_kv_cache_seq_rm of the
//     whole sequence (or _clear / _seq_keep);
//   * KV cells that hold one latent row per caching layer instead of K and V rows; cells are handed out one by one (scattered), so
//     a batch needs no contiguous run of free cells.
#pragma once

#include "engine.cuh"

enum { PIB_MIXER_LATENT = 1, PIB_MIXER_HGRN2 = 2, PIB_MIXER_SWA = 3, PIB_MIXER_WKV = 4, PIB_MIXER_DELTA = 5, PIB_MIXER_SSM = 6, PIB_MIXER_DUAL = 7,
       PIB_MIXER_MAMBA2 = 8, PIB_MIXER_DIFF = 9 };
enum { PIB_MLP_NONE = 0, PIB_MLP_POLYNORM = 1, PIB_MLP_MOE = 2, PIB_MLP_XIELU = 3, PIB_MLP_GLU = 4 };
// which earlier positions j a token at p may read: the last `window` ones (p - window < j <= p), or those of its own chunk (j / window == p / window)
enum { PIB_MASK_WINDOW = 0, PIB_MASK_CHUNK = 1 };
// what a matmul does to an output on its way out: nothing; max(y, 0)^2; xIELU (y > 0: e0 y^2 + y/2, else e1 (exp(y) - 1 - y) + y/2)
//   PIB_EPI_GLU_PAIR: outputs come in pairs (2 i: gate g, 2 i + 1: linear part u; the weight rows are stored interleaved); output i of a row with pitch ldy is
//   a sigmoid(1.702 a) (b + 1), a = min(g, e0), b = clamp(u, -e0, e0).  N counts the weight rows (twice the outputs).
enum { PIB_EPI_NONE = 0, PIB_EPI_RELU2 = 1, PIB_EPI_XIELU = 2, PIB_EPI_GLU_PAIR = 3 };
// layer forms: x += LN(mixer(conv(x))), x += LN(ff(x))   |   x += mixer(N1(x)) + ff(N2(x)), N = RMS norm with weight (1 + w)
//              x += mixer(shift(N(x))), x += ff(N(x)), N = RMS norm times one number, shift(h)_t = h_t + (h_{t-1} - h_t) * mu
//              hyper-connections over S streams X_s: u = sum_s in_s X_s, y = sublayer(LN(u)) (LayerNorm with weight and bias),
//              X_t <- sum_s mix[s][t] X_s + out_t y, for the mixer and then for the feed-forward; the model's output reads sum_s X_s
enum { PIB_FORM_POSTNORM = 0, PIB_FORM_PARALLEL = 1, PIB_FORM_PRENORM = 2, PIB_FORM_HYPER = 3 };
// how a rotation pairs coordinates: (i, i + dims / 2) or (2 i, 2 i + 1)
enum { PIB_PAIR_HALF = 0, PIB_PAIR_ADJACENT = 1 };
// mixture of experts: how the router's logits become weights, where a weight multiplies, what an expert computes
enum { PIB_ROUTE_SOFTMAX_RENORM = 0, PIB_ROUTE_SIGMOID = 1 };
enum { PIB_EXPERT_RELU2 = 0, PIB_EXPERT_GLU_CLAMP = 1 };

struct pib_hlayer {
    int     mixer = 0, mlp = 0;
    float * norm1 = nullptr, * norm2 = nullptr;      // LayerNorm weights applied to the sublayers' OUTPUTS
    float * canon = nullptr;                          // [width][taps] causal convolution in front of the mixer (null: none)
    // ---- latent attention ----
    int   heads = 0, dim = 0, rot_dim = 0, vdim = 0, kv_rank = 0, q_rank = 0, window = 0, rot_dims = 0;
    float rot_base = 10000.f, scale = 1.f;
    int   kv_from = -1;                               // layer whose cache rows this layer reads (-1: its own)
    int   cache_id = -1;                              // index among the layers that own cache rows
    int   rope_id = -1;                               // index of the rotation table (distinct base / dims)
    pib_weight * dqkv = nullptr;                      // rows: W_dq (q_rank) | W_dkv (kv_rank + rot_dim, absent when kv_from >= 0)
    pib_weight * uq = nullptr, * ukT = nullptr, * uv = nullptr, * wo = nullptr;   // ukT: per head [kv_rank][dim] (W_uk transposed)
    float * dq_norm = nullptr, * dkv_norm = nullptr, * sink = nullptr;
    // ---- HGRN2 ----
    pib_weight * qfv = nullptr;                       // rows: W_q (heads*dim) | W_f (heads*dim) | W_v (heads*vdim)
    float * f_bias = nullptr, * lower = nullptr, * onorm = nullptr;
    size_t  state_off = 0;                            // floats into a slot's state: the recurrent matrices [heads][dim][vdim]
    size_t  tail_off = 0;                             // floats into a slot's state: the convolution's last taps-1 inputs [taps-1][width]
    // ---- windowed attention over cached key / value heads (PIB_MIXER_SWA): heads query heads share kv_heads key / value heads ----
    int   kv_heads = 0, taps = 0, v_mix = 0;          // taps: of the convolution on q | k | v (0: none); v_mix 1: the first mixing layer (its values are kept for the step), 2: a later one
    pib_weight * qkv = nullptr;                       // rows: W_q (heads*dim) | W_k (kv_heads*dim) | W_v (kv_heads*vdim); delta rule: ... | W_g (heads*vdim) | W_b (heads) | W_a (heads)
    float * conv = nullptr;                           // [channels of q | k | v][taps]
    float * q_norm = nullptr, * k_norm = nullptr;     // [dim], shared by the heads
    float   lambda = 0.f;                             // v <- (1 - lambda) v + lambda v_first
    // ---- RWKV-style time mixing (PIB_MIXER_WKV) ----
    float * mu = nullptr;                             // [5][width]: r, k, v, g, w
    pib_weight * rkvg = nullptr;                      // 4 problems [heads*dim][width]: r, k, v, g
    pib_weight * w1 = nullptr, * w2 = nullptr;        // decay: W_w2 tanh(W_w1 .)
    int   w_rank = 0;
    float * w0 = nullptr, * bonus = nullptr;          // [heads*dim] each
    size_t  shift_off = 0;                            // floats into a slot's state: the previous token's mixer input [width]
    // ---- gated delta rule (PIB_MIXER_DELTA) ----
    float * a_log = nullptr, * dt_bias = nullptr;     // [heads]
    // ---- a layer of a run that is walked several times: the tensors belong to the first walk's entry (the others point at them) ----
    int     weights_of = -1;                          // index of the entry that owns this one's tensors (-1: itself)
    pib_weight * loop_in = nullptr;                   // set on the first layer of a walk: x <- loop_in [x ; embedding] + loop_step
    float * loop_step = nullptr;                      // [width], this walk's row
    // ---- pre-norm form: the norms' single weights, the token shift in front of the mixer ----
    float   g1 = 1.f, g2 = 1.f;
    float * shift = nullptr;                          // [width]; the previous token's normed row lives at shift_off
    // ---- selective state-space scan (PIB_MIXER_SSM): S[c][n] <- exp(dt_c A[c][n]) S[c][n] + dt_c u_c B_n, y_c = sum_n S[c][n] C_n + D_c u_c ----
    int   inner = 0, n_state = 0, dt_rank = 0;        // taps: of the convolution on u
    pib_weight * ssm_in = nullptr, * ssm_x = nullptr, * ssm_dt = nullptr;   // [2 inner][width]: u | z;  [dt_rank + 2 n_state][inner];  [inner][dt_rank]
    float * conv_b = nullptr, * ssm_a = nullptr, * ssm_d = nullptr;         // [inner]; A = -exp(A_log) [inner][n_state]; [inner]   (dt_bias: [inner])
    // ---- two-branch mixer (PIB_MIXER_DUAL) ----
    // softmax branch: heads / kv_heads / dim (= vdim: the values are the unrotated keys) / rot_dims / rot_base / scale / window + mask / sink;
    // linear branch: heads2 x (dim2 -> vdim2), decay per head.  qkv holds the rows of every projection of the mixer's input:
    // q (heads*dim) | k (kv_heads*dim) | head gates (heads) | q2 (heads2*dim2) | k2 (heads2*dim2) | v2 (heads2*vdim2) | gates2 (heads2*vdim2);
    // wo the columns [softmax branch (heads*dim) | linear branch (heads2*vdim2)]
    int   mask = PIB_MASK_WINDOW;
    int   heads2 = 0, dim2 = 0, vdim2 = 0;
    float * proj_bias = nullptr;                      // [rows of qkv], zeros where a projection has none
    float * o_bias = nullptr;                         // [width], already times mix_a
    float * decay = nullptr;                          // [heads2]
    float   mix_a = 1.f, mix_b = 1.f;                 // mixer = mix_a * softmax branch + mix_b * linear branch
                                                      // (state_off: the linear branch's matrices [heads2][dim2][vdim2])
    // ---- hyper-connections (PIB_FORM_HYPER): per sublayer [in (S) | out (S) | mix (S x S, indexed [from][to])]; LayerNorm biases ----
    float * hc1 = nullptr, * hc2 = nullptr;
    float * norm1_b = nullptr, * norm2_b = nullptr;
    // ---- Mamba-2 (PIB_MIXER_MAMBA2): heads x vdim channels, n_state states, kv_heads groups of heads share B and C.  ssm_in rows
    // [z (I) | x (I) | B (G N) | C (G N) | dt (H)], I = heads * vdim; conv / conv_b over x | B | C (taps); dt_bias, a_log, ssm_d per head;
    // per head S [n_state][vdim] <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + D x; (y silu(z)) RMS-normed in norm_groups parts, times onorm
    // (state_off: the matrices [heads][n_state][vdim]; tail_off: the convolution's last taps - 1 inputs) ----
    int   norm_groups = 1;
    // ---- differential attention (PIB_MIXER_DIFF): `maps` softmax maps per head over the same values; qkv rows
    // [q (heads * maps * dim) | k (kv_heads * maps * dim) | v (kv_heads * vdim)], head by head [map 1 | map 2], proj_bias over all rows;
    // a cell holds [k (kv_heads * maps * dim) | v (kv_heads * vdim)]; o = a1 - diff_lambda a2, o / rms(o) * diff_out ----
    int   maps = 1;                                   // attention rows per head that share its values (1: ordinary attention)
    float diff_lambda = 0.f, diff_out = 1.f;
    int   rot_pairs = PIB_PAIR_HALF;
    // ---- feed-forward ----
    int   ff = 0;
    pib_weight * up = nullptr, * down = nullptr;
    float act[4] = { 0, 0, 0, 0 };
    int   n_experts = 0, top = 0, ff_e = 0, ff_s = 0;
    pib_weight * e_up = nullptr, * e_down = nullptr;  // experts stacked: [E * ff_e][width], [E * width][ff_e]
    pib_weight * router = nullptr;                    // always float32
    pib_weight * s_up = nullptr, * s_down = nullptr;
    int   route = PIB_ROUTE_SOFTMAX_RENORM, expert = PIB_EXPERT_RELU2;
    float limit_e = 0.f, limit_s = 0.f;               // clamped gated experts: e_up / s_up hold rows gate | up (s_up one more row: the shared expert's gate logit)
    int   s_gate = 0;
};

struct pib_hybrid {
    int     dtype = PIB_TYPE_BF16;                    // PIB_TYPE_BF16: matmul operands rounded to bfloat16, fp32 accumulation; PIB_TYPE_F32: all fp32
    int     form = PIB_FORM_POSTNORM;
    int     taps = 1;
    float   eps = 1e-5f;
    float   embd_scale = 1.f, logit_scale = 1.f;      // parallel form: x = embedding * embd_scale, logits = head(norm(x)) * logit_scale
    float * embd_norm = nullptr;
    int     streams = 1;                              // hyper-connections: residual streams per token
    float * final_b = nullptr;                        // hyper-connections: the last LayerNorm's bias (its weight is the model's output_norm)
    std::vector<pib_hlayer> layers;
    size_t  state_floats = 0;                         // per state slot
    float   final_g = 1.f;                            // pre-norm form: the last norm's weight
    int     loops = 0;                                // 1: some layers open a walk (the embedding rows are kept for the step)
    pib_weight * loop_in = nullptr;                   // [width][2 width]
    float * loop_steps = nullptr;                     // [walks][width]
    int     n_cache = 0;
    std::vector<int> cache_row;                       // floats per cell of caching layer i
    // YaRN scaling (factor > 0).  d(n) = dims ln(original / (2 pi n)) / (2 ln base) is the pair index whose wave turns n times over the original
    // context; pairs below a = max(floor(d(fast)), 0) keep their frequency, pairs above b = min(ceil(d(slow)), dims - 1) have it divided by
    // the factor, and between them the blend r_i = clamp((i - a) / max(b - a, 0.001), 0, 1) gives f_i (r_i / factor + 1 - r_i).  The table's
    // cos and sin carry the magnitude 0.1 ln(factor) + 1.
    struct Rope { float base; int dims; double factor = 0, original = 0, fast = 0, slow = 0; };
    std::vector<Rope> ropes;
    // widest per-token scratch rows over all layers
    int     w_proj = 0, w_cq = 0, w_q = 0, w_lat = 0, w_att = 0, w_pairs = 0, w_eup = 0, w_router = 0;
    int     w_conv = 0, w_vfirst = 0, w_shift = 0;    // convolved q | k | v rows, the first mixing layer's values, the five token-shift mixes
    int     w_cat = 0;                                // [stream ; embedding] rows of a walk's opening
};

struct pib_hybrid_ctx;
pib_model * pib_model_load_dir(const char * dir, int dtype);          // model_dir.cu: config.json + model.safetensors
pib_model * pib_hybrid_synthetic(const char * config_json, uint64_t seed, int dtype);   // random weights for a configuration (bench)
void        pib_hybrid_model_free(pib_model * m);
int         pib_hybrid_ctx_init(pib_context * c, int n_slots);
void        pib_hybrid_ctx_free(pib_context * c);
int         pib_hybrid_set_slots(pib_context * c, int n_slots);
int         pib_hybrid_slots_free(const pib_context * c);
const char * pib_hybrid_kind_name(int kind);
int         pib_hybrid_profile_read(pib_context * c, int32_t * kind, float * ms, double * flops, double * bytes, int cap);
void        pib_hybrid_on_kv_ops(pib_context * c, const std::vector<KvOp> & ops);
int         pib_hybrid_decode_start(pib_context * c, int n_tokens, const int32_t * token, const int32_t * pos, const int32_t * n_seq_id,
                                    const int32_t * const * seq_id, int batch_id);
pib_run *   pib_take_run(pib_context * c, int n_tokens);               // engine.cu

// dense_mm.cu -- Y[z][m][n] (op)= sum_k X[z][row(m)][k] * W[z][n][k]
struct pib_mm {
    const void *    W = nullptr; int wtype = PIB_TYPE_BF16; int64_t ldw = 0, wz = 0;
    const float *   X = nullptr; int64_t ldx = 0, xz = 0;
    const int32_t * xrows = nullptr; int xdiv = 1;       // row m reads X row xrows[m] / xdiv (null: m)
    float *         Y = nullptr; int64_t ldy = 0, yz = 0;
    int             M = 0, N = 0, K = 0, Z = 1;
    const int32_t * zrange = nullptr;                    // device [Z + 1]: z owns rows [zrange[z], zrange[z + 1]); null: all M rows, every z
    int             epi = PIB_EPI_NONE;
    float           e0 = 0.f, e1 = 0.f;                  // the epilogue's constants (xIELU: softplus(p), 1/2 + softplus(q))
    int             exact = 0;                           // 1: operands stay fp32 (no bfloat16 rounding of X); W must be float32
    int             x_bf16 = 0;                          // 1: X already holds bfloat16 rows (ldx in elements, a multiple of 8): tensor-core path only, no staging copy
};
#ifdef __CUDACC__
// FAST (served mode, where the result is rounded to bfloat16 as the next matmul's operand): the exponential through ex2.approx, no branch
template <int EPI, bool FAST> __device__ __forceinline__ float pib_epilogue(float v, float e0, float e1) {
    if (EPI == PIB_EPI_RELU2) { v = fmaxf(v, 0.f); return v * v; }
    if (EPI == PIB_EPI_XIELU) {
        if (FAST) { const float n = fminf(v, 0.f), neg = fmaf(e1, (__expf(n) - 1.0f) - n, 0.5f * v), pos = fmaf(e0 * v, v, 0.5f * v); return v > 0.f ? pos : neg; }
        return v > 0.f ? fmaf(e0 * v, v, 0.5f * v) : fmaf(e1, expm1f(v) - v, 0.5f * v);
    }
    return v;
}
template <bool FAST> __device__ __forceinline__ float pib_glu_pair(float g, float u, float limit) {
    const float a = fminf(g, limit), b = fminf(fmaxf(u, -limit), limit);
    return a / (1.0f + (FAST ? __expf(-1.702f * a) : expf(-1.702f * a))) * (b + 1.0f);
}
#endif
int pib_dense_mm(const pib_mm & a, cudaStream_t st);
int pib_dense_mm_check(cudaStream_t st, int enqueue);   // dense_mma.cu: the error word of the bounded waits (1: copy it in stream order, 0: read the copy)
pib_weight * pib_dense_upload(int type, const void * host, int64_t N, int64_t K);   // type: PIB_TYPE_BF16 / PIB_TYPE_F32, row-major [N][K]

// hybrid_kernels.cu
struct pib_hbatch {                  // device view of one batch's bookkeeping
    const int32_t * tok, * pos, * cell, * slot, * seg;       // [T]
    const int32_t * mmflag;                                   // [T] 1: the token's attention runs in the matmul form (long portions, served mode)
    const int32_t * seg_start, * seg_len, * seg_slot;         // [S]
    int T, S;
};
int pib_embed_ln(const pib_weight * embd, const int32_t * tok, const float * w, float eps, int T, int W, float * x, cudaStream_t st);
int pib_layer_norm(const float * in, const float * w, float eps, int T, int W, float * out, int accumulate, cudaStream_t st);
void pib_rope_table(std::vector<float2> & tab, int n_pos, const pib_hybrid::Rope & r);
int pib_canon_conv(const float * x, const float * w, int taps, const pib_hbatch & b, float * state, size_t state_stride, size_t tail_off, int W, float * h,
                   cudaStream_t st);
int pib_chan_conv(const float * u, int ldu, const float * w, int taps, const pib_hbatch & b, float * state, size_t state_stride, size_t tail_off, int C, float * out, int ldo,
                  int add_input, int silu, cudaStream_t st, const float * bias = nullptr);
// kv_off: where W_dkv's rows start in a projection row (the query latent's rank, or the width of the query rows when the layer has no
// query latent: q_rank 0); ldq: pitch of the query rows [heads][dim + rot_dim]
int pib_latent_prep(const float * proj, int ldp, int kv_off, const pib_hlayer & L, const float * dq_norm, const float * dkv_norm, float eps, const pib_hbatch & b,
                    const float2 * rope, int rope_n_pos, float * cq, float * cache, int cache_row, cudaStream_t st);
int pib_latent_attention(const float * q, int ldq, const float * qlat, const pib_hlayer & L, const pib_hbatch & b, const float2 * rope, int rope_n_pos,
                         const float * cache, int cache_row, const int32_t * cellmap, int n_ctx, float * ctx, const int32_t * skip, cudaStream_t st);
int pib_latent_attention_mm(const float * q, int ldq, const float * qlat, const pib_hlayer & L, const pib_hbatch & b, const float2 * rope, const float * cache, int cache_row,
                            const int32_t * map, int t0, int nq, int j0, int NK, void * Kb, void * Vt, float * Qc, float * S, void * P, float * ctx, cudaStream_t st);
int pib_window_softmax(float * S, void * P, int NKp, int NK, int j0, int window, const int32_t * pos, int t0, int n_rows, int rows_per_z, int rep, const float * sink,
                       cudaStream_t st, int mask = PIB_MASK_WINDOW);
int pib_hgrn2_gates(float * qfv, int ld, const float * f_bias, const float * lower, int T, int HD, cudaStream_t st);
int pib_hgrn2_scan(const float * qfv, int ld, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, const float * onorm, float eps,
                   float * out, cudaStream_t st);
int pib_polynorm(float * z, int T, int F, const float * act4, float eps, cudaStream_t st);
int pib_moe_route(const float * logits, int T, int E, int top, int mode, int32_t * ids, float * wts, cudaStream_t st);
int pib_moe_sort(const int32_t * ids, int n_pairs, int E, int32_t * counts, int32_t * offs, int32_t * perm, int32_t * inv, cudaStream_t st);
int pib_moe_combine(const float * shared, const float * edn, const float * wts, const int32_t * inv, int T, int top, int W, float * y, cudaStream_t st);
int pib_cellmap_set(int32_t * cellmap, int n_ctx, const pib_hbatch & b, cudaStream_t st);

// mixer_kernels.cu
int pib_embed_scale(const pib_weight * embd, const int32_t * tok, float scale, int T, int W, float * x, cudaStream_t st, int copies = 1);
int pib_rms_norm2(const float * x, const float * w1, const float * w2, float eps, float out_scale, int T, int W, float * h1, float * h2, cudaStream_t st);
int pib_swa_prep(const float * cv, int ldc, const pib_hlayer & L, float eps, const pib_hbatch & b, float * q, float * cache, int cache_row, float * vfirst, cudaStream_t st);
int pib_kv_attention(const float * q, const pib_hlayer & L, const pib_hbatch & b, const float * cache, int cache_row, const int32_t * cellmap, int n_ctx, float * out,
                     const int32_t * skip, cudaStream_t st);
int pib_kv_attention_mm(const float * q, const pib_hlayer & L, const pib_hbatch & b, const float * cache, int cache_row, const int32_t * map, int t0, int nq, int j0, int NK,
                        void * Kb, void * Vt, float * Qc, float * S, void * P, float * out, cudaStream_t st);
int pib_token_shift(const float * h, const float * mu, int n_mix, const pib_hbatch & b, float * state, size_t state_stride, size_t shift_off, int W, float * mixes, cudaStream_t st);
int pib_rows_act(float * z, int ld, int n, int T, int op, const float * bias, cudaStream_t st);           // op 0: tanh; 1: exp(-exp(z + bias))
int pib_delta_prep(float * cv, int ldc, const pib_hlayer & L, const float * proj, int ldp, int b_off, int a_off, float * bg, int T, cudaStream_t st);
int pib_wkv_scan(const float * rkvg, int ld, const float * wdec, int ldw, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, float * out, cudaStream_t st);
int pib_delta_scan(const float * cv, int ldc, const float * bg, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, float * out, cudaStream_t st);
int pib_gated_head_norm(float * o, int T, int H, int V, const float * w, int w_hs, const float * gate, int ldg, float eps, cudaStream_t st);
int pib_glu_clamp(float * gu, int ld, int F, float limit, const float * scale, const int32_t * scale_of, int n_rows, cudaStream_t st);
// scan_kernels.cu
int pib_prenorm_shift(const float * xin, const float * y, const float * bias, float * xout, float g, float eps, const float * mu, const pib_hbatch & b, float * state,
                      size_t state_stride, size_t shift_off, int W, float * h, cudaStream_t st);
int pib_embed_pair(const pib_weight * embd, const int32_t * tok, int T, int W, float * x, float * cat, cudaStream_t st);
int pib_concat_stream(const float * xin, const float * y, const float * bias, int T, int W, float * cat, cudaStream_t st);
int pib_ssm_scan(const float * u, int ldu, const float * dtr, int lddt, const float * bc, int ldbc, const float * z, int ldz, const pib_hlayer & L, const pib_hbatch & b,
                 float * state, size_t state_stride, float * out, cudaStream_t st);
int pib_dual_prep(float * proj, int ldp, const pib_hlayer & L, float eps, const pib_hbatch & b, const float2 * rope, float * q, float * cache, int cache_row, cudaStream_t st);
int pib_decay_scan(const float * proj, int ldp, int q_off, int k_off, int v_off, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, float * out,
                   cudaStream_t st, float * split_buf = nullptr, int parts = 0, int per = 0);
size_t pib_decay_split_bytes(const pib_hlayer & L, int parts);
int pib_dual_gate(const float * a, const float * bo, const float * proj, int ldp, int ga_off, int gb_off, const pib_hlayer & L, float eps, int T, float * out, cudaStream_t st);
int pib_mamba2_scan(const float * xbc, int ldc, float * dg, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, float * out, cudaStream_t st,
                    float * split_buf = nullptr, int parts = 0, int per = 0);
size_t pib_scan_split_bytes(int H, int D, int V, int parts);
int pib_parallel_sum(float * x, const float * mixer, const float * shared, const float * sgl, int ldsg, const float * edn, const int32_t * inv, int top, int T, int W, cudaStream_t st);
// stream_kernels.cu
int pib_hyper_norm(float * X, int S, const float * y, const float * hc_prev, const float * hc_in, const float * w, const float * bias, float eps, int T, int W, float * h,
                   cudaStream_t st);
int pib_mamba2_prep(const float * proj, int ldp, int dt_off, const pib_hlayer & L, int T, float * dg, cudaStream_t st);
int pib_gated_group_norm(float * y, const float * z, int ldz, int T, int C, int groups, const float * w, float eps, cudaStream_t st);
int pib_qkv_rope(const float * proj, int ldp, const pib_hlayer & L, const pib_hbatch & b, const float2 * rope, float * q, float * cache, int cache_row, cudaStream_t st);
int pib_diff_combine(const float * a, const pib_hlayer & L, float eps, int T, float * out, cudaStream_t st);
