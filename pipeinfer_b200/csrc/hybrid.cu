// hybrid.cu -- contexts and the decode step of layer-list models (hybrid.cuh).
//
// A decode takes a llama_batch like every other model's: tokens of several sequences, each sequence's tokens in order and next to
// each other (a "segment": a portion of a prompt, or one decoded token).  The step
//   1. resolves a state slot for every segment (SeqSlots) and a cell for every token (KvMirror::find_cells) on the host,
//   2. ships the batch's bookkeeping in one copy (token, position, cell, slot, segment per token; start / length / slot per segment),
//   3. runs every layer over ALL tokens of the batch at once: matmuls see one [tokens x width] operand, the attention kernel finds
//      a token's keys through its slot's position -> cell table, the recurrences walk each segment from the slot's state,
//   4. leaves logits rows and the sampler's top-8 records where the other architectures leave them (pib_run).
// Nothing depends on how a prompt was cut into segments, on the other segments of the batch, or on which cells / slots were used,
// beyond the summation order inside the matmuls.
#include "hybrid.cuh"

#include <algorithm>

int  pib_sample_topk(float * logits_dev, int n_rows, int n_vocab, const int32_t * bias_ids_dev, const float * bias_val_dev, int n_bias,
                     void * out_dev, const uint8_t * desc, const int * cancel, cudaStream_t st);
void rope_table_build(std::vector<float2> & tab, int n_pos, int n_dims, int mode, float freq_base, float freq_scale);

struct pib_hybrid_ctx {
    SeqSlots slots;
    float *   state = nullptr;                  // [n_slots][state_floats]
    int32_t * cellmap = nullptr;                // [n_slots][n_ctx]
    std::vector<float *>  cache;                // per caching layer: [n_ctx][cache_row]
    std::vector<float2 *> rope;                 // per rotation: [n_ctx][dims / 2] {cos, sin}
    // scratch, sized for cap tokens
    int cap = 0;
    float * x = nullptr, * h = nullptr, * y = nullptr, * proj = nullptr, * cq = nullptr, * q = nullptr, * qlat = nullptr, * lat = nullptr, * att = nullptr;
    float * rlog = nullptr, * wts = nullptr, * eup = nullptr, * edn = nullptr, * ysh = nullptr;
    float * h2 = nullptr, * cv = nullptr, * vfirst = nullptr, * mixes = nullptr;   // parallel layers: second norm (pre-norm layers: the stream's second buffer); convolved q | k | v; first mixing layer's values; token-shift mixes
    float * cat = nullptr;                      // [stream ; embedding] rows of models whose layers are walked again
    int32_t * ids = nullptr, * perm = nullptr, * inv = nullptr, * counts = nullptr, * offs = nullptr;
    // batch bookkeeping: pinned staging ring + device copy
    static const int RING = 4;
    int32_t *   meta_host[RING] = { nullptr, nullptr, nullptr, nullptr };
    cudaEvent_t meta_ev[RING]   = { nullptr, nullptr, nullptr, nullptr };
    int32_t *   meta_dev = nullptr;
    int         meta_cap = 0, meta_next = 0;
    // operands of the matmul form of the attention: keys [NK][row] and transposed latents [R][NKp] (bfloat16), query rows, score rows
    void * am_kb = nullptr, * am_vt = nullptr, * am_p = nullptr; float * am_q = nullptr, * am_s = nullptr;
    size_t am_kb_cap = 0, am_vt_cap = 0, am_q_cap = 0, am_s_cap = 0, am_p_cap = 0;
    float * split_buf = nullptr; size_t split_cap = 0;     // a long segment of the constant-decay recurrence in parts: the parts' matrices and table
    std::string kv_error;                       // set when a cache op arrived that the states cannot follow
    // per-launch timing (llama_pib_profile_layer(ctx, >= 0) switches it on): CUDA events around every launch of every layer
    struct Rec { int kind; double flops, bytes; cudaEvent_t e0, e1; };
    std::vector<Rec> prof;
};

// kinds of launches, for the profile
static const char * const HK_NAMES[] = { "cellmap", "embed_ln", "canon_conv", "mm_dq_dkv", "latent_prep", "mm_uq", "mm_absorb_uk", "latent_attention", "mm_uv", "mm_attn_o",
                                         "mm_qfv", "hgrn2_gates", "hgrn2_scan", "mm_hgrn2_o", "ln_residual", "mm_up", "polynorm", "mm_down", "mm_router", "moe_route",
                                         "moe_sort", "mm_experts_up", "mm_experts_down", "mm_shared_up", "mm_shared_down", "moe_combine", "final_ln", "mm_head", "sample", "latent_attention_mm",
                                         "embed_scale", "rms_norm_pair", "mm_qkv", "qkv_conv", "attn_prep", "kv_attention", "kv_attention_mm", "token_shift", "mm_rkvg", "mm_decay",
                                         "decay_act", "wkv_scan", "delta_prep", "delta_scan", "gated_head_norm", "glu_clamp", "parallel_sum",
                                         "embed_pair", "prenorm_shift", "loop_concat", "mm_loop_in", "mm_ssm_in", "ssm_conv", "mm_ssm_x", "mm_ssm_dt", "ssm_scan", "mm_ssm_o",
                                         "mm_dual_proj", "dual_prep", "decay_scan", "dual_gate", "mm_dual_o",
                                         "hyper_norm", "mm_mamba2_in", "mamba2_conv", "mamba2_prep", "mamba2_scan", "gated_group_norm", "mm_mamba2_o", "qkv_rope", "diff_combine",
                                         "mm_gate_up" };
enum { HK_CELLMAP, HK_EMBED, HK_CANON, HK_DQKV, HK_LPREP, HK_UQ, HK_ABSORB, HK_LATTN, HK_UV, HK_AO, HK_QFV, HK_GATES, HK_SCAN, HK_HO, HK_LNRES, HK_UP, HK_POLY, HK_DOWN,
       HK_ROUTER, HK_ROUTE, HK_SORT, HK_EUP, HK_EDOWN, HK_SUP, HK_SDOWN, HK_COMBINE, HK_FINAL, HK_HEAD, HK_SAMPLE, HK_LATTN_MM,
       HK_EMBSCALE, HK_NORM2, HK_QKV, HK_QKVCONV, HK_APREP, HK_KVATTN, HK_KVATTN_MM, HK_SHIFT, HK_RKVG, HK_DECAY, HK_DECAYACT, HK_WKVSCAN, HK_DPREP, HK_DSCAN, HK_GHNORM, HK_GLU,
       HK_PSUM, HK_EMBPAIR, HK_PRENORM, HK_CONCAT, HK_LOOPIN, HK_SSMIN, HK_SSMCONV, HK_SSMX, HK_SSMDT, HK_SSMSCAN, HK_SSMO, HK_DUALPROJ, HK_DUALPREP, HK_DECAYSCAN, HK_DUALGATE,
       HK_DUALO, HK_HYPER, HK_M2IN, HK_M2CONV, HK_M2PREP, HK_M2SCAN, HK_GGNORM, HK_M2O, HK_QKVROPE, HK_DIFFCOMB, HK_GATEUP, HK_COUNT };
const char * pib_hybrid_kind_name(int k) { return k >= 0 && k < HK_COUNT ? HK_NAMES[k] : "?"; }

// fetch and clear the records; returns the count (the stream is synchronised)
int pib_hybrid_profile_read(pib_context * c, int32_t * kind, float * ms, double * flops, double * bytes, int cap) {
    if (!c->hy) return 0;
    cudaStreamSynchronize(c->stream);
    int n = 0;
    for (auto & r : c->hy->prof) {
        float t = 0.f;
        cudaEventElapsedTime(&t, r.e0, r.e1);
        if (n < cap) { kind[n] = r.kind; ms[n] = t; flops[n] = r.flops; bytes[n] = r.bytes; n++; }
        cudaEventDestroy(r.e0); cudaEventDestroy(r.e1);
    }
    c->hy->prof.clear();
    return n;
}

#define HCK(expr) do { if ((expr) != cudaSuccess) { pib_set_error("%s:%d %s: %s", __FILE__, __LINE__, #expr, cudaGetErrorString(cudaGetLastError())); return PIB_ERR_CUDA; } } while (0)

int pib_hybrid_ctx_init(pib_context * c, int n_slots) {
    const pib_hybrid * hy = c->model->hy;
    pib_hybrid_ctx * x = new pib_hybrid_ctx();
    c->hy = x;
    if (n_slots < 1) n_slots = 1;
    x->slots.init(n_slots);
    HCK(cudaMalloc(&x->state, (size_t) n_slots * hy->state_floats * 4));
    HCK(cudaMemset(x->state, 0, (size_t) n_slots * hy->state_floats * 4));
    HCK(cudaMalloc(&x->cellmap, (size_t) n_slots * c->n_ctx * 4));
    HCK(cudaMemset(x->cellmap, 0, (size_t) n_slots * c->n_ctx * 4));
    x->cache.assign((size_t) hy->n_cache, nullptr);
    for (int i = 0; i < hy->n_cache; i++) {
        HCK(cudaMalloc(&x->cache[i], (size_t) c->n_ctx * hy->cache_row[i] * 4));
        HCK(cudaMemset(x->cache[i], 0, (size_t) c->n_ctx * hy->cache_row[i] * 4));
    }
    x->rope.assign(hy->ropes.size(), nullptr);
    for (size_t i = 0; i < hy->ropes.size(); i++) {
        std::vector<float2> tab;
        if (hy->ropes[i].factor > 0) pib_rope_table(tab, (int) c->n_ctx, hy->ropes[i]);                // scaled frequencies
        else rope_table_build(tab, (int) c->n_ctx, hy->ropes[i].dims, 4, hy->ropes[i].base, 1.0f);     // mode 4: every angle from its own power, in double
        HCK(cudaMalloc(&x->rope[i], std::max<size_t>(16, tab.size() * sizeof(float2))));
        HCK(cudaMemcpy(x->rope[i], tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice));
    }
    return PIB_OK;
}

// another number of state slots; only before the first decode of the context
int pib_hybrid_set_slots(pib_context * c, int n_slots) {
    pib_hybrid_ctx * x = c->hy;
    if (!x || n_slots < 1 || c->n_decode != 0) { pib_set_error("state slots: needs a layer-list model's context that has not decoded yet"); return PIB_ERR_ARG; }
    const pib_hybrid * hy = c->model->hy;
    cudaStreamSynchronize(c->stream);
    cudaFree(x->state); cudaFree(x->cellmap);
    x->state = nullptr; x->cellmap = nullptr;
    x->slots.init(n_slots);
    HCK(cudaMalloc(&x->state, (size_t) n_slots * hy->state_floats * 4));
    HCK(cudaMemset(x->state, 0, (size_t) n_slots * hy->state_floats * 4));
    HCK(cudaMalloc(&x->cellmap, (size_t) n_slots * c->n_ctx * 4));
    HCK(cudaMemset(x->cellmap, 0, (size_t) n_slots * c->n_ctx * 4));
    return PIB_OK;
}
int pib_hybrid_slots_free(const pib_context * c) { return c->hy ? c->hy->slots.n_free() : 0; }

#define SCAN_SPLIT_MIN 256
static bool scan_split_enabled() { static const int on = getenv("PIB_SCAN_SPLIT") ? atoi(getenv("PIB_SCAN_SPLIT")) : 1; return on != 0; }
static bool attn_mm_enabled() { static const int on = getenv("PIB_ATTN_MM") ? atoi(getenv("PIB_ATTN_MM")) : 1; return on != 0; }

// operands of the matmul form of an attention: key rows of `kw` (+ `kx` extra) bfloat16 each, transposed values [kw][2 NKp], query and
// score rows
static int grow_attn_mm(pib_context * c, size_t kw, size_t kx, int q_rows, int s_rows, int NK) {
    pib_hybrid_ctx * x = c->hy;
    const size_t R = kw, RK = kw + kx, NKp = ((size_t) NK + 7) & ~(size_t) 7, rows = (size_t) s_rows;
    auto grow = [&](void ** p, size_t * cap, size_t need) {
        if (need <= *cap) return true;
        cudaStreamSynchronize(c->stream);
        if (*p) cudaFree(*p);
        *cap = need + need / 4;
        if (cudaMalloc(p, *cap) != cudaSuccess) { cudaGetLastError(); *p = nullptr; *cap = 0; return false; }
        return true;
    };
    if (!grow(&x->am_kb, &x->am_kb_cap, NKp * RK * 2) || !grow(&x->am_vt, &x->am_vt_cap, R * NKp * 4) || !grow((void **) &x->am_q, &x->am_q_cap, (size_t) q_rows * RK * 4) ||
        !grow((void **) &x->am_s, &x->am_s_cap, rows * NKp * 8) || !grow(&x->am_p, &x->am_p_cap, rows * NKp * 4)) { pib_set_error("decode: out of memory for the attention's score rows"); return PIB_ERR_NOMEM; }
    return PIB_OK;
}

static void free_scratch(pib_hybrid_ctx * x) {
    for (void * b : { (void *) x->x, (void *) x->h, (void *) x->y, (void *) x->proj, (void *) x->cq, (void *) x->q, (void *) x->qlat, (void *) x->lat, (void *) x->att,
                      (void *) x->rlog, (void *) x->wts, (void *) x->eup, (void *) x->edn, (void *) x->ysh, (void *) x->ids, (void *) x->perm, (void *) x->inv,
                      (void *) x->counts, (void *) x->offs, (void *) x->h2, (void *) x->cv, (void *) x->vfirst, (void *) x->mixes, (void *) x->cat }) if (b) cudaFree(b);
    x->x = x->h = x->y = x->proj = x->cq = x->q = x->qlat = x->lat = x->att = x->rlog = x->wts = x->eup = x->edn = x->ysh = nullptr;
    x->h2 = x->cv = x->vfirst = x->mixes = x->cat = nullptr;
    x->ids = x->perm = x->inv = x->counts = x->offs = nullptr;
    x->cap = 0;
}

void pib_hybrid_ctx_free(pib_context * c) {
    pib_hybrid_ctx * x = c->hy;
    if (!x) return;
    free_scratch(x);
    if (x->state) cudaFree(x->state);
    if (x->cellmap) cudaFree(x->cellmap);
    for (void * p : { x->am_kb, x->am_vt, x->am_p, (void *) x->am_q, (void *) x->am_s, (void *) x->split_buf }) if (p) cudaFree(p);
    for (float * p : x->cache) if (p) cudaFree(p);
    for (float2 * p : x->rope) if (p) cudaFree(p);
    for (int i = 0; i < pib_hybrid_ctx::RING; i++) { if (x->meta_host[i]) cudaFreeHost(x->meta_host[i]); if (x->meta_ev[i]) cudaEventDestroy(x->meta_ev[i]); }
    if (x->meta_dev) cudaFree(x->meta_dev);
    delete x;
    c->hy = nullptr;
}

void pib_hybrid_on_kv_ops(pib_context * c, const std::vector<KvOp> & ops) {
    for (const KvOp & op : ops)
        if (!c->hy->slots.apply(op) && c->hy->kv_error.empty())
            c->hy->kv_error = "a sequence with recurrent state was copied or partly removed (op " + std::to_string(op.op) + "): its state cannot follow";
}

static int grow_scratch(pib_context * c, int T) {
    pib_hybrid_ctx * x = c->hy;
    if (T <= x->cap) return PIB_OK;
    const pib_hybrid * hy = c->model->hy;
    cudaStreamSynchronize(c->stream);
    for (auto & g : c->graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);        // they hold the old buffers' addresses
    c->graphs.clear();
    free_scratch(x);
    const size_t n = (size_t) ((T + 63) / 64 * 64), W = (size_t) c->model->n_embd;
    auto fl = [&](float ** p, size_t per) { return per == 0 || cudaMalloc(p, n * per * 4) == cudaSuccess; };
    auto in = [&](int32_t ** p, size_t cnt) { return cnt == 0 || cudaMalloc(p, cnt * 4) == cudaSuccess; };
    const bool ok = fl(&x->x, W * (size_t) hy->streams) && fl(&x->h, W) && fl(&x->y, W) && fl(&x->proj, (size_t) hy->w_proj) && fl(&x->cq, (size_t) hy->w_cq) && fl(&x->q, (size_t) hy->w_q) &&
                    fl(&x->qlat, (size_t) hy->w_lat) && fl(&x->lat, (size_t) hy->w_lat) && fl(&x->att, (size_t) hy->w_att) && fl(&x->rlog, (size_t) hy->w_router) &&
                    fl(&x->wts, (size_t) hy->w_pairs) && fl(&x->eup, (size_t) hy->w_eup) && fl(&x->edn, (size_t) hy->w_pairs * W) && fl(&x->ysh, hy->w_pairs ? W : 0) &&
                    in(&x->ids, n * hy->w_pairs) && in(&x->perm, n * hy->w_pairs) && in(&x->inv, n * hy->w_pairs) && in(&x->counts, (size_t) hy->w_router + 1) &&
                    in(&x->offs, (size_t) hy->w_router + 2) && fl(&x->h2, hy->form == PIB_FORM_PARALLEL || hy->form == PIB_FORM_PRENORM ? W : 0) && fl(&x->cv, (size_t) hy->w_conv) &&
                    fl(&x->vfirst, (size_t) hy->w_vfirst) && fl(&x->mixes, (size_t) hy->w_shift) && fl(&x->cat, (size_t) hy->w_cat);
    if (!ok) { cudaGetLastError(); free_scratch(x); pib_set_error("decode: out of memory for the work buffers of %d tokens", T); return PIB_ERR_NOMEM; }
    x->cap = (int) n;
    return PIB_OK;
}

// ---- the layers -----------------------------------------------------------------------------------------------------------------------
// Attention of a segment of at least MM_ATTN_MIN_LEN tokens runs as matmuls on the tensor cores in served mode, in blocks of at most
// MM_ATTN_BLOCK tokens: latent attention when its rows have at least MM_ATTN_MIN_ROW floats (a multiple of 8), key / value-head
// attention when the head size is a multiple of 8.  Everything else (decoded tokens, short portions, float32 contexts) stays with the
// per-token kernels.
#define MM_ATTN_MIN_LEN 128
#define MM_ATTN_MIN_ROW 192
#define MM_ATTN_BLOCK   512
struct pib_hseg { int start, len, seq, slot; bool fresh; };


static int run_layers(pib_context * c, pib_run & run, const pib_hbatch & B, const int32_t * B_pos_host, const std::vector<pib_hseg> & segs) {
    pib_hybrid_ctx *   x  = c->hy;
    const pib_model *  m  = c->model;
    const pib_hybrid * hy = m->hy;
    cudaStream_t       st = c->stream;
    const int   T = B.T, W = m->n_embd, exact = hy->dtype == PIB_TYPE_F32;
    const float eps = hy->eps;
    int rc;
    uint64_t & nk = c->n_kernels;
    const bool profiling = c->prof_layer >= 0 && x->prof.size() < (1u << 16);
    // one launch (or the few launches of one step) of kind k; fl / by: its floating-point operations and algorithmic bytes
#define RC(k, fl, by, e) do {                                                                                        \
        pib_hybrid_ctx::Rec r__ = { (k), (double) (fl), (double) (by), nullptr, nullptr };                           \
        if (profiling) { cudaEventCreate(&r__.e0); cudaEventCreate(&r__.e1); cudaEventRecord(r__.e0, st); }          \
        rc = (e);                                                                                                    \
        if (profiling) { cudaEventRecord(r__.e1, st); x->prof.push_back(r__); }                                      \
        if (rc != PIB_OK) return rc;                                                                                 \
        nk++;                                                                                                        \
    } while (0)
    const double Td = T, Wd = W;
    auto wbytes = [](const pib_weight * w) { return (double) w->bytes; };
    auto mmfl = [&](const pib_weight * w) { return 2.0 * Td * (double) w->N * (double) w->K; };
    auto mmby = [&](const pib_weight * w) { return (double) w->bytes + 4.0 * Td * ((double) w->N + (double) w->K); };
    auto key_pairs = [&](int window, int mask = PIB_MASK_WINDOW) {
        double n = 0;
        for (int i = 0; i < T; i++) n += mask == PIB_MASK_CHUNK ? B_pos_host[i] % window + 1 : std::min(B_pos_host[i] + 1, window);
        return n;
    };
    auto mm = [&](const pib_weight * w, const float * X, int ldx, float * Y, int ldy, int epi, float e0 = 0.f, float e1 = 0.f) {
        pib_mm a;
        a.W = w->base; a.wtype = w->type; a.ldw = w->K; a.X = X; a.ldx = ldx; a.Y = Y; a.ldy = ldy; a.M = T; a.N = (int) w->N; a.K = (int) w->K; a.epi = epi;
        a.e0 = e0; a.e1 = e1;
        a.exact = exact || w->type == PIB_TYPE_F32;
        return pib_dense_mm(a, st);
    };
    // ---- mixers: read hin [T][W], leave their output in x->y ----
    auto mixer_latent = [&](const pib_hlayer & L, const float * hin) -> int {
        const int H = L.heads, D = L.dim, rd = L.rot_dim, R = L.kv_rank, V = L.vdim, ldp = (int) L.dqkv->N, row = hy->cache_row[L.cache_id];
        float * cache = x->cache[L.cache_id];
        const double keys = key_pairs(L.window);
        // with a query latent: proj = [W_dq h | W_dkv h], the queries come from the normed latent; without: proj = [W_q h | W_dkv h], the queries stay there
        const float * qrows = L.q_rank > 0 ? x->q : x->proj;
        const int     ldq = L.q_rank > 0 ? H * (D + rd) : ldp, kv_off = L.q_rank > 0 ? L.q_rank : H * (D + rd);
        RC(HK_DQKV, mmfl(L.dqkv), mmby(L.dqkv), mm(L.dqkv, hin, W, x->proj, ldp, PIB_EPI_NONE));
        RC(HK_LPREP, 0, 8.0 * Td * ldp, pib_latent_prep(x->proj, ldp, kv_off, L, L.dq_norm, L.dkv_norm, eps, B, x->rope[L.rope_id], (int) c->n_ctx, x->cq, L.kv_from < 0 ? cache : nullptr, row, st));
        if (L.q_rank > 0) RC(HK_UQ, mmfl(L.uq), mmby(L.uq), mm(L.uq, x->cq, L.q_rank, x->q, H * (D + rd), PIB_EPI_NONE));
        {   // q_lat[t][h] = W_uk,h^T q_unrotated[t][h]: one problem per head
            pib_mm a;
            a.W = L.ukT->base; a.wtype = L.ukT->type; a.ldw = D; a.wz = (int64_t) R * D; a.X = qrows; a.ldx = ldq; a.xz = D + rd;
            a.Y = x->qlat; a.ldy = (int64_t) H * R; a.yz = R; a.M = T; a.N = R; a.K = D; a.Z = H; a.exact = exact;
            RC(HK_ABSORB, 2.0 * Td * H * R * D, wbytes(L.ukT) + 4.0 * Td * H * (D + R), pib_dense_mm(a, st));
        }
        const bool mm_ok = !exact && row >= MM_ATTN_MIN_ROW && row % 8 == 0 && attn_mm_enabled();
        bool any_mm = false, any_simt = false;
        for (const pib_hseg & g : segs) { if (mm_ok && g.len >= MM_ATTN_MIN_LEN) any_mm = true; else any_simt = true; }
        if (any_simt)
            RC(HK_LATTN, 4.0 * keys * H * (R + rd), 4.0 * keys * (R + rd) + 8.0 * Td * H * R,
               pib_latent_attention(qrows, ldq, x->qlat, L, B, x->rope[L.rope_id], (int) c->n_ctx, cache, row, x->cellmap, (int) c->n_ctx, x->lat, any_mm ? B.mmflag : nullptr, st));
        for (const pib_hseg & g : segs) {
            if (!mm_ok || g.len < MM_ATTN_MIN_LEN) continue;
            for (int o = 0; o < g.len; o += MM_ATTN_BLOCK) {
                const int nq = std::min(MM_ATTN_BLOCK, g.len - o), p0 = B_pos_host[g.start + o];
                const int j0 = std::max(0, p0 - L.window + 1), NK = p0 + nq - j0;
                if ((rc = grow_attn_mm(c, (size_t) R, (size_t) L.rot_dim, nq * H, nq * H, NK)) != PIB_OK) return rc;
                RC(HK_LATTN_MM, 2.0 * nq * H * (double) NK * (2.0 * R + rd), 2.0 * NK * (2.0 * R + rd) + 8.0 * nq * H * (2.0 * R + rd) + 8.0 * nq * H * (double) NK,
                   pib_latent_attention_mm(qrows, ldq, x->qlat, L, B, x->rope[L.rope_id], cache, row, x->cellmap + (size_t) g.slot * c->n_ctx, g.start + o, nq, j0, NK,
                                           x->am_kb, x->am_vt, x->am_q, x->am_s, x->am_p, x->lat, st));
                nk += 5;
            }
        }
        {   // value of head h = W_uv,h (sum_j p_j c_j)
            pib_mm a;
            a.W = L.uv->base; a.wtype = L.uv->type; a.ldw = R; a.wz = (int64_t) V * R; a.X = x->lat; a.ldx = (int64_t) H * R; a.xz = R;
            a.Y = x->att; a.ldy = (int64_t) H * V; a.yz = V; a.M = T; a.N = V; a.K = R; a.Z = H; a.exact = exact;
            RC(HK_UV, 2.0 * Td * H * R * V, wbytes(L.uv) + 4.0 * Td * H * (V + R), pib_dense_mm(a, st));
        }
        RC(HK_AO, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, H * V, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    auto mixer_hgrn2 = [&](const pib_hlayer & L, const float * hin) -> int {
        const int H = L.heads, HD = H * L.dim, ldp = (int) L.qfv->N;
        RC(HK_QFV, mmfl(L.qfv), mmby(L.qfv), mm(L.qfv, hin, W, x->proj, ldp, PIB_EPI_NONE));
        RC(HK_GATES, 0, 16.0 * Td * HD, pib_hgrn2_gates(x->proj, ldp, L.f_bias, L.lower, T, HD, st));
        RC(HK_SCAN, 5.0 * Td * HD * L.vdim, 4.0 * Td * ldp + 8.0 * Td * H * L.vdim, pib_hgrn2_scan(x->proj, ldp, L, B, x->state, hy->state_floats, L.onorm, eps, x->att, st)); nk++;
        RC(HK_HO, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, H * L.vdim, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    // the attention of cached key / value heads over `q`: per-token kernel, or the matmul form for long portions in served mode
    auto kv_attend = [&](const pib_hlayer & L, float * cache, int row, float * out) -> int {
        const int H = L.heads * L.maps, G = L.kv_heads * L.maps, D = L.dim, V = L.vdim;      // query rows and key heads: one per map
        const double keys = key_pairs(L.window, L.mask);
        const bool mm_ok = !exact && D % 8 == 0 && D >= 16 && V >= 16 && attn_mm_enabled();
        bool any_mm = false, any_simt = false;
        for (const pib_hseg & g : segs) { if (mm_ok && g.len >= MM_ATTN_MIN_LEN) any_mm = true; else any_simt = true; }
        if (any_simt)
            RC(HK_KVATTN, 2.0 * keys * H * (D + V), 4.0 * keys * G * (D + V) + 4.0 * Td * H * (D + V),
               pib_kv_attention(x->q, L, B, cache, row, x->cellmap, (int) c->n_ctx, out, any_mm ? B.mmflag : nullptr, st));
        for (const pib_hseg & g : segs) {
            if (!mm_ok || g.len < MM_ATTN_MIN_LEN) continue;
            const int nb = (g.len + MM_ATTN_BLOCK - 1) / MM_ATTN_BLOCK, per = (g.len + nb - 1) / nb;      // blocks of equal size: none is left with a handful of rows
            for (int o = 0; o < g.len; o += per) {
                const int nq = std::min(per, g.len - o), p0 = B_pos_host[g.start + o];
                const int j0 = L.mask == PIB_MASK_CHUNK ? p0 - p0 % L.window : std::max(0, p0 - L.window + 1), NK = p0 + nq - j0;
                if ((rc = grow_attn_mm(c, (size_t) G * std::max(D, V), (size_t) 3 * G * D + V, nq * H, nq * H, NK)) != PIB_OK) return rc;
                RC(HK_KVATTN_MM, 2.0 * nq * H * (double) NK * (D + 2.0 * V), 2.0 * NK * G * (D + 2.0 * V) + 8.0 * nq * H * (D + V) + 8.0 * nq * H * (double) NK,
                   pib_kv_attention_mm(x->q, L, B, cache, row, x->cellmap + (size_t) g.slot * c->n_ctx, g.start + o, nq, j0, NK, x->am_kb, x->am_vt, x->am_q, x->am_s, x->am_p,
                                       out, st));
                nk += 5;
            }
        }
        return PIB_OK;
    };
    // windowed attention over cached key / value heads: projections, convolution, norms + value mixing + cache write, attention, output
    auto mixer_swa = [&](const pib_hlayer & L, const float * hin) -> int {
        const int H = L.heads, V = L.vdim, C = (int) L.qkv->N, row = hy->cache_row[L.cache_id];
        float * cache = x->cache[L.cache_id];
        RC(HK_QKV, mmfl(L.qkv), mmby(L.qkv), mm(L.qkv, hin, W, x->proj, C, PIB_EPI_NONE));
        const float * src = x->proj;
        if (L.conv) {
            RC(HK_QKVCONV, 2.0 * Td * C * L.taps, 8.0 * Td * C, pib_chan_conv(x->proj, C, L.conv, L.taps, B, x->state, hy->state_floats, L.tail_off, C, x->cv, C, 0, 0, st));
            nk += L.taps > 1 && T > B.S;
            src = x->cv;
        }
        RC(HK_APREP, 0, 8.0 * Td * C, pib_swa_prep(src, C, L, eps, B, x->q, cache, row, x->vfirst, st));
        if ((rc = kv_attend(L, cache, row, x->att)) != PIB_OK) return rc;
        RC(HK_AO, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, H * V, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    // RWKV-style time mixing: the five token-shift mixes, r | k | v | g as four problems of one launch, the decay's two small matmuls, the recurrence
    auto mixer_wkv = [&](const pib_hlayer & L, const float * hin) -> int {
        const int H = L.heads, D = L.dim, HD = H * D, R = L.w_rank;
        RC(HK_SHIFT, 10.0 * Td * Wd, 24.0 * Td * Wd, pib_token_shift(hin, L.mu, 5, B, x->state, hy->state_floats, L.shift_off, W, x->mixes, st)); nk++;
        {
            pib_mm a;
            a.W = L.rkvg->base; a.wtype = L.rkvg->type; a.ldw = W; a.wz = (int64_t) HD * W; a.X = x->mixes; a.ldx = 5 * (int64_t) W; a.xz = W;
            a.Y = x->proj; a.ldy = 4 * (int64_t) HD; a.yz = HD; a.M = T; a.N = HD; a.K = W; a.Z = 4; a.exact = exact;
            RC(HK_RKVG, mmfl(L.rkvg), mmby(L.rkvg), pib_dense_mm(a, st));
        }
        RC(HK_DECAY, mmfl(L.w1), mmby(L.w1), mm(L.w1, x->mixes + 4 * (size_t) W, 5 * W, x->cq, R, PIB_EPI_NONE));
        RC(HK_DECAYACT, 0, 8.0 * Td * R, pib_rows_act(x->cq, R, R, T, 0, nullptr, st));
        RC(HK_DECAY, mmfl(L.w2), mmby(L.w2), mm(L.w2, x->cq, R, x->lat, HD, PIB_EPI_NONE));
        RC(HK_DECAYACT, 0, 8.0 * Td * HD, pib_rows_act(x->lat, HD, HD, T, 1, L.w0, st));
        RC(HK_WKVSCAN, 7.0 * Td * HD * D, 4.0 * Td * 5 * HD, pib_wkv_scan(x->proj, 4 * HD, x->lat, HD, L, B, x->state, hy->state_floats, x->att, st));
        RC(HK_GHNORM, 0, 12.0 * Td * HD, pib_gated_head_norm(x->att, T, H, D, L.onorm, D, x->proj + 3 * (size_t) HD, 4 * HD, eps, st));
        RC(HK_HO, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, HD, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    // gated delta rule: q | k | v | gate | beta | decay logits in one matmul, convolution + silu, unit vectors and gates, the recurrence
    auto mixer_delta = [&](const pib_hlayer & L, const float * hin) -> int {
        const int H = L.heads, G = L.kv_heads, D = L.dim, V = L.vdim, C = 2 * G * D + H * V, N = (int) L.qkv->N, b_off = C + H * V, a_off = b_off + H;
        RC(HK_QKV, mmfl(L.qkv), mmby(L.qkv), mm(L.qkv, hin, W, x->proj, N, PIB_EPI_NONE));
        RC(HK_QKVCONV, 2.0 * Td * C * L.taps, 8.0 * Td * C, pib_chan_conv(x->proj, N, L.conv, L.taps, B, x->state, hy->state_floats, L.tail_off, C, x->cv, C, 0, 1, st));
        nk += L.taps > 1 && T > B.S;
        RC(HK_DPREP, 0, 8.0 * Td * 2 * G * D, pib_delta_prep(x->cv, C, L, x->proj, N, b_off, a_off, x->cq, T, st));
        RC(HK_DSCAN, 8.0 * Td * H * D * V, 4.0 * Td * (C + 2.0 * H + H * V), pib_delta_scan(x->cv, C, x->cq, L, B, x->state, hy->state_floats, x->att, st));
        RC(HK_GHNORM, 0, 12.0 * Td * H * V, pib_gated_head_norm(x->att, T, H, V, L.onorm, 0, x->proj + C, N, eps, st));
        RC(HK_HO, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, H * V, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    // selective state-space scan: u | z in one matmul, convolution + bias + silu on u, [dt | B | C] from u, dt widened to the channels, the scan
    // (softplus, decays, the skip D u and the gate silu(z) inside), output matmul
    auto mixer_ssm = [&](const pib_hlayer & L, const float * hin) -> int {
        const int I = L.inner, N = L.n_state, R = L.dt_rank, ldx = (R + 2 * N + 3) & ~3;
        RC(HK_SSMIN, mmfl(L.ssm_in), mmby(L.ssm_in), mm(L.ssm_in, hin, W, x->proj, 2 * I, PIB_EPI_NONE));
        RC(HK_SSMCONV, 2.0 * Td * I * L.taps, 8.0 * Td * I, pib_chan_conv(x->proj, 2 * I, L.conv, L.taps, B, x->state, hy->state_floats, L.tail_off, I, x->cv, I, 0, 1, st, L.conv_b));
        nk += L.taps > 1 && T > B.S;
        RC(HK_SSMX, mmfl(L.ssm_x), mmby(L.ssm_x), mm(L.ssm_x, x->cv, I, x->cq, ldx, PIB_EPI_NONE));
        RC(HK_SSMDT, mmfl(L.ssm_dt), mmby(L.ssm_dt), mm(L.ssm_dt, x->cq, ldx, x->lat, I, PIB_EPI_NONE));
        RC(HK_SSMSCAN, 6.0 * Td * I * N, 4.0 * Td * (4.0 * I + 2.0 * N), pib_ssm_scan(x->cv, I, x->lat, I, x->cq + R, ldx, x->proj + I, 2 * I, L, B, x->state, hy->state_floats, x->att, st));
        RC(HK_SSMO, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, I, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    // two branches on the same input: every projection in one matmul; biases, rotation, unit norms, cache write and the linear branch's
    // activations in one kernel; attention over the token's chunk; the constant-decay recurrence; gates, the norm over the linear branch's
    // heads and both scales in one kernel; one output matmul over [softmax branch | linear branch] (its bias joins the residual sum)
    // a batch that is one long segment walks a recurrence with scalar decays in several parts at once; this sizes the parts and their buffer
    auto split_plan = [&](int Hn, int Dn, int Vn, int & parts, int & per) -> int {
        parts = per = 0;
        if (B.S == 1 && T >= SCAN_SPLIT_MIN && scan_split_enabled()) {
            static const int max_parts = getenv("PIB_SCAN_PARTS") ? std::max(2, atoi(getenv("PIB_SCAN_PARTS"))) : 8;
            per = std::max(64, ((T + max_parts - 1) / max_parts + 31) & ~31);
            parts = (T + per - 1) / per;
            if (parts < 2) parts = 0;
        }
        if (parts) {
            const size_t need = pib_scan_split_bytes(Hn, Dn, Vn, parts);
            if (need > x->split_cap) {
                cudaStreamSynchronize(st);
                if (x->split_buf) cudaFree(x->split_buf);
                x->split_buf = nullptr; x->split_cap = 0;
                if (cudaMalloc(&x->split_buf, need + need / 4) != cudaSuccess) { cudaGetLastError(); pib_set_error("decode: out of memory for the recurrence's parts"); return PIB_ERR_NOMEM; }
                x->split_cap = need + need / 4;
            }
        }
        return PIB_OK;
    };
    auto mixer_dual = [&](const pib_hlayer & L, const float * hin) -> int {
        const int H = L.heads, G = L.kv_heads, D = L.dim, H2 = L.heads2, D2 = L.dim2, V2 = L.vdim2, row = hy->cache_row[L.cache_id];
        const int ldp = ((int) L.qkv->N + 3) & ~3, ga = (H + G) * D, q2 = ga + H, k2 = q2 + H2 * D2, v2 = k2 + H2 * D2, gb = v2 + H2 * V2;
        float * cache = x->cache[L.cache_id];
        RC(HK_DUALPROJ, mmfl(L.qkv), mmby(L.qkv), mm(L.qkv, hin, W, x->proj, ldp, PIB_EPI_NONE));
        RC(HK_DUALPREP, 0, 8.0 * Td * ldp, pib_dual_prep(x->proj, ldp, L, eps, B, x->rope[L.rope_id], x->q, cache, row, st));
        if ((rc = kv_attend(L, cache, row, x->lat)) != PIB_OK) return rc;
        int parts = 0, per = 0;
        if ((rc = split_plan(H2, D2, V2, parts, per)) != PIB_OK) return rc;
        RC(HK_DECAYSCAN, 5.0 * Td * H2 * D2 * V2, 4.0 * Td * H2 * (2.0 * D2 + 2.0 * V2),
           pib_decay_scan(x->proj, ldp, q2, k2, v2, L, B, x->state, hy->state_floats, x->cv, st, x->split_buf, parts, per));
        nk += parts ? 3 : 0;
        RC(HK_DUALGATE, 0, 8.0 * Td * (H * D + 2.0 * H2 * V2), pib_dual_gate(x->lat, x->cv, x->proj, ldp, ga, gb, L, eps, T, x->att, st));
        RC(HK_DUALO, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, H * D + H2 * V2, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    // Mamba-2: z | x | B | C | dt in one matmul; convolution + bias + silu over x | B | C; step sizes and decays; the recurrence (with the
    // skip D x); the gate silu(z) and the RMS norm over equal parts of the channels; output matmul
    auto mixer_mamba2 = [&](const pib_hlayer & L, const float * hin) -> int {
        const int H = L.heads, I = H * L.vdim, GN = L.kv_heads * L.n_state, C = I + 2 * GN, ldp = ((int) L.ssm_in->N + 3) & ~3;
        RC(HK_M2IN, mmfl(L.ssm_in), mmby(L.ssm_in), mm(L.ssm_in, hin, W, x->proj, ldp, PIB_EPI_NONE));
        RC(HK_M2CONV, 2.0 * Td * C * L.taps, 8.0 * Td * C, pib_chan_conv(x->proj + I, ldp, L.conv, L.taps, B, x->state, hy->state_floats, L.tail_off, C, x->cv, C, 0, 1, st, L.conv_b));
        nk += L.taps > 1 && T > B.S;
        RC(HK_M2PREP, 0, 12.0 * Td * H, pib_mamba2_prep(x->proj, ldp, I + C, L, T, x->cq, st));
        int parts = 0, per = 0;
        if ((rc = split_plan(H, L.n_state, L.vdim, parts, per)) != PIB_OK) return rc;
        RC(HK_M2SCAN, 5.0 * Td * I * L.n_state, 4.0 * Td * (C + 2.0 * H + I), pib_mamba2_scan(x->cv, C, x->cq, L, B, x->state, hy->state_floats, x->att, st, x->split_buf, parts, per));
        nk += parts ? 4 : 0;
        RC(HK_GGNORM, 0, 12.0 * Td * I, pib_gated_group_norm(x->att, x->proj, ldp, T, I, L.norm_groups, L.onorm, eps, st));
        RC(HK_M2O, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, I, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    // differential attention: q | k | v in one matmul; biases, rotation and the cache write in one kernel; both maps of every head through
    // the attention of cached key / value heads (a map is a query row of its own over the head's values); a1 - lambda a2 and the unit RMS; output matmul
    auto mixer_diff = [&](const pib_hlayer & L, const float * hin) -> int {
        const int H = L.heads, V = L.vdim, N = (int) L.qkv->N, ldp = (N + 3) & ~3, row = hy->cache_row[L.cache_id];
        float * cache = x->cache[L.cache_id];
        RC(HK_QKV, mmfl(L.qkv), mmby(L.qkv), mm(L.qkv, hin, W, x->proj, ldp, PIB_EPI_NONE));
        RC(HK_QKVROPE, 0, 8.0 * Td * N, pib_qkv_rope(x->proj, ldp, L, B, x->rope[L.rope_id], x->q, cache, row, st));
        if ((rc = kv_attend(L, cache, row, x->lat)) != PIB_OK) return rc;
        RC(HK_DIFFCOMB, 0, 4.0 * Td * H * V * (L.maps + 1.0), pib_diff_combine(x->lat, L, eps, T, x->att, st));
        RC(HK_AO, mmfl(L.wo), mmby(L.wo), mm(L.wo, x->att, H * V, x->y, W, PIB_EPI_NONE));
        return PIB_OK;
    };
    auto run_mixer = [&](const pib_hlayer & L, const float * hin) -> int {
        switch (L.mixer) {
            case PIB_MIXER_LATENT: return mixer_latent(L, hin);
            case PIB_MIXER_HGRN2:  return mixer_hgrn2(L, hin);
            case PIB_MIXER_SWA:    return mixer_swa(L, hin);
            case PIB_MIXER_WKV:    return mixer_wkv(L, hin);
            case PIB_MIXER_DELTA:  return mixer_delta(L, hin);
            case PIB_MIXER_SSM:    return mixer_ssm(L, hin);
            case PIB_MIXER_DUAL:   return mixer_dual(L, hin);
            case PIB_MIXER_MAMBA2: return mixer_mamba2(L, hin);
            case PIB_MIXER_DIFF:   return mixer_diff(L, hin);
        }
        pib_set_error("decode: mixer %d", L.mixer);
        return PIB_ERR_UNSUPP;
    };
    // routed experts + shared expert of `min` [T][W]: x->edn holds the experts' outputs per (token, expert) pair in sorted order, x->ysh the
    // shared expert's; the caller combines them.  relu^2 experts: up rows only, the weights multiply the outputs (moe_combine); clamped gated
    // experts: rows gate | up, the router's weight multiplies the expert's input, i.e. both products before the clamp (glu_clamp)
    auto run_experts = [&](const pib_hlayer & L, const float * min, int * ld_shared) -> int {
        const int E = L.n_experts, top = L.top, P = T * top, glu = L.expert == PIB_EXPERT_GLU_CLAMP, NU = (glu ? 2 : 1) * L.ff_e;
        const double touched = P >= E ? 1.0 : (double) P / E;          // weights of experts without a row are not read
        RC(HK_ROUTER, mmfl(L.router), mmby(L.router), mm(L.router, min, W, x->rlog, E, PIB_EPI_NONE));
        RC(HK_ROUTE, 0, 4.0 * Td * E, pib_moe_route(x->rlog, T, E, top, L.route, x->ids, x->wts, st));
        RC(HK_SORT, 0, 4.0 * P * (E + 3.0), pib_moe_sort(x->ids, P, E, x->counts, x->offs, x->perm, x->inv, st)); nk++;
        {   // up-projection of every (token, expert) pair, pairs grouped by expert
            pib_mm a;
            a.W = L.e_up->base; a.wtype = L.e_up->type; a.ldw = W; a.wz = (int64_t) NU * W; a.X = min; a.ldx = W; a.xrows = x->perm; a.xdiv = top;
            a.Y = x->eup; a.ldy = NU; a.M = P; a.N = NU; a.K = W; a.Z = E; a.zrange = x->offs; a.epi = glu ? PIB_EPI_NONE : PIB_EPI_RELU2; a.exact = exact;
            RC(HK_EUP, 2.0 * P * NU * Wd, wbytes(L.e_up) * touched + 4.0 * P * (Wd + NU), pib_dense_mm(a, st));
            if (glu) RC(HK_GLU, 0, 12.0 * P * L.ff_e, pib_glu_clamp(x->eup, NU, L.ff_e, L.limit_e, x->wts, x->perm, P, st));
            pib_mm b;
            b.W = L.e_down->base; b.wtype = L.e_down->type; b.ldw = L.ff_e; b.wz = (int64_t) W * L.ff_e; b.X = x->eup; b.ldx = NU;
            b.Y = x->edn; b.ldy = W; b.M = P; b.N = W; b.K = L.ff_e; b.Z = E; b.zrange = x->offs; b.exact = exact;
            RC(HK_EDOWN, 2.0 * P * L.ff_e * Wd, wbytes(L.e_down) * touched + 4.0 * P * (Wd + L.ff_e), pib_dense_mm(b, st));
        }
        if (L.s_up) {
            const int NS = (int) L.s_up->N, ld = (NS + 3) & ~3;
            *ld_shared = ld;
            RC(HK_SUP, mmfl(L.s_up), mmby(L.s_up), mm(L.s_up, min, W, x->proj, ld, glu ? PIB_EPI_NONE : PIB_EPI_RELU2));
            if (glu) RC(HK_GLU, 0, 12.0 * Td * L.ff_s, pib_glu_clamp(x->proj, ld, L.ff_s, L.limit_s, nullptr, nullptr, T, st));
            pib_mm d;
            d.W = L.s_down->base; d.wtype = L.s_down->type; d.ldw = L.ff_s; d.X = x->proj; d.ldx = ld; d.Y = x->ysh; d.ldy = W; d.M = T; d.N = W; d.K = L.ff_s;
            d.exact = exact || L.s_down->type == PIB_TYPE_F32;
            RC(HK_SDOWN, mmfl(L.s_down), mmby(L.s_down), pib_dense_mm(d, st));
        }
        return PIB_OK;
    };

    RC(HK_CELLMAP, 0, 16.0 * Td, pib_cellmap_set(x->cellmap, (int) c->n_ctx, B, st));
    if (hy->form == PIB_FORM_HYPER)        RC(HK_EMBSCALE, 0, (2.0 + 4.0 * hy->streams) * Td * Wd, pib_embed_scale(m->tok_embd, B.tok, hy->embd_scale, T, W, x->x, st, hy->streams));
    else if (hy->form == PIB_FORM_PARALLEL) RC(HK_EMBSCALE, 0, 6.0 * Td * Wd, pib_embed_scale(m->tok_embd, B.tok, hy->embd_scale, T, W, x->x, st));
    else if (hy->form == PIB_FORM_PRENORM) RC(HK_EMBPAIR, 0, (hy->loops ? 10.0 : 6.0) * Td * Wd, pib_embed_pair(m->tok_embd, B.tok, T, W, x->x, hy->loops ? x->cat : nullptr, st));
    else                                   RC(HK_EMBED, 0, 6.0 * Td * Wd, pib_embed_ln(m->tok_embd, B.tok, hy->embd_norm, eps, T, W, x->x, st));
    // pre-norm form: the stream is (have_x ? cur : 0) + pend_y + pend_b; the sum is formed by the next norm's kernel, which leaves it in the
    // other of the two stream buffers (the block of the next token reads this token's inputs for the shift)
    float * cur = x->x, * other = x->h2;
    const float * pend_y = nullptr, * pend_b = nullptr;
    bool have_x = true;
    auto prenorm = [&](float g, const float * mu, size_t shift_off, bool keep) -> int {
        const bool upd = keep && (pend_y || pend_b || !have_x);
        RC(HK_PRENORM, 0, (upd ? 16.0 : 12.0) * Td * Wd, pib_prenorm_shift(have_x ? cur : nullptr, pend_y, pend_b, upd ? other : nullptr, g, eps, mu, B, x->state, hy->state_floats,
                                                                         shift_off, W, x->h, st));
        nk += mu != nullptr && T > B.S;
        if (upd) { std::swap(cur, other); have_x = true; pend_y = pend_b = nullptr; }
        return PIB_OK;
    };
    for (int il = 0; il < m->n_layer; il++) {
        const pib_hlayer & L = hy->layers[il];
        int lds = 0;
        if (hy->form == PIB_FORM_HYPER) {
            // the write of the sublayer before rides on the kernel that reads and norms the streams for the next one
            const int Sn = hy->streams;
            const double hby = (8.0 * Sn + 8.0) * Td * Wd;
            RC(HK_HYPER, 0, hby, pib_hyper_norm(x->x, Sn, pend_y, pend_b, L.hc1, L.norm1, L.norm1_b, eps, T, W, x->h, st));
            if ((rc = run_mixer(L, x->h)) != PIB_OK) return rc;
            pend_y = x->y; pend_b = L.hc1;
            if (L.mlp == PIB_MLP_GLU) {
                RC(HK_HYPER, 0, hby, pib_hyper_norm(x->x, Sn, pend_y, pend_b, L.hc2, L.norm2, L.norm2_b, eps, T, W, x->h, st));
                // gate and up rows are interleaved: the clamps, the gate's sigmoid and the product ride on the matmul's way out
                RC(HK_GATEUP, mmfl(L.up), wbytes(L.up) + 4.0 * Td * (Wd + L.ff), mm(L.up, x->h, W, x->proj, L.ff, PIB_EPI_GLU_PAIR, L.limit_s));
                RC(HK_DOWN, mmfl(L.down), mmby(L.down), mm(L.down, x->proj, L.ff, x->y, W, PIB_EPI_NONE));
                pend_y = x->y; pend_b = L.hc2;
            } else if (L.mlp != PIB_MLP_NONE) { pib_set_error("decode: feed-forward %d in a layer with hyper-connections", L.mlp); return PIB_ERR_UNSUPP; }
        } else if (hy->form == PIB_FORM_PRENORM) {
            if (L.loop_in) {       // a walk opens: x <- W [x ; embedding] + this walk's vector
                RC(HK_CONCAT, 0, 12.0 * Td * Wd, pib_concat_stream(have_x ? cur : nullptr, pend_y, pend_b, T, W, x->cat, st));
                RC(HK_LOOPIN, mmfl(L.loop_in), mmby(L.loop_in), mm(L.loop_in, x->cat, 2 * W, x->y, W, PIB_EPI_NONE));
                have_x = false; pend_y = x->y; pend_b = L.loop_step;
            }
            if ((rc = prenorm(L.g1, L.shift, L.shift_off, true)) != PIB_OK) return rc;
            if ((rc = run_mixer(L, x->h)) != PIB_OK) return rc;
            pend_y = x->y; pend_b = L.o_bias;
            if (L.mlp == PIB_MLP_XIELU) {
                if ((rc = prenorm(L.g2, nullptr, 0, true)) != PIB_OK) return rc;
                RC(HK_UP, mmfl(L.up), mmby(L.up), mm(L.up, x->h, W, x->proj, L.ff, PIB_EPI_XIELU, L.act[2], L.act[3]));      // the activation rides on the matmul's way out
                RC(HK_DOWN, mmfl(L.down), mmby(L.down), mm(L.down, x->proj, L.ff, x->y, W, PIB_EPI_NONE));
                pend_y = x->y; pend_b = nullptr;
            } else if (L.mlp != PIB_MLP_NONE) { pib_set_error("decode: feed-forward %d in a pre-norm layer", L.mlp); return PIB_ERR_UNSUPP; }
        } else if (hy->form == PIB_FORM_PARALLEL) {
            // x += mixer(N1 x) + ff(N2 x): both norms in one pass over x, the sum in one pass at the end
            RC(HK_NORM2, 0, (L.mlp ? 12.0 : 8.0) * Td * Wd, pib_rms_norm2(x->x, L.norm1, L.mlp ? L.norm2 : nullptr, eps, 1.0f, T, W, x->h, x->h2, st));
            if ((rc = run_mixer(L, x->h)) != PIB_OK) return rc;
            if (L.mlp == PIB_MLP_MOE) {
                if ((rc = run_experts(L, x->h2, &lds)) != PIB_OK) return rc;
                if (L.expert != PIB_EXPERT_GLU_CLAMP) { pib_set_error("decode: parallel layers take experts whose weights multiply their inputs"); return PIB_ERR_UNSUPP; }
                RC(HK_PSUM, 2.0 * Td * L.top * Wd, 4.0 * Wd * Td * (L.top + 4.0),
                   pib_parallel_sum(x->x, x->y, L.s_up ? x->ysh : nullptr, L.s_gate ? x->proj + 2 * (size_t) L.ff_s : nullptr, lds, x->edn, x->inv, L.top, T, W, st));
            } else if (L.mlp == PIB_MLP_NONE) {
                RC(HK_PSUM, 0, 12.0 * Wd * Td, pib_parallel_sum(x->x, x->y, nullptr, nullptr, 0, nullptr, nullptr, 0, T, W, st));
            } else { pib_set_error("decode: feed-forward %d in a parallel layer", L.mlp); return PIB_ERR_UNSUPP; }
        } else {
            const float * hin = x->x;
            if (L.canon) { RC(HK_CANON, 2.0 * Td * Wd * hy->taps, 8.0 * Td * Wd, pib_canon_conv(x->x, L.canon, hy->taps, B, x->state, hy->state_floats, L.tail_off, W, x->h, st)); nk += hy->taps > 1 && T > B.S; hin = x->h; }
            if ((rc = run_mixer(L, hin)) != PIB_OK) return rc;
            RC(HK_LNRES, 0, 12.0 * Td * Wd, pib_layer_norm(x->y, L.norm1, eps, T, W, x->x, 1, st));
            if (L.mlp == PIB_MLP_POLYNORM) {
                RC(HK_UP, mmfl(L.up), mmby(L.up), mm(L.up, x->x, W, x->proj, L.ff, PIB_EPI_NONE));
                RC(HK_POLY, 0, 8.0 * Td * L.ff, pib_polynorm(x->proj, T, L.ff, L.act, eps, st));
                RC(HK_DOWN, mmfl(L.down), mmby(L.down), mm(L.down, x->proj, L.ff, x->y, W, PIB_EPI_NONE));
                RC(HK_LNRES, 0, 12.0 * Td * Wd, pib_layer_norm(x->y, L.norm2, eps, T, W, x->x, 1, st));
            } else if (L.mlp == PIB_MLP_MOE) {
                if ((rc = run_experts(L, x->x, &lds)) != PIB_OK) return rc;
                RC(HK_COMBINE, 2.0 * Td * L.top * Wd, 4.0 * Wd * Td * (L.top + 2.0), pib_moe_combine(L.s_up ? x->ysh : nullptr, x->edn, x->wts, x->inv, T, L.top, W, x->y, st));
                RC(HK_LNRES, 0, 12.0 * Td * Wd, pib_layer_norm(x->y, L.norm2, eps, T, W, x->x, 1, st));
            }
        }
        if (getenv("PIB_HYBRID_DUMP") && hy->form == PIB_FORM_HYPER) {   // debugging: the sum of the streams after every layer, one file per layer and decode
            if (pend_y) { RC(HK_HYPER, 0, 0, pib_hyper_norm(x->x, hy->streams, pend_y, pend_b, nullptr, nullptr, nullptr, eps, T, W, nullptr, st)); pend_y = pend_b = nullptr; }
            std::vector<float> xb((size_t) T * hy->streams * W), hb((size_t) T * W, 0.f);
            cudaMemcpyAsync(xb.data(), x->x, xb.size() * 4, cudaMemcpyDeviceToHost, st);
            cudaStreamSynchronize(st);
            for (int t = 0; t < T; t++) for (int sn = 0; sn < hy->streams; sn++) for (int i = 0; i < W; i++) hb[(size_t) t * W + i] += xb[((size_t) t * hy->streams + sn) * W + i];
            char path[512];
            snprintf(path, sizeof(path), "%s/d%llu_l%d.f32", getenv("PIB_HYBRID_DUMP"), (unsigned long long) c->n_decode, il);
            if (FILE * f = fopen(path, "wb")) { fwrite(hb.data(), 4, hb.size(), f); fclose(f); }
        } else if (const char * dump = getenv("PIB_HYBRID_DUMP")) {          // debugging: the residual stream after every layer, one file per layer and decode
            std::vector<float> hb((size_t) T * W), yb, bb;
            if (!(hy->form == PIB_FORM_PRENORM && !have_x)) cudaMemcpyAsync(hb.data(), hy->form == PIB_FORM_PRENORM ? cur : x->x, hb.size() * 4, cudaMemcpyDeviceToHost, st);
            if (pend_y) { yb.resize(hb.size()); cudaMemcpyAsync(yb.data(), pend_y, hb.size() * 4, cudaMemcpyDeviceToHost, st); }
            if (pend_b) { bb.resize((size_t) W); cudaMemcpyAsync(bb.data(), pend_b, (size_t) W * 4, cudaMemcpyDeviceToHost, st); }
            cudaStreamSynchronize(st);
            for (size_t i = 0; i < hb.size(); i++) hb[i] += (pend_y ? yb[i] : 0.f) + (pend_b ? bb[i % (size_t) W] : 0.f);      // what the next norm's kernel will add
            char path[512];
            snprintf(path, sizeof(path), "%s/d%llu_l%d.f32", dump, (unsigned long long) c->n_decode, il);
            if (FILE * f = fopen(path, "wb")) { fwrite(hb.data(), 4, hb.size(), f); fclose(f); }
        }
    }
    if (hy->form == PIB_FORM_HYPER)         RC(HK_FINAL, 0, (4.0 * hy->streams + 8.0) * Td * Wd, pib_hyper_norm(x->x, hy->streams, pend_y, pend_b, nullptr, m->output_norm, hy->final_b, eps, T, W, x->h, st));
    else if (hy->form == PIB_FORM_PRENORM)  { if ((rc = prenorm(hy->final_g, nullptr, 0, false)) != PIB_OK) return rc; }
    else if (hy->form == PIB_FORM_PARALLEL) RC(HK_FINAL, 0, 8.0 * Td * Wd, pib_rms_norm2(x->x, m->output_norm, nullptr, eps, hy->logit_scale, T, W, x->h, nullptr, st));
    else                                    RC(HK_FINAL, 0, 8.0 * Td * Wd, pib_layer_norm(x->x, m->output_norm, eps, T, W, x->h, 0, st));
    RC(HK_HEAD, mmfl(m->output), mmby(m->output), mm(m->output, x->h, W, run.logits, m->n_vocab, PIB_EPI_NONE));
    RC(HK_SAMPLE, 0, 4.0 * Td * m->n_vocab, pib_sample_topk(run.logits, T, m->n_vocab, c->bias_ids_dev, c->bias_val_dev, c->n_bias, run.res_dev, c->desc_dev, c->cancel_table, st));
#undef RC
    return PIB_OK;
}

// ---- decode -----------------------------------------------------------------------------------------------------------------------------
int pib_hybrid_decode_start(pib_context * c, int n_tokens, const int32_t * token, const int32_t * pos, const int32_t * n_seq_id,
                            const int32_t * const * seq_id, int batch_id) {
    pib_hybrid_ctx *   x  = c->hy;
    const pib_model *  m  = c->model;
    const pib_hybrid * hy = m->hy;
    pib_kv_flush_host(c);
    if (!x->kv_error.empty()) { pib_set_error("decode: %s", x->kv_error.c_str()); return -1; }
    const int T = n_tokens, W = c->n_words;
    // segments: runs of one sequence with consecutive positions
    std::vector<pib_hseg> segs;
    for (int i = 0; i < T; i++) {
        if (token[i] < 0 || token[i] >= m->n_vocab) { pib_set_error("decode: token id %d out of range", token[i]); return -1; }
        if (n_seq_id[i] != 1) { pib_set_error("decode: a token of a model with per-sequence state belongs to exactly one sequence"); return -1; }
        const int s = seq_id[i][0];
        if (s < 0 || s >= W * 32) { pib_set_error("decode: sequence id %d out of range (max_seq %d)", s, c->max_seq); return -1; }
        if (pos[i] < 0 || (uint32_t) pos[i] >= c->n_ctx) { pib_set_error("decode: position %d outside the context of %u", pos[i], c->n_ctx); return -1; }
        if (!segs.empty() && segs.back().seq == s) {
            if (pos[i] != pos[i - 1] + 1) { pib_set_error("decode: positions of sequence %d are not consecutive", s); return -1; }
            segs.back().len++;
        } else {
            for (const pib_hseg & g : segs) if (g.seq == s) { pib_set_error("decode: tokens of sequence %d are not next to each other in the batch", s); return -1; }
            segs.push_back({ i, 1, s, -1, false });
        }
    }
    int need = 0;
    for (pib_hseg & g : segs) {
        g.slot = x->slots.find(g.seq);
        const int have = g.slot >= 0 ? x->slots.len[(size_t) g.slot] : 0;
        if (pos[g.start] != have) { pib_set_error("decode: sequence %d continues at position %d, the batch starts at %d", g.seq, have, pos[g.start]); return -1; }
        if (g.slot < 0) need++;
    }
    if (need > x->slots.n_free()) { pib_set_error("decode: no state slot for %d new sequences (%d slots)", need, x->slots.n_slots()); return -1; }
    // cells
    std::vector<uint32_t> tb((size_t) T * W, 0u);
    for (int i = 0; i < T; i++) tb[(size_t) i * W + (seq_id[i][0] >> 5)] |= 1u << (seq_id[i][0] & 31);
    std::vector<int32_t> cells((size_t) T);
    if (!c->kv.find_cells(T, pos, tb.data(), cells.data())) { pib_set_error("decode: no KV cells for %d tokens (%u of %u used)", T, c->kv.used, c->kv.size); return -1; }
    const int32_t cm = c->kv.cell_max();
    c->kv.n = (uint32_t) std::min<int32_t>((int32_t) c->kv.size, std::max<int32_t>(cm, 32));
    pib_run * run = pib_take_run(c, T);
    if (!run || grow_scratch(c, T) != PIB_OK) {
        for (int i = 0; i < T; i++) { c->kv.pos[(size_t) cells[i]] = -1; memset(&c->kv.bits[(size_t) cells[i] * W], 0, (size_t) W * 4); }
        c->kv.used -= (uint32_t) T;
        return -1;
    }
    cudaStream_t st = c->stream;
    for (pib_hseg & g : segs) {
        if (g.slot < 0) {
            g.slot = x->slots.acquire(g.seq);
            g.fresh = true;
            cudaMemsetAsync(x->state + (size_t) g.slot * hy->state_floats, 0, hy->state_floats * 4, st);      // a new owner starts from zero
        }
        x->slots.len[(size_t) g.slot] += g.len;
    }
    // bookkeeping: [tok | pos | cell | slot | seg] x T, then [seg_start | seg_len | seg_slot] x S
    const int S = (int) segs.size(), words = 6 * T + 3 * S;
    if (words > x->meta_cap) {
        cudaStreamSynchronize(st);
        for (auto & g : c->graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
        c->graphs.clear();
        for (int i = 0; i < pib_hybrid_ctx::RING; i++) { if (x->meta_host[i]) cudaFreeHost(x->meta_host[i]); x->meta_host[i] = nullptr; }
        if (x->meta_dev) cudaFree(x->meta_dev);
        x->meta_cap = words * 2 + 64;
        bool ok = cudaMalloc(&x->meta_dev, (size_t) x->meta_cap * 4) == cudaSuccess;
        for (int i = 0; ok && i < pib_hybrid_ctx::RING; i++) {
            ok = cudaMallocHost(&x->meta_host[i], (size_t) x->meta_cap * 4) == cudaSuccess;
            if (ok && !x->meta_ev[i]) ok = cudaEventCreateWithFlags(&x->meta_ev[i], cudaEventDisableTiming) == cudaSuccess;
        }
        if (!ok) { cudaGetLastError(); x->meta_cap = 0; pib_set_error("decode: out of memory for the batch bookkeeping"); return -1; }
    }
    const int ring = x->meta_next;
    x->meta_next = (x->meta_next + 1) % pib_hybrid_ctx::RING;
    cudaEventSynchronize(x->meta_ev[ring]);
    int32_t * mh = x->meta_host[ring];
    for (int sgi = 0; sgi < S; sgi++) {
        const pib_hseg & g = segs[(size_t) sgi];
        for (int i = g.start; i < g.start + g.len; i++) { mh[3 * T + i] = g.slot; mh[4 * T + i] = sgi; mh[5 * T + i] = g.len >= MM_ATTN_MIN_LEN ? 1 : 0; }
        mh[6 * T + sgi] = g.start; mh[6 * T + S + sgi] = g.len; mh[6 * T + 2 * S + sgi] = g.slot;
    }
    memcpy(mh, token, (size_t) T * 4);
    memcpy(mh + T, pos, (size_t) T * 4);
    memcpy(mh + 2 * T, cells.data(), (size_t) T * 4);
    cudaMemcpyAsync(x->meta_dev, mh, (size_t) words * 4, cudaMemcpyHostToDevice, st);
    cudaEventRecord(x->meta_ev[ring], st);
    c->h2d_bytes += (size_t) words * 4;
    const int32_t * md = x->meta_dev;
    pib_hbatch B = { md, md + T, md + 2 * T, md + 3 * T, md + 4 * T, md + 5 * T, md + 6 * T, md + 6 * T + S, md + 6 * T + 2 * S, T, S };
    run->in_use = true; run->batch_id = batch_id; run->n_tokens = T; run->failed = false; run->has_walk = false;
    c->tree_pending.n_branches = 0;
    cudaMemcpyAsync(c->cancel_table, c->run_id_host + run->id, sizeof(int), cudaMemcpyHostToDevice, st);
    // decode steps (few tokens) are launch-bound: like the other architectures' single-chunk decodes they replay a CUDA graph, captured on
    // the second use of its shape.  Every address a kernel gets is fixed for a given (tokens, segments, run slot); what varies between
    // steps (tokens, positions, cells, slots) lives in the bookkeeping block on the device.
    bool done = false;
    if (c->use_graphs && T <= 16 && c->prof_layer < 0 && !getenv("PIB_HYBRID_DUMP")) {
        pib_context::GraphEntry & g = c->graphs[(T << 16) | (S << 8) | run->id];
        g.uses++;
        if (!g.exec && !g.failed && g.uses >= 2) {
            const uint64_t k0 = c->n_kernels;
            cudaGraph_t graph = nullptr;
            bool ok = cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed) == cudaSuccess;
            if (ok) {
                const int rc = run_layers(c, *run, B, pos, segs);
                ok = cudaStreamEndCapture(st, &graph) == cudaSuccess && rc == PIB_OK && graph != nullptr;
            }
            if (ok) ok = cudaGraphInstantiate(&g.exec, graph, 0) == cudaSuccess;
            if (graph) cudaGraphDestroy(graph);
            g.n_kernels = (int) (c->n_kernels - k0);
            c->n_kernels = k0;
            if (!ok) { cudaGetLastError(); g.exec = nullptr; g.failed = true; }
        }
        if (g.exec) {
            if (cudaGraphLaunch(g.exec, st) != cudaSuccess) { pib_set_error("decode: graph launch failed: %s", cudaGetErrorString(cudaGetLastError())); run->failed = true; }
            c->n_kernels += (uint64_t) g.n_kernels;
            c->n_graph_launches++;
            done = true;
        }
    }
    if (!done) {
        // event-timed launches run in plain stream order: with programmatic dependent launch a kernel starts before the event in front of it fires
        if (c->prof_layer >= 0) pib_pdl_suspend(true);
        if (run_layers(c, *run, B, pos, segs) != PIB_OK) run->failed = true;
        if (c->prof_layer >= 0) pib_pdl_suspend(false);
    }
    if (!run->failed) {
        cudaMemcpyAsync(run->res_host, run->res_dev, sizeof(pib_row_result) * (size_t) T, cudaMemcpyDeviceToHost, st);
        c->d2h_bytes += sizeof(pib_row_result) * (size_t) T;
        run->rows_on_host = true;
    }
    if (hy->dtype == PIB_TYPE_BF16) pib_dense_mm_check(st, 1);
    cudaEventRecord(run->done, st);
    c->inflight.push_back(run->id);
    c->n_decode++;
    return run->id;
}
