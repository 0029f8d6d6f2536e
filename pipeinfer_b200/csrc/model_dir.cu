// model_dir.cu -- models that come as a folder: config.json (sizes, constants and the list of layers) + model.safetensors (weights).
//
// A safetensors file is an 8-byte little-endian length, that many bytes of JSON (tensor name -> dtype, shape, data_offsets) and
// then the tensors' bytes.  config.json's "architecture" picks the builder from the registry below, as general.architecture does
// for GGUF files (engine.cu).  Weights arrive as bfloat16; for a float32 context they are widened once at load (exactly).
#include "hybrid.cuh"

#include <cuda_bf16.h>
#include <math.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <memory>

// ---- a small JSON reader ---------------------------------------------------------------------------------------------------------
struct Json {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    double num = 0; bool b = false; std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;
    const Json * get(const char * k) const { for (auto & kv : obj) if (kv.first == k) return &kv.second; return nullptr; }
    bool is_null() const { return kind == NUL; }
};
struct JsonParser {
    const char * p, * end; bool ok = true;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool lit(const char * s) { size_t n = strlen(s); if ((size_t) (end - p) >= n && !memcmp(p, s, n)) { p += n; return true; } return false; }
    std::string string() {
        std::string s;
        if (p >= end || *p != '"') { ok = false; return s; }
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                p++;
                switch (*p) {
                    case 'n': s += '\n'; break; case 't': s += '\t'; break; case 'r': s += '\r'; break; case 'b': s += '\b'; break; case 'f': s += '\f'; break;
                    case 'u': { unsigned cp = 0; for (int i = 0; i < 4 && p + 1 < end; i++) { p++; cp = cp * 16 + (unsigned) (isdigit((unsigned char) *p) ? *p - '0' : (tolower(*p) - 'a' + 10)); }
                                if (cp < 0x80) s += (char) cp; else if (cp < 0x800) { s += (char) (0xC0 | (cp >> 6)); s += (char) (0x80 | (cp & 0x3F)); }
                                else { s += (char) (0xE0 | (cp >> 12)); s += (char) (0x80 | ((cp >> 6) & 0x3F)); s += (char) (0x80 | (cp & 0x3F)); } break; }
                    default: s += *p;
                }
                p++;
            } else s += *p++;
        }
        if (p >= end) { ok = false; return s; }
        p++;
        return s;
    }
    Json value(int depth = 0) {
        Json v;
        ws();
        if (p >= end || depth > 64) { ok = false; return v; }
        if (*p == '{') {
            v.kind = Json::OBJ; p++; ws();
            if (p < end && *p == '}') { p++; return v; }
            while (ok) {
                ws();
                std::string k = string();
                ws();
                if (p >= end || *p != ':') { ok = false; break; }
                p++;
                v.obj.emplace_back(k, value(depth + 1));
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') { p++; break; }
                ok = false;
            }
        } else if (*p == '[') {
            v.kind = Json::ARR; p++; ws();
            if (p < end && *p == ']') { p++; return v; }
            while (ok) {
                v.arr.push_back(value(depth + 1));
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') { p++; break; }
                ok = false;
            }
        } else if (*p == '"') { v.kind = Json::STR; v.str = string(); }
        else if (lit("true")) { v.kind = Json::BOOL; v.b = true; }
        else if (lit("false")) { v.kind = Json::BOOL; }
        else if (lit("null")) {}
        else {
            char * e = nullptr;
            std::string t(p, std::min<size_t>(64, (size_t) (end - p)));
            v.num = strtod(t.c_str(), &e);
            if (e == t.c_str()) { ok = false; return v; }
            v.kind = Json::NUM; p += e - t.c_str();
        }
        return v;
    }
};
static bool json_parse(const char * s, size_t n, Json & out) { JsonParser P{ s, s + n }; out = P.value(); P.ws(); return P.ok; }

static bool read_file(const std::string & path, std::string & out) {
    FILE * f = fopen(path.c_str(), "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END); long n = ftell(f); fseek(f, 0, SEEK_SET);
    out.resize(n > 0 ? (size_t) n : 0);
    const bool ok = n >= 0 && fread(&out[0], 1, out.size(), f) == out.size();
    fclose(f);
    return ok;
}

// ---- safetensors ------------------------------------------------------------------------------------------------------------------
struct StTensor { std::string dtype; std::vector<int64_t> shape; const uint8_t * data = nullptr; size_t bytes = 0; int64_t numel() const { int64_t n = 1; for (auto d : shape) n *= d; return n; } };
struct SafeTensors {
    void * map = nullptr; size_t size = 0;
    std::map<std::string, StTensor> t;
    ~SafeTensors() { if (map) munmap(map, size); }
    bool open(const std::string & path) {
        const int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0) { pib_set_error("model: cannot open %s", path.c_str()); return false; }
        struct stat sb;
        if (fstat(fd, &sb) != 0 || sb.st_size < 8) { close(fd); pib_set_error("model: %s is too short", path.c_str()); return false; }
        size = (size_t) sb.st_size;
        map = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        close(fd);
        if (map == MAP_FAILED) { map = nullptr; pib_set_error("model: mmap of %s failed", path.c_str()); return false; }
        const uint8_t * b = (const uint8_t *) map;
        uint64_t hl = 0;
        for (int i = 7; i >= 0; i--) hl = (hl << 8) | b[i];
        if (hl > size - 8) { pib_set_error("model: %s: header length %llu exceeds the file", path.c_str(), (unsigned long long) hl); return false; }
        Json h;
        if (!json_parse((const char *) b + 8, (size_t) hl, h) || h.kind != Json::OBJ) { pib_set_error("model: %s: header is not JSON", path.c_str()); return false; }
        const uint8_t * data = b + 8 + hl;
        const size_t    dsz  = size - 8 - (size_t) hl;
        for (auto & kv : h.obj) {
            if (kv.first == "__metadata__") continue;
            const Json * dt = kv.second.get("dtype"), * sh = kv.second.get("shape"), * of = kv.second.get("data_offsets");
            if (!dt || !sh || !of || of->arr.size() != 2) { pib_set_error("model: tensor %s: incomplete header entry", kv.first.c_str()); return false; }
            StTensor x;
            x.dtype = dt->str;
            for (auto & d : sh->arr) x.shape.push_back((int64_t) d.num);
            const size_t a = (size_t) of->arr[0].num, e = (size_t) of->arr[1].num;
            if (e < a || e > dsz) { pib_set_error("model: tensor %s: data offsets outside the file", kv.first.c_str()); return false; }
            x.data = data + a; x.bytes = e - a;
            const size_t es = x.dtype == "BF16" || x.dtype == "F16" ? 2 : (x.dtype == "F32" || x.dtype == "I32") ? 4 : 0;
            if (es == 0 || (size_t) x.numel() * es != x.bytes) { pib_set_error("model: tensor %s: dtype %s / shape do not fit %zu bytes", kv.first.c_str(), x.dtype.c_str(), x.bytes); return false; }
            t[kv.first] = x;
        }
        return true;
    }
};

// ---- tensor sources: a file, or a seeded generator (synthetic models of a configuration, for benchmarks) -----------------------------
struct TensorSource {
    SafeTensors * st = nullptr;
    uint64_t      seed = 0;
    bool          failed = false;
    bool          norms_around_zero = false;       // synthetic weights: layer norms are stored as w with (1 + w) applied
    // extent `axis` of a tensor in the file (negative: from the end); `dflt` for a synthetic source or a missing tensor
    int64_t dim(const std::string & name, int axis, int64_t dflt) const {
        if (!st) return dflt;
        auto it = st->t.find(name);
        if (it == st->t.end()) return dflt;
        const int n = (int) it->second.shape.size();
        if (axis < 0) axis += n;
        return axis >= 0 && axis < n ? it->second.shape[(size_t) axis] : dflt;
    }
    bool has(const std::string & name) const { return !st || st->t.count(name) != 0; }
    // the tensor as float32, shape checked
    bool get(const std::string & name, std::initializer_list<int64_t> shape, std::vector<float> & out) {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        out.resize((size_t) n);
        if (!st) { synth(name, shape, out); return true; }
        auto it = st->t.find(name);
        if (it == st->t.end()) { pib_set_error("model: tensor %s is missing", name.c_str()); failed = true; return false; }
        const StTensor & x = it->second;
        if (x.shape != std::vector<int64_t>(shape)) { pib_set_error("model: tensor %s has another shape than the configuration gives", name.c_str()); failed = true; return false; }
        if (x.dtype == "BF16") { const uint16_t * s = (const uint16_t *) x.data; for (int64_t i = 0; i < n; i++) { uint32_t u = (uint32_t) s[i] << 16; memcpy(&out[i], &u, 4); } }
        else if (x.dtype == "F32") memcpy(out.data(), x.data, (size_t) n * 4);
        else if (x.dtype == "F16") { const __half * s = (const __half *) x.data; for (int64_t i = 0; i < n; i++) out[i] = __half2float(s[i]); }
        else { pib_set_error("model: tensor %s: dtype %s", name.c_str(), x.dtype.c_str()); failed = true; return false; }
        return true;
    }
    static bool ends(const std::string & s, const char * e) { const size_t n = strlen(e); return s.size() >= n && !s.compare(s.size() - n, n, e); }
    void synth(const std::string & name, std::initializer_list<int64_t> shape, std::vector<float> & out) {
        uint64_t h = seed * 0x9E3779B97F4A7C15ull + 0x1234567;
        for (char ch : name) h = (h ^ (uint8_t) ch) * 0x100000001B3ull;
        auto next = [&]() { h ^= h << 13; h ^= h >> 7; h ^= h << 17; return (float) ((h >> 11) & 0xFFFFFF) / 16777216.0f; };     // [0, 1)
        const int64_t last = shape.size() ? *(shape.end() - 1) : 1;
        const bool norm = ends(name, "norm") || ends(name, "norm1") || ends(name, "norm2");
        const bool around_zero = norms_around_zero && (ends(name, "norm1") || ends(name, "norm2") || name == "final.norm");
        const float amp = 1.5f * sqrtf(3.0f / (float) last);
        for (size_t i = 0; i < out.size(); i++) {
            const float u = next() * 2.f - 1.f;
            float v;
            if (around_zero) v = 0.2f * u;
            else if (norm) v = 1.0f + 0.2f * u;
            else if (name.find(".mu.") != std::string::npos) v = 0.5f + 0.5f * u;
            else if (name.find(".hc") != std::string::npos)                // hyper-connections: read about evenly, write with weights near 1, mix near the identity
                v = ends(name, ".in") ? 1.0f / (float) last + 0.1f * u : ends(name, ".out") ? 0.8f + 0.2f * u : ((i / (size_t) last == i % (size_t) last) ? 0.9f : 0.f) + 0.1f * u;
            else if (ends(name, "vmix")) v = 0.3f;
            else if (ends(name, ".conv")) v = 0.5f * u + ((int64_t) (i % (size_t) last) == last - 1 ? 0.5f : 0.f);
            else if (ends(name, "w0") || ends(name, "A_log") || ends(name, "dt_bias") || ends(name, "mix.u")) v = u;
            else if (ends(name, "lower")) v = 0.45f + 0.45f * u;
            else if (ends(name, ".act")) v = (i == 0 ? 0.6f : i == 1 ? 0.3f : i == 2 ? 0.2f : 0.05f);
            else if (ends(name, "sink") || ends(name, "f.b")) v = u;
            else if (ends(name, "canon1")) v = 0.3f * u;
            else if (name == "embed") v = 1.7f * u;
            else v = amp * u;
            out[i] = __bfloat162float(__float2bfloat16_rn(v));
        }
    }
};

static float * upload_f32v(const std::vector<float> & v) {
    float * d = nullptr;
    if (cudaMalloc(&d, std::max<size_t>(16, v.size() * 4)) != cudaSuccess || cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
        pib_set_error("model: upload of %zu floats failed: %s", v.size(), cudaGetErrorString(cudaGetLastError()));
        return nullptr;
    }
    return d;
}
// a matrix for the dense matmul: bfloat16 rows in served mode, float32 rows in exact mode (dtype = PIB_TYPE_BF16 / PIB_TYPE_F32)
static pib_weight * upload_mat(const std::vector<float> & v, int64_t N, int64_t K, int dtype, pib_model * m) {
    pib_weight * w;
    if (dtype == PIB_TYPE_F32) w = pib_dense_upload(PIB_TYPE_F32, v.data(), N, K);
    else {
        std::vector<__nv_bfloat16> hb(v.size());
        for (size_t i = 0; i < v.size(); i++) hb[i] = __float2bfloat16_rn(v[i]);
        w = pib_dense_upload(PIB_TYPE_BF16, hb.data(), N, K);
    }
    if (w) m->weight_bytes += w->bytes;
    return w;
}

static double jnum(const Json * o, const char * k, double dflt, bool * ok = nullptr) {
    const Json * v = o ? o->get(k) : nullptr;
    if (!v || v->kind != Json::NUM) { if (ok) *ok = false; return dflt; }
    return v->num;
}

// ---- the Rapisun builder ----------------------------------------------------------------------------------------------------------
// Sequential layers with LayerNorm on the sublayers' outputs, a causal convolution in front of every mixer, latent attention and HGRN2
// mixers, PolyNorm and relu^2 mixture-of-experts feed-forwards.  Reads every size and constant from the configuration; tensor names are '<layer>.mix.*', '<layer>.mlp.*', '<layer>.norm1|norm2|canon1'.
static pib_model * build_rapisun(const Json & cfg, TensorSource & src, int dtype) {
    std::unique_ptr<pib_model, void (*)(pib_model *)> mp(new pib_model(), pib_model_free);
    pib_model * m = mp.get();
    pib_hybrid * hy = new pib_hybrid();
    m->hy = hy;
    m->arch = 2; m->name = "Rapisun";
    bool ok = true;
    const int W = (int) jnum(&cfg, "width", 0, &ok), V = (int) jnum(&cfg, "vocab", 0, &ok);
    const Json * layers = cfg.get("layers");
    if (!ok || W <= 0 || V <= 0 || !layers || layers->kind != Json::ARR) { pib_set_error("model: config.json needs width, vocab and layers"); return nullptr; }
    hy->dtype = dtype;
    hy->eps = (float) jnum(cfg.get("norm"), "eps", 1e-5);
    hy->taps = cfg.get("canon") ? (int) jnum(cfg.get("canon"), "taps", 1) : 0;
    m->n_embd = W; m->n_vocab = V; m->n_layer = (int) layers->arr.size(); m->layer_begin = 0; m->layer_end = m->n_layer;
    m->wtype = dtype; m->n_ctx_train = 1 << 20; m->n_head = 1; m->n_head_kv = 1; m->tok_bos = -1; m->tok_eos = -1;
    std::vector<float> v;
#define GET(name, ...) do { if (!src.get((name), { __VA_ARGS__ }, v)) return nullptr; } while (0)
#define VEC(dst, name, n) do { GET(name, (int64_t) (n)); if (!((dst) = upload_f32v(v))) return nullptr; } while (0)
#define MAT(dst, name, N, K) do { GET(name, (int64_t) (N), (int64_t) (K)); if (!((dst) = upload_mat(v, (N), (K), dtype, m))) return nullptr; } while (0)
    MAT(m->tok_embd, "embed", V, W);
    VEC(hy->embd_norm, "embed.norm", W);
    VEC(m->output_norm, "final.norm", W);
    MAT(m->output, "head", V, W);
    hy->layers.resize(m->n_layer);
    size_t state = 0;
    auto widen = [](int & a, int64_t b) { if (b > a) a = (int) b; };
    for (int il = 0; il < m->n_layer; il++) {
        const Json & jl = layers->arr[il];
        pib_hlayer & L = hy->layers[il];
        const std::string p = "l" + std::to_string(il) + ".", px = p + "mix.", pm = p + "mlp.";
        const Json * ty = jl.get("type"), * mx = jl.get("mixer"), * ml = jl.get("mlp");
        if (!ty || ty->kind != Json::STR || !mx) { pib_set_error("model: layer %d needs type and mixer", il); return nullptr; }
        VEC(L.norm1, p + "norm1", W);
        if (hy->taps > 0) { GET(p + "canon1", W, hy->taps); if (!(L.canon = upload_f32v(v))) return nullptr; L.tail_off = state; state += (size_t) (hy->taps - 1) * W; }
        L.heads = (int) jnum(mx, "heads", 0); L.dim = (int) jnum(mx, "dim", 0); L.vdim = (int) jnum(mx, "vdim", 0);
        if (L.heads <= 0 || L.dim <= 0 || L.vdim <= 0) { pib_set_error("model: layer %d: heads / dim / vdim", il); return nullptr; }
        if (ty->str == "hgrn2") {
            L.mixer = PIB_MIXER_HGRN2;
            const int64_t HD = (int64_t) L.heads * L.dim, HV = (int64_t) L.heads * L.vdim;
            std::vector<float> all;
            GET(px + "q", HD, W); all = v;
            GET(px + "f", HD, W); all.insert(all.end(), v.begin(), v.end());
            GET(px + "v", HV, W); all.insert(all.end(), v.begin(), v.end());
            if (!(L.qfv = upload_mat(all, 2 * HD + HV, W, dtype, m))) return nullptr;
            VEC(L.f_bias, px + "f.b", HD);
            VEC(L.lower, px + "lower", HD);
            VEC(L.onorm, px + "norm", L.vdim);
            MAT(L.wo, px + "o", W, HV);
            L.state_off = state; state += (size_t) HD * L.vdim;
            widen(hy->w_proj, 2 * HD + HV); widen(hy->w_att, HV);
        } else if (ty->str == "latent_attention") {
            L.mixer = PIB_MIXER_LATENT;
            L.rot_dim = (int) jnum(mx, "rot_dim", 0); L.kv_rank = (int) jnum(mx, "kv_rank", 0); L.q_rank = (int) jnum(mx, "q_rank", 0);
            L.scale = (float) jnum(mx, "scale", 1.0 / sqrt((double) (L.dim + L.rot_dim)));
            const Json * mk = mx->get("mask"), * rt = mx->get("rot");
            L.window = mk ? (int) jnum(mk, "size", 0) : 0;
            if (L.window <= 0) L.window = 1 << 30;                              // no mask: every earlier token is seen
            L.rot_base = (float) jnum(rt, "base", 10000.0); L.rot_dims = rt ? (int) jnum(rt, "dims", L.rot_dim) : 0;
            L.kv_from = mx->get("kv_from") ? (int) jnum(mx, "kv_from", -1) : -1;
            if (L.kv_rank <= 0 || L.q_rank <= 0 || L.rot_dim < 0 || L.rot_dims > L.rot_dim || (L.rot_dims & 1)) { pib_set_error("model: layer %d: kv_rank / q_rank / rot_dim / rot.dims", il); return nullptr; }
            const int64_t H = L.heads, D = L.dim, rd = L.rot_dim, R = L.kv_rank, Q = L.q_rank;
            std::vector<float> all;
            GET(px + "dq", Q, W); all = v;
            if (L.kv_from < 0) {
                GET(px + "dkv", R + rd, W); all.insert(all.end(), v.begin(), v.end());
                VEC(L.dkv_norm, px + "dkv.norm", R);
                L.cache_id = hy->n_cache++;
                hy->cache_row.push_back((int) (R + rd));
            } else {
                if (L.kv_from >= il || hy->layers[L.kv_from].mixer != PIB_MIXER_LATENT || hy->layers[L.kv_from].kv_from >= 0 ||
                    hy->layers[L.kv_from].kv_rank != L.kv_rank || hy->layers[L.kv_from].rot_dim != L.rot_dim) {
                    pib_set_error("model: layer %d: kv_from %d is not an earlier latent-attention layer with a cache of the same shape", il, L.kv_from);
                    return nullptr;
                }
                L.cache_id = hy->layers[L.kv_from].cache_id;
            }
            if (!(L.dqkv = upload_mat(all, (int64_t) all.size() / W, W, dtype, m))) return nullptr;
            VEC(L.dq_norm, px + "dq.norm", Q);
            MAT(L.uq, px + "uq", H * (D + rd), Q);
            GET(px + "uk", H * D, R);
            {   // per head W_uk^T: [kv_rank][dim], so that folding a query through it is the same row-times-row product as every other matmul
                std::vector<float> tr((size_t) (H * D * R));
                for (int64_t h = 0; h < H; h++) for (int64_t d = 0; d < D; d++) for (int64_t r = 0; r < R; r++) tr[(size_t) ((h * R + r) * D + d)] = v[(size_t) ((h * D + d) * R + r)];
                if (!(L.ukT = upload_mat(tr, H * R, D, dtype, m))) return nullptr;
            }
            MAT(L.uv, px + "uv", H * L.vdim, R);
            VEC(L.sink, px + "sink", H);
            MAT(L.wo, px + "o", W, H * L.vdim);
            L.rope_id = -1;
            for (size_t i = 0; i < hy->ropes.size(); i++) if (hy->ropes[i].base == L.rot_base && hy->ropes[i].dims == L.rot_dims) L.rope_id = (int) i;
            if (L.rope_id < 0) { L.rope_id = (int) hy->ropes.size(); hy->ropes.push_back({ L.rot_base, L.rot_dims }); }
            widen(hy->w_proj, Q + R + rd); widen(hy->w_cq, Q); widen(hy->w_q, H * (D + rd)); widen(hy->w_lat, H * R); widen(hy->w_att, H * L.vdim);
        } else { pib_set_error("model: layer %d: unknown mixer '%s'", il, ty->str.c_str()); return nullptr; }
        if (ml && !ml->is_null()) {
            VEC(L.norm2, p + "norm2", W);
            const Json * kind = ml->get("kind");
            if (kind && kind->str == "dense") {
                L.mlp = PIB_MLP_POLYNORM; L.ff = (int) jnum(ml, "ff", 0);
                if (L.ff <= 0) { pib_set_error("model: layer %d: mlp.ff", il); return nullptr; }
                MAT(L.up, pm + "up", L.ff, W);
                MAT(L.down, pm + "down", W, L.ff);
                GET(pm + "act", 4);
                memcpy(L.act, v.data(), 16);
                widen(hy->w_proj, L.ff);
            } else if (kind && kind->str == "moe") {
                L.mlp = PIB_MLP_MOE;
                L.n_experts = (int) jnum(ml->get("router"), "experts", 0); L.top = (int) jnum(ml->get("router"), "top", 0);
                L.ff_e = (int) jnum(ml->get("expert"), "ff", 0);
                const Json * sh = ml->get("shared");
                L.ff_s = sh && !sh->is_null() ? (int) jnum(sh, "ff", 0) : 0;
                if (L.n_experts <= 0 || L.top <= 0 || L.top > L.n_experts || L.ff_e <= 0) { pib_set_error("model: layer %d: router.experts / router.top / expert.ff", il); return nullptr; }
                std::vector<float> ups, downs;
                for (int e = 0; e < L.n_experts; e++) {
                    const std::string pe = pm + "e" + std::to_string(e) + ".";
                    GET(pe + "up", L.ff_e, W); ups.insert(ups.end(), v.begin(), v.end());
                    GET(pe + "down", W, L.ff_e); downs.insert(downs.end(), v.begin(), v.end());
                }
                if (!(L.e_up = upload_mat(ups, (int64_t) L.n_experts * L.ff_e, W, dtype, m)) || !(L.e_down = upload_mat(downs, (int64_t) L.n_experts * W, L.ff_e, dtype, m))) return nullptr;
                GET(pm + "router", L.n_experts, W);
                if (!(L.router = upload_mat(v, L.n_experts, W, PIB_TYPE_F32, m))) return nullptr;          // the router is always 32-bit
                if (L.ff_s > 0) { MAT(L.s_up, pm + "shared.up", L.ff_s, W); MAT(L.s_down, pm + "shared.down", W, L.ff_s); widen(hy->w_proj, L.ff_s); }
                widen(hy->w_pairs, L.top); widen(hy->w_eup, (int64_t) L.top * L.ff_e); widen(hy->w_router, L.n_experts);
            } else { pib_set_error("model: layer %d: unknown mlp kind", il); return nullptr; }
        }
    }
    hy->state_floats = state ? state : 4;
#undef GET
#undef VEC
#undef MAT
    return mp.release();
}

// ---- the Fabivik builder ----------------------------------------------------------------------------------------------------------
// Parallel layers (x += mixer(N1 x) + ff(N2 x), RMS norms with weights stored around zero), mixers "attention" (windowed softmax
// attention with short convolutions on q / k / v, per-head query / key norms, grouped queries and value mixing), "wkv" (RWKV-style
// time mixing) and "delta" (gated delta rule), mixtures of clamped gated experts behind a sigmoid router whose weights multiply the
// experts' inputs, a gated shared expert.  Every size comes from the configuration or a tensor's shape.
static pib_model * build_fabivik(const Json & cfg, TensorSource & src, int dtype) {
    std::unique_ptr<pib_model, void (*)(pib_model *)> mp(new pib_model(), pib_model_free);
    pib_model * m = mp.get();
    pib_hybrid * hy = new pib_hybrid();
    m->hy = hy;
    m->arch = 2; m->name = "Fabivik";
    src.norms_around_zero = true;
    bool ok = true;
    const int W = (int) jnum(&cfg, "width", 0, &ok), V = (int) jnum(&cfg, "vocab", 0, &ok);
    const Json * layers = cfg.get("layers");
    if (!ok || W <= 0 || V <= 0 || !layers || layers->kind != Json::ARR) { pib_set_error("model: config.json needs width, vocab and layers"); return nullptr; }
    hy->dtype = dtype;
    hy->form = PIB_FORM_PARALLEL;
    hy->eps = (float) jnum(cfg.get("norm"), "eps", 1e-5);
    hy->embd_scale = (float) jnum(cfg.get("embedding"), "scale", 1.0);
    hy->logit_scale = (float) jnum(&cfg, "logit_scale", 1.0);
    hy->taps = 0;
    m->n_embd = W; m->n_vocab = V; m->n_layer = (int) layers->arr.size(); m->layer_begin = 0; m->layer_end = m->n_layer;
    m->wtype = dtype; m->n_ctx_train = 1 << 20; m->n_head = 1; m->n_head_kv = 1; m->tok_bos = -1; m->tok_eos = -1;
    std::vector<float> v;
#define GET(name, ...) do { if (!src.get((name), { __VA_ARGS__ }, v)) return nullptr; } while (0)
#define VEC(dst, name, n) do { GET(name, (int64_t) (n)); if (!((dst) = upload_f32v(v))) return nullptr; } while (0)
#define MAT(dst, name, N, K) do { GET(name, (int64_t) (N), (int64_t) (K)); if (!((dst) = upload_mat(v, (N), (K), dtype, m))) return nullptr; } while (0)
#define APPEND(all, name, N, K) do { GET(name, (int64_t) (N), (int64_t) (K)); (all).insert((all).end(), v.begin(), v.end()); } while (0)
    MAT(m->tok_embd, "embed", V, W);
    VEC(m->output_norm, "final.norm", W);
    MAT(m->output, "head", V, W);
    hy->layers.resize(m->n_layer);
    size_t state = 0;
    int first_mix = -1;
    auto widen = [](int & a, int64_t b) { if (b > a) a = (int) b; };
    for (int il = 0; il < m->n_layer; il++) {
        const Json & jl = layers->arr[il];
        pib_hlayer & L = hy->layers[il];
        const std::string p = "l" + std::to_string(il) + ".", px = p + "mix.", pm = p + "mlp.";
        const Json * ty = jl.get("type"), * mx = jl.get("mixer"), * ml = jl.get("mlp");
        if (!ty || ty->kind != Json::STR || !mx) { pib_set_error("model: layer %d needs type and mixer", il); return nullptr; }
        VEC(L.norm1, p + "norm1", W);
        L.heads = (int) jnum(mx, "heads", 0); L.dim = (int) jnum(mx, "dim", 0);
        L.kv_heads = (int) jnum(mx, "kv_heads", L.heads); L.vdim = (int) jnum(mx, "vdim", L.dim);
        L.taps = (int) jnum(mx, "conv", 0);
        if (L.heads <= 0 || L.dim <= 0 || L.vdim <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads) { pib_set_error("model: layer %d: heads / kv_heads / dim / vdim", il); return nullptr; }
        const int64_t H = L.heads, G = L.kv_heads, D = L.dim, Vd = L.vdim;
        if (ty->str == "attention") {
            L.mixer = PIB_MIXER_SWA;
            L.scale = (float) jnum(mx, "scale", 1.0 / sqrt((double) D));
            const Json * mk = mx->get("mask");
            L.window = mk && !mk->is_null() ? (int) jnum(mk, "size", 0) : 0;
            if (L.window <= 0) L.window = 1 << 30;                              // no mask: every earlier token is seen
            const Json * vm = mx->get("v_mix");
            const bool mixes = vm && ((vm->kind == Json::BOOL && vm->b) || (vm->kind == Json::NUM && vm->num != 0));
            const int64_t C = H * D + G * D + G * Vd;
            std::vector<float> all;
            APPEND(all, px + "q", H * D, W); APPEND(all, px + "k", G * D, W); APPEND(all, px + "v", G * Vd, W);
            if (!(L.qkv = upload_mat(all, C, W, dtype, m))) return nullptr;
            if (L.taps > 0) {
                all.clear();
                APPEND(all, px + "q.conv", H * D, L.taps); APPEND(all, px + "k.conv", G * D, L.taps); APPEND(all, px + "v.conv", G * Vd, L.taps);
                if (!(L.conv = upload_f32v(all))) return nullptr;
                L.tail_off = state; state += (size_t) (L.taps - 1) * C;
            }
            VEC(L.q_norm, px + "q.norm", D);
            VEC(L.k_norm, px + "k.norm", D);
            if (mixes) {
                if (first_mix < 0) { first_mix = il; L.v_mix = 1; }
                else {
                    const pib_hlayer & F = hy->layers[first_mix];
                    if ((int64_t) F.kv_heads * F.vdim != G * Vd) { pib_set_error("model: layer %d mixes its values with layer %d's, which have another size", il, first_mix); return nullptr; }
                    L.v_mix = 2;
                    GET(px + "vmix");
                    L.lambda = v[0];
                }
                widen(hy->w_vfirst, G * Vd);
            }
            MAT(L.wo, px + "o", W, H * Vd);
            L.cache_id = hy->n_cache++;
            hy->cache_row.push_back((int) (G * (D + Vd)));
            widen(hy->w_proj, C); widen(hy->w_conv, C); widen(hy->w_q, H * D); widen(hy->w_att, H * Vd);
        } else if (ty->str == "wkv") {
            L.mixer = PIB_MIXER_WKV;
            L.kv_heads = L.heads; L.vdim = L.dim;
            const int64_t HD = H * D;
            L.w_rank = (int) src.dim(px + "w1", 0, (int64_t) jnum(mx, "decay_rank", 64));
            if (L.w_rank <= 0) { pib_set_error("model: layer %d: rank of the decay's projections", il); return nullptr; }
            std::vector<float> all;
            for (const char * s : { "r", "k", "v", "g", "w" }) { GET(px + "mu." + s, W); all.insert(all.end(), v.begin(), v.end()); }
            if (!(L.mu = upload_f32v(all))) return nullptr;
            all.clear();
            for (const char * s : { "r", "k", "v", "g" }) APPEND(all, px + s, HD, W);
            if (!(L.rkvg = upload_mat(all, 4 * HD, W, dtype, m))) return nullptr;
            MAT(L.w1, px + "w1", L.w_rank, W);
            MAT(L.w2, px + "w2", HD, L.w_rank);
            VEC(L.w0, px + "w0", HD);
            GET(px + "u", H, D);
            if (!(L.bonus = upload_f32v(v))) return nullptr;
            VEC(L.onorm, px + "norm", HD);
            MAT(L.wo, px + "o", W, HD);
            L.shift_off = state; state += (size_t) W;
            L.state_off = state; state += (size_t) (HD * D);
            widen(hy->w_shift, 5 * (int64_t) W); widen(hy->w_proj, 4 * HD); widen(hy->w_cq, L.w_rank); widen(hy->w_lat, HD); widen(hy->w_att, HD);
        } else if (ty->str == "delta") {
            L.mixer = PIB_MIXER_DELTA;
            const int64_t C = 2 * G * D + H * Vd, N = C + H * Vd + 2 * H;
            std::vector<float> all;
            APPEND(all, px + "q", G * D, W); APPEND(all, px + "k", G * D, W); APPEND(all, px + "v", H * Vd, W); APPEND(all, px + "g", H * Vd, W);
            APPEND(all, px + "b", H, W); APPEND(all, px + "a", H, W);
            if (!(L.qkv = upload_mat(all, N, W, dtype, m))) return nullptr;
            if (L.taps <= 0) L.taps = 1;
            all.clear();
            APPEND(all, px + "q.conv", G * D, L.taps); APPEND(all, px + "k.conv", G * D, L.taps); APPEND(all, px + "v.conv", H * Vd, L.taps);
            if (!(L.conv = upload_f32v(all))) return nullptr;
            L.tail_off = state; state += (size_t) (L.taps - 1) * C;
            VEC(L.a_log, px + "A_log", H);
            VEC(L.dt_bias, px + "dt_bias", H);
            VEC(L.onorm, px + "norm", Vd);
            MAT(L.wo, px + "o", W, H * Vd);
            L.state_off = state; state += (size_t) (H * D * Vd);
            widen(hy->w_proj, N); widen(hy->w_conv, C); widen(hy->w_cq, 2 * H); widen(hy->w_att, H * Vd);
        } else { pib_set_error("model: layer %d: unknown mixer '%s'", il, ty->str.c_str()); return nullptr; }
        if (ml && !ml->is_null()) {
            VEC(L.norm2, p + "norm2", W);
            const Json * kind = ml->get("kind");
            if (!kind || kind->str != "moe") { pib_set_error("model: layer %d: unknown mlp kind", il); return nullptr; }
            L.mlp = PIB_MLP_MOE; L.route = PIB_ROUTE_SIGMOID; L.expert = PIB_EXPERT_GLU_CLAMP;
            L.n_experts = (int) jnum(ml->get("router"), "experts", 0); L.top = (int) jnum(ml->get("router"), "top", 0);
            L.ff_e = (int) jnum(ml->get("expert"), "ff", 0); L.limit_e = (float) jnum(ml->get("expert"), "limit", INFINITY);
            const Json * sh = ml->get("shared");
            L.ff_s = sh && !sh->is_null() ? (int) jnum(sh, "ff", 0) : 0;
            L.limit_s = L.ff_s > 0 ? (float) jnum(sh, "limit", INFINITY) : 0.f;
            if (L.n_experts <= 0 || L.top <= 0 || L.top > L.n_experts || L.ff_e <= 0) { pib_set_error("model: layer %d: router.experts / router.top / expert.ff", il); return nullptr; }
            std::vector<float> ups, downs;
            for (int e = 0; e < L.n_experts; e++) {
                const std::string pe = pm + "e" + std::to_string(e) + ".";
                APPEND(ups, pe + "gate", L.ff_e, W); APPEND(ups, pe + "up", L.ff_e, W);
                APPEND(downs, pe + "down", W, L.ff_e);
            }
            if (!(L.e_up = upload_mat(ups, (int64_t) L.n_experts * 2 * L.ff_e, W, dtype, m)) || !(L.e_down = upload_mat(downs, (int64_t) L.n_experts * W, L.ff_e, dtype, m))) return nullptr;
            GET(pm + "router", L.n_experts, W);
            if (!(L.router = upload_mat(v, L.n_experts, W, PIB_TYPE_F32, m))) return nullptr;          // the router is always 32-bit
            if (L.ff_s > 0) {
                ups.clear();
                APPEND(ups, pm + "shared.gate", L.ff_s, W); APPEND(ups, pm + "shared.up", L.ff_s, W);
                L.s_gate = src.has(pm + "shared.sg") ? 1 : 0;
                if (L.s_gate) APPEND(ups, pm + "shared.sg", 1, W);
                if (!(L.s_up = upload_mat(ups, 2 * (int64_t) L.ff_s + L.s_gate, W, dtype, m))) return nullptr;
                MAT(L.s_down, pm + "shared.down", W, L.ff_s);
                widen(hy->w_proj, 2 * (int64_t) L.ff_s + 8);
            }
            widen(hy->w_pairs, L.top); widen(hy->w_eup, (int64_t) L.top * 2 * L.ff_e); widen(hy->w_router, L.n_experts);
        }
    }
    hy->state_floats = state ? state : 4;
#undef GET
#undef VEC
#undef MAT
#undef APPEND
    return mp.release();
}

// ---- the Lulenex builder ----------------------------------------------------------------------------------------------------------
// Sequential pre-norm layers (RMS norms whose weight is one number, a token shift in front of every mixer), mixers "mamba1" (selective
// state-space scan) and "parallel" (chunked softmax attention with a sink beside a linear attention with constant decays), dense xIELU
// feed-forwards, and a "loop": layers start .. stop-1 are walked `times` times with the same tensors.  The list the runtime walks holds one
// entry per layer RUN: entries of later walks point at the first walk's tensors and own only their cache rows and state.
// Tensor names: '<layer>.norm1|norm2|shift', '<layer>.mix.*', '<layer>.mlp.*', 'loop.in', 'loop.step', 'final.norm', 'embed', 'head'.
static pib_model * build_lulenex(const Json & cfg, TensorSource & src, int dtype) {
    std::unique_ptr<pib_model, void (*)(pib_model *)> mp(new pib_model(), pib_model_free);
    pib_model * m = mp.get();
    pib_hybrid * hy = new pib_hybrid();
    m->hy = hy;
    m->arch = 2; m->name = "Lulenex";
    bool ok = true;
    const int W = (int) jnum(&cfg, "width", 0, &ok), V = (int) jnum(&cfg, "vocab", 0, &ok);
    const Json * layers = cfg.get("layers");
    if (!ok || W <= 0 || V <= 0 || !layers || layers->kind != Json::ARR || layers->arr.empty()) { pib_set_error("model: config.json needs width, vocab and layers"); return nullptr; }
    const int n_base = (int) layers->arr.size();
    hy->dtype = dtype;
    hy->form = PIB_FORM_PRENORM;
    hy->eps = (float) jnum(cfg.get("norm"), "eps", 1e-6);
    hy->taps = 0;
    m->n_embd = W; m->n_vocab = V; m->layer_begin = 0;
    m->wtype = dtype; m->n_ctx_train = 1 << 20; m->n_head = 1; m->n_head_kv = 1; m->tok_bos = -1; m->tok_eos = -1;
    std::vector<float> v;
#define GET(name, ...) do { if (!src.get((name), { __VA_ARGS__ }, v)) return nullptr; } while (0)
#define VEC(dst, name, n) do { GET(name, (int64_t) (n)); if (!((dst) = upload_f32v(v))) return nullptr; } while (0)
#define MAT(dst, name, N, K) do { GET(name, (int64_t) (N), (int64_t) (K)); if (!((dst) = upload_mat(v, (N), (K), dtype, m))) return nullptr; } while (0)
#define APPEND(all, name, N, K) do { GET(name, (int64_t) (N), (int64_t) (K)); (all).insert((all).end(), v.begin(), v.end()); } while (0)
#define ONE(dst, name) do { GET(name); (dst) = v[0]; } while (0)
    MAT(m->tok_embd, "embed", V, W);
    ONE(hy->final_g, "final.norm");
    MAT(m->output, "head", V, W);
    // the walked run
    int lp_start = 0, lp_stop = 0, lp_times = 0;
    const Json * lp = cfg.get("loop");
    if (lp && !lp->is_null()) {
        lp_start = (int) jnum(lp, "start", 0); lp_stop = (int) jnum(lp, "stop", 0); lp_times = (int) jnum(lp, "times", 1);
        if (lp_start < 0 || lp_stop <= lp_start || lp_stop > n_base || lp_times < 1) { pib_set_error("model: loop start %d, stop %d, times %d over %d layers", lp_start, lp_stop, lp_times, n_base); return nullptr; }
        hy->loops = 1;
        MAT(hy->loop_in, "loop.in", W, 2 * (int64_t) W);
        GET("loop.step", (int64_t) lp_times, (int64_t) W);
        if (!(hy->loop_steps = upload_f32v(v))) return nullptr;
        hy->w_cat = 2 * W;
    }
    auto widen = [](int & a, int64_t b) { if (b > a) a = (int) b; };
    // ---- the layers as the file holds them ----
    std::vector<pib_hlayer> base((size_t) n_base);
    for (int il = 0; il < n_base; il++) {
        const Json & jl = layers->arr[il];
        pib_hlayer & L = base[il];
        const std::string p = "l" + std::to_string(il) + ".", px = p + "mix.", pm = p + "mlp.";
        const Json * ty = jl.get("type"), * mx = jl.get("mixer"), * ml = jl.get("mlp");
        if (!ty || ty->kind != Json::STR || !mx) { pib_set_error("model: layer %d needs type and mixer", il); return nullptr; }
        ONE(L.g1, p + "norm1");
        VEC(L.shift, p + "shift", W);
        if (ty->str == "mamba1") {
            L.mixer = PIB_MIXER_SSM;
            // sizes the configuration leaves out are read from the tensors' shapes
            L.inner = (int) jnum(mx, "inner", (double) (src.dim(px + "in", 0, 0) / 2)); L.n_state = (int) jnum(mx, "state", (double) src.dim(px + "A_log", 1, 0));
            L.dt_rank = (int) jnum(mx, "dt_rank", (double) src.dim(px + "dt", 1, 0)); L.taps = (int) jnum(mx, "conv", (double) src.dim(px + "conv", 1, 1));
            if (L.inner <= 0 || L.n_state <= 0 || L.dt_rank <= 0 || L.taps < 1) { pib_set_error("model: layer %d: inner / state / dt_rank / conv", il); return nullptr; }
            const int64_t I = L.inner, N = L.n_state, R = L.dt_rank;
            MAT(L.ssm_in, px + "in", 2 * I, W);
            GET(px + "conv", I, (int64_t) L.taps);
            if (!(L.conv = upload_f32v(v))) return nullptr;
            VEC(L.conv_b, px + "conv.b", I);
            MAT(L.ssm_x, px + "x", R + 2 * N, I);
            MAT(L.ssm_dt, px + "dt", I, R);
            VEC(L.dt_bias, px + "dt.b", I);
            GET(px + "A_log", I, N);
            for (float & a : v) a = (float) -exp((double) a);                  // A = -exp(A_log)
            if (!(L.ssm_a = upload_f32v(v))) return nullptr;
            VEC(L.ssm_d, px + "D", I);
            MAT(L.wo, px + "o", W, I);
            widen(hy->w_proj, 2 * I); widen(hy->w_conv, I); widen(hy->w_cq, (R + 2 * N + 3) & ~(int64_t) 3); widen(hy->w_lat, I); widen(hy->w_att, I);
        } else if (ty->str == "parallel") {
            L.mixer = PIB_MIXER_DUAL;
            const Json * a = mx->get("left"), * b = mx->get("right");
            if (!a || !b) { pib_set_error("model: layer %d: the mixer needs left and right", il); return nullptr; }
            L.heads = (int) jnum(a, "heads", (double) src.dim(px + "left.sink", 0, 0));
            L.dim = (int) jnum(a, "dim", L.heads > 0 ? (double) (src.dim(px + "left.q", 0, 0) / L.heads) : 0.0);
            L.kv_heads = (int) jnum(a, "kv_heads", L.dim > 0 ? (double) src.dim(px + "left.k", 0, (int64_t) L.heads * L.dim) / L.dim : 0.0); L.vdim = (int) jnum(a, "vdim", L.dim);
            if (L.heads <= 0 || L.dim <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads) { pib_set_error("model: layer %d: left heads / kv_heads / dim", il); return nullptr; }
            if (L.vdim != L.dim) { pib_set_error("model: layer %d: the values are the keys, so vdim (%d) must equal dim (%d)", il, L.vdim, L.dim); return nullptr; }
            L.scale = (float) jnum(a, "scale", 1.0 / sqrt((double) L.dim));
            const Json * mk = a->get("mask"), * rt = a->get("rot");
            L.window = mk && !mk->is_null() ? (int) jnum(mk, "size", 0) : 0;
            if (L.window > 0) L.mask = PIB_MASK_CHUNK; else L.window = 1 << 30;             // no mask: every earlier token is seen
            L.rot_base = (float) jnum(rt, "base", 10000.0); L.rot_dims = rt && !rt->is_null() ? (int) jnum(rt, "dims", L.dim) : 0;
            if (L.rot_dims < 0 || L.rot_dims > L.dim || (L.rot_dims & 1)) { pib_set_error("model: layer %d: rot.dims %d of %d", il, L.rot_dims, L.dim); return nullptr; }
            const Json * dc = b->get("decay");
            L.heads2 = (int) jnum(b, "heads", dc && dc->kind == Json::ARR ? (double) dc->arr.size() : 0.0);
            L.dim2 = (int) jnum(b, "dim", L.heads2 > 0 ? (double) (src.dim(px + "right.q", 0, 0) / L.heads2) : 0.0);
            L.vdim2 = (int) jnum(b, "vdim", L.heads2 > 0 ? (double) (src.dim(px + "right.v", 0, (int64_t) L.heads2 * L.dim2) / L.heads2) : 0.0);
            if (L.heads2 <= 0 || L.dim2 <= 0 || L.vdim2 <= 0 || !dc || dc->kind != Json::ARR || (int) dc->arr.size() != L.heads2) { pib_set_error("model: layer %d: right heads / dim / vdim / decay", il); return nullptr; }
            L.mix_a = (float) jnum(mx, "left_scale", 1.0); L.mix_b = (float) jnum(mx, "right_scale", 1.0);
            const int64_t H = L.heads, G = L.kv_heads, D = L.dim, H2 = L.heads2, D2 = L.dim2, V2 = L.vdim2;
            const int64_t rows = (H + G) * D + H + 2 * H2 * D2 + 2 * H2 * V2;
            std::vector<float> all, bias((size_t) rows, 0.f);
            APPEND(all, px + "left.q", H * D, W); APPEND(all, px + "left.k", G * D, W); APPEND(all, px + "left.g", H, W);
            APPEND(all, px + "right.q", H2 * D2, W); APPEND(all, px + "right.k", H2 * D2, W); APPEND(all, px + "right.v", H2 * V2, W); APPEND(all, px + "right.g", H2 * V2, W);
            if (!(L.qkv = upload_mat(all, rows, W, dtype, m))) return nullptr;
            GET(px + "left.q.b", H * D); std::copy(v.begin(), v.end(), bias.begin());
            GET(px + "left.k.b", G * D); std::copy(v.begin(), v.end(), bias.begin() + H * D);
            if (!(L.proj_bias = upload_f32v(bias))) return nullptr;
            VEC(L.sink, px + "left.sink", H);
            {   // one output matrix over the columns [softmax branch | linear branch]
                std::vector<float> lo, ro;
                GET(px + "left.o", W, H * D); lo = v;
                GET(px + "right.o", W, H2 * V2); ro = v;
                const int64_t Kc = H * D + H2 * V2;
                all.assign((size_t) (W * Kc), 0.f);
                for (int64_t r = 0; r < W; r++) {
                    std::copy(lo.begin() + r * H * D, lo.begin() + (r + 1) * H * D, all.begin() + r * Kc);
                    std::copy(ro.begin() + r * H2 * V2, ro.begin() + (r + 1) * H2 * V2, all.begin() + r * Kc + H * D);
                }
                if (!(L.wo = upload_mat(all, W, Kc, dtype, m))) return nullptr;
                GET(px + "left.o.b", W);
                for (float & x : v) x *= L.mix_a;
                if (!(L.o_bias = upload_f32v(v))) return nullptr;
                widen(hy->w_att, Kc);
            }
            VEC(L.onorm, px + "right.norm", H2 * V2);
            v.resize((size_t) H2);
            for (int64_t h = 0; h < H2; h++) v[(size_t) h] = (float) dc->arr[(size_t) h].num;
            if (!(L.decay = upload_f32v(v))) return nullptr;
            widen(hy->w_proj, (rows + 3) & ~(int64_t) 3); widen(hy->w_q, H * D); widen(hy->w_lat, H * D); widen(hy->w_conv, H2 * V2);
        } else { pib_set_error("model: layer %d: unknown mixer '%s'", il, ty->str.c_str()); return nullptr; }
        if (ml && !ml->is_null()) {
            const Json * kind = ml->get("kind");
            if (kind && kind->str != "dense") { pib_set_error("model: layer %d: unknown mlp kind", il); return nullptr; }
            L.mlp = PIB_MLP_XIELU; L.ff = (int) jnum(ml, "ff", (double) src.dim(pm + "up", 0, 0));
            if (L.ff <= 0) { pib_set_error("model: layer %d: mlp.ff", il); return nullptr; }
            ONE(L.g2, p + "norm2");
            MAT(L.up, pm + "up", L.ff, W);
            MAT(L.down, pm + "down", W, L.ff);
            GET(pm + "act", 2);
            L.act[0] = v[0]; L.act[1] = v[1];
            auto softplus = [](double z) { return z > 30 ? z : log1p(exp(z)); };
            L.act[2] = (float) softplus((double) v[0]); L.act[3] = (float) (0.5 + softplus((double) v[1]));      // the two numbers the matmul's epilogue uses
            widen(hy->w_proj, L.ff);
        }
    }
    // ---- the runs: each with cache rows and state of its own ----
    std::vector<std::pair<int, int>> order;                                       // (layer, walk or -1)
    for (int il = 0; il < (hy->loops ? lp_start : n_base); il++) order.push_back({ il, -1 });
    if (hy->loops) {
        for (int r = 0; r < lp_times; r++) for (int il = lp_start; il < lp_stop; il++) order.push_back({ il, r });
        for (int il = lp_stop; il < n_base; il++) order.push_back({ il, -1 });
    }
    std::vector<int> first((size_t) n_base, -1);
    size_t state = 0;
    for (size_t ir = 0; ir < order.size(); ir++) {
        const int il = order[ir].first, walk = order[ir].second;
        pib_hlayer L = base[(size_t) il];
        if (first[(size_t) il] >= 0) L.weights_of = first[(size_t) il]; else first[(size_t) il] = (int) ir;
        if (walk >= 0 && il == lp_start) { L.loop_in = hy->loop_in; L.loop_step = hy->loop_steps + (size_t) walk * W; }
        L.shift_off = state; state += (size_t) W;
        if (L.mixer == PIB_MIXER_SSM) {
            L.tail_off = state; state += (size_t) (L.taps - 1) * L.inner;
            L.state_off = state; state += (size_t) L.inner * L.n_state;
        } else {
            L.state_off = state; state += (size_t) L.heads2 * L.dim2 * L.vdim2;
            L.cache_id = hy->n_cache++;
            hy->cache_row.push_back(2 * L.kv_heads * L.dim);
            L.rope_id = -1;
            for (size_t i = 0; i < hy->ropes.size(); i++) if (hy->ropes[i].base == L.rot_base && hy->ropes[i].dims == L.rot_dims) L.rope_id = (int) i;
            if (L.rope_id < 0) { L.rope_id = (int) hy->ropes.size(); hy->ropes.push_back({ L.rot_base, L.rot_dims }); }
        }
        hy->layers.push_back(L);
    }
    m->n_layer = (int) hy->layers.size(); m->layer_end = m->n_layer;
    hy->state_floats = state ? state : 4;
#undef GET
#undef VEC
#undef MAT
#undef APPEND
#undef ONE
    return mp.release();
}

// ---- the Putazen builder ----------------------------------------------------------------------------------------------------------
// Layers with hyper-connections (several residual streams; a sublayer reads a weighted sum of them through a LayerNorm with weight and
// bias), mixers "mamba2" (state-space duality), "attention" (differential attention: two softmax maps per head, biases, partial rotation in
// halves with optional YaRN scaling) and "latent_attention" (keys and values from a cached latent, no query latent, rotation in adjacent
// pairs), dense clamped gated feed-forwards, and an optional "loop": layers start .. stop-1 are walked `times` times with the same
// tensors, nothing happening between the walks.  The list the runtime walks holds one entry per layer RUN, as for Lulenex.
// Tensor names: '<layer>.norm1|norm2' (+ '.b'), '<layer>.hc1|hc2.in|out|mix', '<layer>.mix.*', '<layer>.mlp.gate|up|down', 'final.norm' (+ '.b'), 'embed', 'head'.
static pib_model * build_putazen(const Json & cfg, TensorSource & src, int dtype) {
    std::unique_ptr<pib_model, void (*)(pib_model *)> mp(new pib_model(), pib_model_free);
    pib_model * m = mp.get();
    pib_hybrid * hy = new pib_hybrid();
    m->hy = hy;
    m->arch = 2; m->name = "Putazen";
    bool ok = true;
    const int W = (int) jnum(&cfg, "width", 0, &ok), V = (int) jnum(&cfg, "vocab", 0, &ok);
    const Json * layers = cfg.get("layers");
    if (!ok || W <= 0 || V <= 0 || !layers || layers->kind != Json::ARR || layers->arr.empty()) { pib_set_error("model: config.json needs width, vocab and layers"); return nullptr; }
    const int n_base = (int) layers->arr.size(), S = (int) jnum(&cfg, "streams", 1);
    if (S < 1 || S > 16) { pib_set_error("model: streams %d (1 to 16)", S); return nullptr; }
    hy->dtype = dtype;
    hy->form = PIB_FORM_HYPER;
    hy->streams = S;
    hy->eps = (float) jnum(cfg.get("norm"), "eps", 1e-5);
    hy->embd_scale = (float) jnum(cfg.get("embedding"), "scale", 1.0);
    hy->taps = 0;
    m->n_embd = W; m->n_vocab = V; m->layer_begin = 0;
    m->wtype = dtype; m->n_ctx_train = 1 << 20; m->n_head = 1; m->n_head_kv = 1; m->tok_bos = -1; m->tok_eos = -1;
    std::vector<float> v;
#define GET(name, ...) do { if (!src.get((name), { __VA_ARGS__ }, v)) return nullptr; } while (0)
#define VEC(dst, name, n) do { GET(name, (int64_t) (n)); if (!((dst) = upload_f32v(v))) return nullptr; } while (0)
#define MAT(dst, name, N, K) do { GET(name, (int64_t) (N), (int64_t) (K)); if (!((dst) = upload_mat(v, (N), (K), dtype, m))) return nullptr; } while (0)
#define APPEND(all, name, ...) do { GET(name, __VA_ARGS__); (all).insert((all).end(), v.begin(), v.end()); } while (0)
    MAT(m->tok_embd, "embed", V, W);
    VEC(m->output_norm, "final.norm", W);
    VEC(hy->final_b, "final.norm.b", W);
    MAT(m->output, "head", V, W);
    int lp_start = 0, lp_stop = 0, lp_times = 0;
    const Json * lp = cfg.get("loop");
    if (lp && !lp->is_null()) {
        lp_start = (int) jnum(lp, "start", 0); lp_stop = (int) jnum(lp, "stop", 0); lp_times = (int) jnum(lp, "times", 1);
        if (lp_start < 0 || lp_stop <= lp_start || lp_stop > n_base || lp_times < 1) { pib_set_error("model: loop start %d, stop %d, times %d over %d layers", lp_start, lp_stop, lp_times, n_base); return nullptr; }
    }
    auto widen = [](int & a, int64_t b) { if (b > a) a = (int) b; };
    // [in (S) | out (S) | mix (S x S)] of one sublayer
    auto hyper = [&](const std::string & pre, float *& dst) -> bool {
        std::vector<float> all;
        if (!src.get(pre + "in", { (int64_t) S }, v)) return false;
        all = v;
        if (!src.get(pre + "out", { (int64_t) S }, v)) return false;
        all.insert(all.end(), v.begin(), v.end());
        if (!src.get(pre + "mix", { (int64_t) S, (int64_t) S }, v)) return false;
        all.insert(all.end(), v.begin(), v.end());
        return (dst = upload_f32v(all)) != nullptr;
    };
    std::vector<pib_hlayer> base((size_t) n_base);
    for (int il = 0; il < n_base; il++) {
        const Json & jl = layers->arr[il];
        pib_hlayer & L = base[il];
        const std::string p = "l" + std::to_string(il) + ".", px = p + "mix.", pm = p + "mlp.";
        const Json * ty = jl.get("type"), * mx = jl.get("mixer"), * ml = jl.get("mlp");
        if (!ty || ty->kind != Json::STR || !mx) { pib_set_error("model: layer %d needs type and mixer", il); return nullptr; }
        VEC(L.norm1, p + "norm1", W);
        VEC(L.norm1_b, p + "norm1.b", W);
        if (!hyper(p + "hc1.", L.hc1)) return nullptr;
        L.heads = (int) jnum(mx, "heads", 0); L.vdim = (int) jnum(mx, "vdim", 0);
        if (L.heads <= 0 || L.vdim <= 0) { pib_set_error("model: layer %d: heads / vdim", il); return nullptr; }
        const int64_t H = L.heads, Vd = L.vdim;
        const Json * rt = mx->get("rot");
        if (ty->str == "mamba2") {
            L.mixer = PIB_MIXER_MAMBA2;
            L.n_state = (int) jnum(mx, "state", 0); L.kv_heads = (int) jnum(mx, "groups", 1); L.taps = (int) jnum(mx, "conv", 1); L.norm_groups = (int) jnum(mx, "norm_groups", 1);
            const int64_t I = H * Vd, GN = (int64_t) L.kv_heads * L.n_state, C = I + 2 * GN;
            if (L.n_state <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads || L.taps < 1 || L.norm_groups < 1 || I % L.norm_groups) {
                pib_set_error("model: layer %d: state / groups / conv / norm_groups", il); return nullptr;
            }
            MAT(L.ssm_in, px + "in", I + C + H, W);
            GET(px + "conv", C, (int64_t) L.taps);
            if (!(L.conv = upload_f32v(v))) return nullptr;
            VEC(L.conv_b, px + "conv.b", C);
            VEC(L.dt_bias, px + "dt_bias", H);
            VEC(L.a_log, px + "A_log", H);
            VEC(L.ssm_d, px + "D", H);
            VEC(L.onorm, px + "norm", I);
            MAT(L.wo, px + "o", W, I);
            widen(hy->w_proj, (I + C + H + 3) & ~(int64_t) 3); widen(hy->w_conv, C); widen(hy->w_cq, 3 * H); widen(hy->w_att, I);
        } else if (ty->str == "attention") {
            L.mixer = PIB_MIXER_DIFF;
            L.maps = 2;
            L.dim = (int) jnum(mx, "dim", 0); L.kv_heads = (int) jnum(mx, "kv_heads", L.heads);
            if (L.dim <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads) { pib_set_error("model: layer %d: dim / kv_heads", il); return nullptr; }
            const int64_t G = L.kv_heads, D = L.dim, NQ = H * 2 * D, NK = G * 2 * D, NV = G * Vd;
            L.scale = (float) jnum(mx, "scale", 1.0 / sqrt((double) D));
            L.window = 1 << 30;
            const double diff = jnum(mx, "diff", 0.0);
            L.rot_base = (float) jnum(rt, "base", 10000.0); L.rot_dims = rt && !rt->is_null() ? (int) jnum(rt, "dims", (double) D) : 0;
            L.rot_pairs = PIB_PAIR_HALF;
            if (L.rot_dims < 0 || L.rot_dims > L.dim || (L.rot_dims & 1)) { pib_set_error("model: layer %d: rot.dims %d of %d", il, L.rot_dims, L.dim); return nullptr; }
            std::vector<float> all, bias;
            APPEND(all, px + "q", NQ, W); APPEND(all, px + "k", NK, W); APPEND(all, px + "v", NV, W);
            if (!(L.qkv = upload_mat(all, NQ + NK + NV, W, dtype, m))) return nullptr;
            APPEND(bias, px + "q.b", NQ); APPEND(bias, px + "k.b", NK); APPEND(bias, px + "v.b", NV);
            if (!(L.proj_bias = upload_f32v(bias))) return nullptr;
            double dots[4];
            {
                std::vector<float> a, b;
                const char * names[4][2] = { { "lq1", "lk1" }, { "lq2", "lk2" } };
                for (int i = 0; i < 2; i++) {
                    GET(px + names[i][0], D); a = v;
                    GET(px + names[i][1], D); b = v;
                    dots[i] = 0;
                    for (int64_t d = 0; d < D; d++) dots[i] += (double) a[(size_t) d] * (double) b[(size_t) d];
                }
            }
            L.diff_lambda = (float) (exp(dots[0]) - exp(dots[1]) + diff);       // a scalar shared by every head of the layer
            L.diff_out = (float) (1.0 - diff);
            MAT(L.wo, px + "o", W, H * Vd);
            widen(hy->w_proj, (NQ + NK + NV + 3) & ~(int64_t) 3); widen(hy->w_q, NQ); widen(hy->w_lat, H * 2 * Vd); widen(hy->w_att, H * Vd);
        } else if (ty->str == "latent_attention") {
            L.mixer = PIB_MIXER_LATENT;
            L.dim = (int) jnum(mx, "dim", 0); L.rot_dim = (int) jnum(mx, "rot_dim", 0); L.kv_rank = (int) jnum(mx, "kv_rank", 0); L.q_rank = 0;
            if (L.dim <= 0 || L.rot_dim < 0 || (L.rot_dim & 1) || L.kv_rank <= 0) { pib_set_error("model: layer %d: dim / rot_dim / kv_rank", il); return nullptr; }
            L.scale = (float) jnum(mx, "scale", 1.0 / sqrt((double) (L.dim + L.rot_dim)));
            L.window = 1 << 30;
            L.rot_base = (float) jnum(rt, "base", 10000.0); L.rot_dims = L.rot_dim;              // the rotated vector is the rot_dim part, all of it
            L.rot_pairs = PIB_PAIR_ADJACENT;
            const int64_t D = L.dim, rd = L.rot_dim, R = L.kv_rank;
            std::vector<float> all;
            APPEND(all, px + "q", H * (D + rd), W); APPEND(all, px + "dkv", R + rd, W);
            if (!(L.dqkv = upload_mat(all, H * (D + rd) + R + rd, W, dtype, m))) return nullptr;
            VEC(L.dkv_norm, px + "dkv.norm", R);
            GET(px + "uk", H * D, R);
            {   // per head W_uk^T: [kv_rank][dim]
                std::vector<float> tr((size_t) (H * D * R));
                for (int64_t h = 0; h < H; h++) for (int64_t d = 0; d < D; d++) for (int64_t r = 0; r < R; r++) tr[(size_t) ((h * R + r) * D + d)] = v[(size_t) ((h * D + d) * R + r)];
                if (!(L.ukT = upload_mat(tr, H * R, D, dtype, m))) return nullptr;
            }
            MAT(L.uv, px + "uv", H * Vd, R);
            MAT(L.wo, px + "o", W, H * Vd);
            widen(hy->w_proj, (H * (D + rd) + R + rd + 3) & ~(int64_t) 3); widen(hy->w_lat, H * R); widen(hy->w_att, H * Vd);
        } else { pib_set_error("model: layer %d: unknown mixer '%s'", il, ty->str.c_str()); return nullptr; }
        if (ml && !ml->is_null()) {
            const Json * kind = ml->get("kind");
            if (kind && kind->str != "dense") { pib_set_error("model: layer %d: unknown mlp kind", il); return nullptr; }
            L.mlp = PIB_MLP_GLU; L.ff = (int) jnum(ml, "ff", (double) src.dim(pm + "up", 0, 0)); L.limit_s = (float) jnum(ml, "limit", INFINITY);
            if (L.ff <= 0) { pib_set_error("model: layer %d: mlp.ff", il); return nullptr; }
            VEC(L.norm2, p + "norm2", W);
            VEC(L.norm2_b, p + "norm2.b", W);
            if (!hyper(p + "hc2.", L.hc2)) return nullptr;
            // gate row i and up row i next to each other: the matmul's paired epilogue forms the activation on the way out
            std::vector<float> all((size_t) 2 * L.ff * W);
            GET(pm + "gate", (int64_t) L.ff, W);
            for (int64_t i = 0; i < L.ff; i++) memcpy(&all[(size_t) (2 * i) * W], &v[(size_t) i * W], (size_t) W * 4);
            GET(pm + "up", (int64_t) L.ff, W);
            for (int64_t i = 0; i < L.ff; i++) memcpy(&all[(size_t) (2 * i + 1) * W], &v[(size_t) i * W], (size_t) W * 4);
            if (!(L.up = upload_mat(all, 2 * (int64_t) L.ff, W, dtype, m))) return nullptr;
            MAT(L.down, pm + "down", W, L.ff);
            widen(hy->w_proj, (int64_t) L.ff);
        }
    }
    // ---- the runs: each with cache rows and state of its own ----
    std::vector<int> order;
    for (int il = 0; il < (lp_times ? lp_start : n_base); il++) order.push_back(il);
    if (lp_times) {
        for (int r = 0; r < lp_times; r++) for (int il = lp_start; il < lp_stop; il++) order.push_back(il);
        for (int il = lp_stop; il < n_base; il++) order.push_back(il);
    }
    std::vector<int> first((size_t) n_base, -1);
    size_t state = 0;
    for (size_t ir = 0; ir < order.size(); ir++) {
        const int il = order[ir];
        pib_hlayer L = base[(size_t) il];
        if (first[(size_t) il] >= 0) L.weights_of = first[(size_t) il]; else first[(size_t) il] = (int) ir;
        if (L.mixer == PIB_MIXER_MAMBA2) {
            L.tail_off = state; state += (size_t) (L.taps - 1) * ((size_t) L.heads * L.vdim + 2 * (size_t) L.kv_heads * L.n_state);
            L.state_off = state; state += (size_t) L.heads * L.n_state * L.vdim;
        } else {
            L.cache_id = hy->n_cache++;
            hy->cache_row.push_back(L.mixer == PIB_MIXER_DIFF ? L.kv_heads * (L.maps * L.dim + L.vdim) : L.kv_rank + L.rot_dim);
            pib_hybrid::Rope r = { L.rot_base, L.rot_dims };
            const Json * mx = layers->arr[(size_t) il].get("mixer"), * rt = mx ? mx->get("rot") : nullptr, * sc = rt ? rt->get("scaling") : nullptr;
            if (L.mixer == PIB_MIXER_DIFF && sc && !sc->is_null()) {
                r.factor = jnum(sc, "factor", 1.0); r.original = jnum(sc, "original", 1.0); r.fast = jnum(sc, "fast", 32.0); r.slow = jnum(sc, "slow", 1.0);
                if (!(r.factor > 0) || !(r.original > 0) || !(r.fast > 0) || !(r.slow > 0)) { pib_set_error("model: layer %d: rot.scaling", il); return nullptr; }
            }
            L.rope_id = -1;
            for (size_t i = 0; i < hy->ropes.size(); i++) {
                const pib_hybrid::Rope & o = hy->ropes[i];
                if (o.base == r.base && o.dims == r.dims && o.factor == r.factor && o.original == r.original && o.fast == r.fast && o.slow == r.slow) L.rope_id = (int) i;
            }
            if (L.rope_id < 0) { L.rope_id = (int) hy->ropes.size(); hy->ropes.push_back(r); }
        }
        hy->layers.push_back(L);
    }
    m->n_layer = (int) hy->layers.size(); m->layer_end = m->n_layer;
    hy->state_floats = state ? state : 4;
#undef GET
#undef VEC
#undef MAT
#undef APPEND
    return mp.release();
}

// ---- registry: config.json "architecture" -> builder ---------------------------------------------------------------------------------
struct DirArch { const char * name; pib_model * (*build)(const Json &, TensorSource &, int); };
static const DirArch DIR_ARCHS[] = { { "Rapisun", build_rapisun }, { "Fabivik", build_fabivik }, { "Lulenex", build_lulenex }, { "Putazen", build_putazen } };

static pib_model * build_from_config(const Json & cfg, TensorSource & src, int dtype) {
    const Json * a = cfg.get("architecture");
    if (cfg.kind != Json::OBJ || !a || a->kind != Json::STR) { pib_set_error("model: config.json has no \"architecture\""); return nullptr; }
    for (const DirArch & d : DIR_ARCHS) if (a->str == d.name) return d.build(cfg, src, dtype);
    pib_set_error("model: unknown architecture '%s'", a->str.c_str());
    return nullptr;
}

pib_model * pib_model_load_dir(const char * dir, int dtype) {
    std::string d(dir), txt;
    if (d.size() > 12 && !d.compare(d.size() - 12, 12, "/config.json")) d.resize(d.size() - 12);
    if (!read_file(d + "/config.json", txt)) { pib_set_error("model: cannot read %s/config.json", d.c_str()); return nullptr; }
    Json cfg;
    if (!json_parse(txt.data(), txt.size(), cfg)) { pib_set_error("model: %s/config.json is not JSON", d.c_str()); return nullptr; }
    SafeTensors st;
    if (!st.open(d + "/model.safetensors")) return nullptr;
    TensorSource src;
    src.st = &st;
    return build_from_config(cfg, src, dtype);
}

pib_model * pib_hybrid_synthetic(const char * config_json, uint64_t seed, int dtype) {
    Json cfg;
    if (!json_parse(config_json, strlen(config_json), cfg)) { pib_set_error("model: the configuration is not JSON"); return nullptr; }
    TensorSource src;
    src.seed = seed;
    return build_from_config(cfg, src, dtype);
}

void pib_hybrid_model_free(pib_model * m) {
    pib_hybrid * hy = m->hy;
    if (!hy) return;
    for (pib_hlayer & L : hy->layers) {
        if (L.weights_of >= 0) continue;                  // a later walk of the same layer: the tensors are the first walk's
        for (float * f : { L.norm1, L.norm2, L.canon, L.dq_norm, L.dkv_norm, L.sink, L.f_bias, L.lower, L.onorm, L.conv, L.q_norm, L.k_norm, L.mu, L.w0, L.bonus, L.a_log,
                           L.dt_bias, L.shift, L.conv_b, L.ssm_a, L.ssm_d, L.proj_bias, L.o_bias, L.decay, L.hc1, L.hc2, L.norm1_b, L.norm2_b }) if (f) cudaFree(f);
        for (pib_weight * w : { L.dqkv, L.uq, L.ukT, L.uv, L.wo, L.qfv, L.up, L.down, L.e_up, L.e_down, L.router, L.s_up, L.s_down, L.qkv, L.rkvg, L.w1, L.w2, L.ssm_in, L.ssm_x,
                                L.ssm_dt }) if (w) pib_weight_free(w);
    }
    if (hy->embd_norm) cudaFree(hy->embd_norm);
    if (hy->final_b) cudaFree(hy->final_b);
    if (hy->loop_in) pib_weight_free(hy->loop_in);
    if (hy->loop_steps) cudaFree(hy->loop_steps);
    delete hy;
    m->hy = nullptr;
}
