// mixer_kernels.cu -- more parts for layer-list models (hybrid.cuh), all fp32:
//
//   embedding rows times a constant; RMS norm with a weight stored around zero, two norms of the same row in one pass
//   windowed softmax attention over cached key / value heads: per-head RMS norm of queries and keys, value mixing with the values an
//       earlier layer computed for the same token, grouped queries, an optional sink logit
//   RWKV-style time mixing: the five token-shift mixes, the per-channel decay, and the recurrence
//       o_t = (S + diag(u) k_t v_t^T)^T r_t,  S <- diag(w_t) S + k_t v_t^T
//   the gated delta rule: S <- g_t S,  e_t = beta_t (v_t - S^T k_t),  S <- S + k_t e_t^T,  o_t = S^T q_t
//   RMS norm of each head's output times a weight times silu(gate)
//   clamped gated experts: y = a sigmoid(1.702 a) (b + 1), a = min(gate, limit), b = clamp(up, -limit, limit)
//   the parallel layer's sum: x += mixer + shared expert * sigmoid(gate logit) + routed experts
#include "hybrid.cuh"

#include <cuda_bf16.h>

#define CKL() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) { pib_set_error("%s:%d: launch failed: %s", __FILE__, __LINE__, cudaGetErrorString(e__)); return PIB_ERR_CUDA; } } while (0)

__device__ __forceinline__ float mk_block_sum(float v, float * red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}
__device__ __forceinline__ float mk_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float mk_silu(float z) { return z / (1.0f + expf(-z)); }

// ---- embedding, norms ------------------------------------------------------------------------------------------------------------
template <typename WT>
__global__ void __launch_bounds__(256) embed_scale_kernel(const WT * __restrict__ embd, const int32_t * __restrict__ tok, float scale, int W, float * __restrict__ x, int copies) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const WT * r = embd + (size_t) tok[blockIdx.x] * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = (float) r[i] * scale;
        for (int s = 0; s < copies; s++) x[((size_t) blockIdx.x * copies + s) * W + i] = v;
    }
}
// copies: every token's row is written that many times, one after the other (the residual streams of hyper-connections start equal)
int pib_embed_scale(const pib_weight * embd, const int32_t * tok, float scale, int T, int W, float * x, cudaStream_t st, int copies) {
    if (embd->type == PIB_TYPE_BF16) pib_launch(embed_scale_kernel<__nv_bfloat16>, dim3(T), dim3(256), (size_t) 0, st, (const __nv_bfloat16 *) embd->base, tok, scale, W, x, copies);
    else                             pib_launch(embed_scale_kernel<float>, dim3(T), dim3(256), (size_t) 0, st, (const float *) embd->base, tok, scale, W, x, copies);
    CKL();
    return PIB_OK;
}

// h1 = x / sqrt(mean(x^2) + eps) * (1 + w1) * out_scale, and (w2 != null) h2 the same with w2: both norms of a parallel layer read x once
__global__ void __launch_bounds__(256) rms_norm2_kernel(const float * __restrict__ x, const float * __restrict__ w1, const float * __restrict__ w2, float eps, float out_scale,
                                                        int W, float * __restrict__ h1, float * __restrict__ h2) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float srow[];
    __shared__ float red[32];
    const float * r = x + (size_t) blockIdx.x * W;
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) { const float v = r[i]; srow[i] = v; s = fmaf(v, v, s); }
    const float inv = out_scale / sqrtf(mk_block_sum(s, red) / W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = srow[i] * inv;
        h1[(size_t) blockIdx.x * W + i] = v * (1.0f + w1[i]);
        if (w2) h2[(size_t) blockIdx.x * W + i] = v * (1.0f + w2[i]);
    }
}
int pib_rms_norm2(const float * x, const float * w1, const float * w2, float eps, float out_scale, int T, int W, float * h1, float * h2, cudaStream_t st) {
    pib_launch(rms_norm2_kernel, dim3(T), dim3(256), (size_t) W * 4, st, x, w1, w2, eps, out_scale, W, h1, h2);
    CKL();
    return PIB_OK;
}

// ---- windowed attention: what follows the convolution ------------------------------------------------------------------------------
// cv[t] = [q (H*D) | k (G*D) | v (G*V)] after the convolution.  q[t][h] = RMS(q_h) * q_norm; the token's cell gets
// [RMS(k_g) * k_norm (G*D) | v' (G*V)], v' = v, or (1 - lambda) v + lambda v_first for a later mixing layer; the first mixing layer
// leaves its v in vfirst.  One warp per head (query heads, then key heads), the block's threads over the values.
__global__ void __launch_bounds__(256) swa_prep_kernel(const float * __restrict__ cv, int ldc, int H, int G, int D, int V, const float * __restrict__ q_norm,
                                                       const float * __restrict__ k_norm, float eps, int v_mix, float lambda, const int32_t * __restrict__ cell,
                                                       float * __restrict__ q, float * __restrict__ cache, int cache_row, float * __restrict__ vfirst) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float * r = cv + (size_t) t * ldc;
    float * row = cache + (size_t) cell[t] * cache_row;
    for (int hh = warp; hh < H + G; hh += nw) {
        const float * src = r + (size_t) hh * D;
        const float * w = hh < H ? q_norm : k_norm;
        float * dst = hh < H ? q + ((size_t) t * H + hh) * D : row + (size_t) (hh - H) * D;
        float s = 0.f;
        for (int i = lane; i < D; i += 32) s = fmaf(src[i], src[i], s);
        const float inv = 1.0f / sqrtf(warp_sum(s) / D + eps);
        for (int i = lane; i < D; i += 32) dst[i] = src[i] * inv * w[i];
    }
    const float * v = r + (size_t) (H + G) * D;
    for (int i = threadIdx.x; i < G * V; i += blockDim.x) {
        float x = v[i];
        if (v_mix == 1) vfirst[(size_t) t * G * V + i] = x;
        else if (v_mix == 2) x = (1.0f - lambda) * x + lambda * vfirst[(size_t) t * G * V + i];
        row[(size_t) G * D + i] = x;
    }
}
int pib_swa_prep(const float * cv, int ldc, const pib_hlayer & L, float eps, const pib_hbatch & b, float * q, float * cache, int cache_row, float * vfirst, cudaStream_t st) {
    pib_launch(swa_prep_kernel, dim3(b.T), dim3(256), (size_t) 0, st, cv, ldc, L.heads, L.kv_heads, L.dim, L.vdim, L.q_norm, L.k_norm, eps, L.v_mix, L.lambda, b.cell, q, cache,
               cache_row, vfirst);
    CKL();
    return PIB_OK;
}

// grid (token, head group); a block holds HPB query heads x KS key shares, one warp each.  A warp walks its share of the window
// [max(0, p - window + 1), p] (chunk mask: of the token's chunk [p - p % window, p]) through the slot's position -> cell table, keeps a running maximum / denominator / weighted sum of value
// rows, and the shares of a head are merged in shared memory.  A sink (optional) is one more logit without a row: the running state of
// share 0 starts at (max = sink, denominator = 1).
template <int RPL>
__global__ void __launch_bounds__(512) kv_attn_kernel(const float * __restrict__ q, int H, int G, int maps, int D, int V, float scale, int window, int mask, const float * __restrict__ sink,
                                                      const int32_t * __restrict__ pos, const int32_t * __restrict__ slot, const float * __restrict__ cache, int cache_row,
                                                      const int32_t * __restrict__ cellmap, int n_ctx, int HPB, int KS, float * __restrict__ out,
                                                      const int32_t * __restrict__ skip) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float sm[];                 // [HPB * KS][V + 2] partial states
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (skip && skip[t]) return;                  // this token's segment goes through the matmul form
    const int hl = warp / KS, ks = warp % KS, h = blockIdx.y * HPB + hl;
    const int p = pos[t], lo = mask == PIB_MASK_CHUNK ? p - p % window : max(0, p - window + 1);
    const bool live = h < H;
    float qv[RPL], acc[RPL];
    float m = -INFINITY, l = 0.f;
    if (live) {
        // H counts query rows: `maps` rows per head, next to each other; row h reads map h % maps of its key / value head's keys and that head's values
        const int g = h / maps / (H / (G * maps)), mp = h % maps;
        const float * qp = q + ((size_t) t * H + h) * D;
#pragma unroll
        for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; qv[i] = r < D ? qp[r] * scale : 0.f; acc[i] = 0.f; }
        if (ks == 0 && sink) { m = sink[h]; l = 1.f; }
        const int32_t * map = cellmap + (size_t) slot[t] * n_ctx;
        const size_t ko = (size_t) (g * maps + mp) * D, vo = (size_t) G * maps * D + (size_t) g * V;
        for (int j = lo + ks; j <= p; j += KS) {
            const float * row = cache + (size_t) map[j] * cache_row;
            float s = 0.f, c[RPL];
#pragma unroll
            for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; if (r < D) s = fmaf(qv[i], row[ko + r], s); c[i] = r < V ? row[vo + r] : 0.f; }
            s = warp_sum(s);
            const float mn = fmaxf(m, s), a = expf(m - mn), e = expf(s - mn);         // m == -inf only before the first key: a = 0
            l = l * a + e;
#pragma unroll
            for (int i = 0; i < RPL; i++) acc[i] = fmaf(acc[i], a, e * c[i]);
            m = mn;
        }
        float * part = sm + (size_t) warp * (V + 2);
#pragma unroll
        for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; if (r < V) part[r] = acc[i]; }
        if (lane == 0) { part[V] = m; part[V + 1] = l; }
    }
    __syncthreads();
    if (live && ks == 0) {
        const float * base = sm + (size_t) (hl * KS) * (V + 2);
        float M = -INFINITY;
        for (int k = 0; k < KS; k++) M = fmaxf(M, base[(size_t) k * (V + 2) + V]);
        float Lsum = 0.f, o[RPL];
#pragma unroll
        for (int i = 0; i < RPL; i++) o[i] = 0.f;
        for (int k = 0; k < KS; k++) {
            const float * pk = base + (size_t) k * (V + 2);
            const float   mk = pk[V];
            if (mk == -INFINITY) continue;           // a share that saw no key
            const float f = expf(mk - M);
            Lsum = fmaf(pk[V + 1], f, Lsum);
#pragma unroll
            for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; if (r < V) o[i] = fmaf(pk[r], f, o[i]); }
        }
        const float inv = 1.0f / Lsum;
        float * op = out + ((size_t) t * H + h) * V;
#pragma unroll
        for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; if (r < V) op[r] = o[i] * inv; }
    }
}

int pib_kv_attention(const float * q, const pib_hlayer & L, const pib_hbatch & b, const float * cache, int cache_row, const int32_t * cellmap, int n_ctx, float * out,
                     const int32_t * skip, cudaStream_t st) {
    const int H = L.heads * L.maps, V = L.vdim, R = L.dim > L.vdim ? L.dim : L.vdim;
    const int HPB = (long long) b.T * H <= 1024 ? 1 : (H < 4 ? H : 4);
    int KS = 16 / HPB;
    if (L.window < 64) KS = 1;
    const size_t smem = (size_t) HPB * KS * (V + 2) * 4;
    dim3 grid((unsigned) b.T, (unsigned) ((H + HPB - 1) / HPB));
    const int threads = HPB * KS * 32;
#define KA_GO(RPL) do {                                                                                                              \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kv_attn_kernel<RPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);   \
        pib_launch(kv_attn_kernel<RPL>, dim3(grid), dim3(threads), (size_t) smem, st, q, H, L.kv_heads, L.maps, L.dim, V, L.scale, L.window, L.mask, (const float *) L.sink, b.pos, b.slot, cache, \
                   cache_row, cellmap, n_ctx, HPB, KS, out, skip);                                                                  \
    } while (0)
    if (R <= 32) KA_GO(1); else if (R <= 64) KA_GO(2); else if (R <= 128) KA_GO(4); else if (R <= 256) KA_GO(8); else if (R <= 512) KA_GO(16);
    else { pib_set_error("attention: head size %d (max 512)", R); return PIB_ERR_UNSUPP; }
#undef KA_GO
    CKL();
    return PIB_OK;
}

// ---- the same attention as matmuls (long portions, served mode) -----------------------------------------------------------------------
// For a block of nq consecutive tokens of one segment and the keys [j0, j0 + NK) it can see, one problem per key / value head g:
// scores [nq * rep][NK] = (scale * queries of the rep heads that share g) x keys^T, the masked softmax over each row, outputs = weights x
// values.  Scores keep fp32 accuracy on bfloat16 tensor cores: a number enters as its bfloat16 part and the remainder of that rounding,
// queries as rows [hi | lo | hi], keys as rows [hi | hi | lo] (3 D wide: hi.hi + lo.hi + hi.lo), and a weight enters the value matmul as
// [hi | lo] against the values twice side by side.  These kernels prepare the operands -- keys [G][NKp][3 D], values transposed
// [G][V][2 NKp], query rows [G][nq * rep][3 D], all bfloat16 -- and put the outputs [G][nq * rep][V] back in token order.
__device__ __forceinline__ void mk_split(float x, __nv_bfloat16 & hi, __nv_bfloat16 & lo) { hi = __float2bfloat16_rn(x); lo = __float2bfloat16_rn(x - __bfloat162float(hi)); }
__global__ void __launch_bounds__(128) kv_gather_kernel(const float * __restrict__ cache, int cache_row, const int32_t * __restrict__ map, int j0, int NK, int NKp, int G, int maps,
                                                        int D, int V, __nv_bfloat16 * __restrict__ Kb, __nv_bfloat16 * __restrict__ Vt) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int j = blockIdx.x, GK = G * maps;          // one problem per (key / value head, map): its own keys, the head's values
    const float * row = j < NK ? cache + (size_t) map[j0 + j] * cache_row : nullptr;
    for (int i = threadIdx.x; i < GK * D; i += blockDim.x) {
        __nv_bfloat16 hi, lo;
        mk_split(row ? row[i] : 0.f, hi, lo);
        __nv_bfloat16 * k = Kb + ((size_t) (i / D) * NKp + j) * 3 * D + i % D;
        k[0] = hi; k[D] = hi; k[2 * D] = lo;
    }
    for (int i = threadIdx.x; i < GK * V; i += blockDim.x) {
        const int z = i / V, c = i % V;
        const __nv_bfloat16 v = __float2bfloat16_rn(row ? row[(size_t) GK * D + (size_t) (z / maps) * V + c] : 0.f);
        Vt[(size_t) i * 2 * NKp + j] = v; Vt[(size_t) i * 2 * NKp + NKp + j] = v;
    }
}
// query row h of a token (maps rows per head, next to each other) belongs to problem z = (head / rep) * maps + h % maps, row ti * rep + head % rep
__device__ __forceinline__ size_t kv_problem_row(int h, int maps, int rep, int nq, int ti) {
    const int hq = h / maps, z = (hq / rep) * maps + h % maps;
    return (size_t) z * nq * rep + (size_t) ti * rep + hq % rep;
}
// Qc[z][ti * rep + hr] = [hi | lo | hi] of scale * q[t0 + ti][h]
__global__ void __launch_bounds__(128) kv_query_rows_kernel(const float * __restrict__ q, __nv_bfloat16 * __restrict__ Qc, int H, int maps, int rep, int nq, int D, int t0, float scale) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int ti = blockIdx.x, h = blockIdx.y;
    const float * src = q + ((size_t) (t0 + ti) * H + h) * D;
    __nv_bfloat16 * dst = Qc + kv_problem_row(h, maps, rep, nq, ti) * 3 * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        __nv_bfloat16 hi, lo;
        mk_split(src[i] * scale, hi, lo);
        dst[i] = hi; dst[D + i] = lo; dst[2 * D + i] = hi;
    }
}
// out[t0 + ti][h][V] = O[z][ti * rep + hr][V]
__global__ void __launch_bounds__(128) kv_token_order_kernel(const float * __restrict__ O, float * __restrict__ out, int H, int maps, int rep, int nq, int V, int t0) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int ti = blockIdx.x, h = blockIdx.y;
    const float * src = O + kv_problem_row(h, maps, rep, nq, ti) * V;
    float * dst = out + ((size_t) (t0 + ti) * H + h) * V;
    for (int i = threadIdx.x; i < V; i += blockDim.x) dst[i] = src[i];
}
int pib_kv_attention_mm(const float * q, const pib_hlayer & L, const pib_hbatch & b, const float * cache, int cache_row, const int32_t * map, int t0, int nq, int j0, int NK,
                        void * Kb, void * Vt, float * Qc, float * S, void * P, float * out, cudaStream_t st) {
    const int maps = L.maps, H = L.heads * maps, G = L.kv_heads, GK = G * maps, D = L.dim, V = L.vdim, rep = L.heads / G, NKp = (NK + 7) & ~7, M = nq * rep;
    if (maps > 1 && L.sink) { pib_set_error("attention: a sink with several maps per head"); return PIB_ERR_UNSUPP; }
    pib_launch(kv_gather_kernel, dim3(NKp), dim3(128), (size_t) 0, st, cache, cache_row, map, j0, NK, NKp, G, maps, D, V, (__nv_bfloat16 *) Kb, (__nv_bfloat16 *) Vt);
    CKL();
    pib_launch(kv_query_rows_kernel, dim3((unsigned) nq, (unsigned) H), dim3(128), (size_t) 0, st, q, (__nv_bfloat16 *) Qc, H, maps, rep, nq, D, t0, L.scale);
    CKL();
    pib_mm a;
    a.W = Kb; a.wtype = PIB_TYPE_BF16; a.ldw = 3 * D; a.wz = (int64_t) NKp * 3 * D; a.X = Qc; a.ldx = 3 * D; a.xz = (int64_t) M * 3 * D; a.x_bf16 = 1;
    a.Y = S; a.ldy = NKp; a.yz = (int64_t) M * NKp; a.M = M; a.N = NK; a.K = 3 * D; a.Z = GK;
    int rc = pib_dense_mm(a, st);
    if (rc != PIB_OK) return rc;
    if ((rc = pib_window_softmax(S, P, NKp, NK, j0, L.window, b.pos, t0, GK * M, M, rep, L.sink, st, L.mask)) != PIB_OK) return rc;
    pib_mm v;
    v.W = Vt; v.wtype = PIB_TYPE_BF16; v.ldw = 2 * NKp; v.wz = (int64_t) V * 2 * NKp; v.X = (const float *) P; v.ldx = 2 * NKp; v.xz = (int64_t) M * 2 * NKp; v.x_bf16 = 1;
    v.Y = Qc; v.ldy = V; v.yz = (int64_t) M * V; v.M = M; v.N = V; v.K = 2 * NKp; v.Z = GK;              // the query rows are used up: the outputs take their place
    if ((rc = pib_dense_mm(v, st)) != PIB_OK) return rc;
    pib_launch(kv_token_order_kernel, dim3((unsigned) nq, (unsigned) H), dim3(128), (size_t) 0, st, (const float *) Qc, out, H, maps, rep, nq, V, t0);
    CKL();
    return PIB_OK;
}

// ---- RWKV-style time mixing -----------------------------------------------------------------------------------------------------
// mixes[t][s] = h[t] + (h[t - 1] - h[t]) * mu[s], s = 0 .. n_mix - 1; h[t - 1] of a segment's first token is the slot's row (zeros at a
// sequence's start).  The second kernel leaves each segment's last row in the slot.
__global__ void __launch_bounds__(256) token_shift_kernel(const float * __restrict__ h, const float * __restrict__ mu, int n_mix, const int32_t * __restrict__ seg,
                                                          const int32_t * __restrict__ seg_start, const int32_t * __restrict__ seg_slot, const float * __restrict__ state,
                                                          size_t state_stride, size_t shift_off, int W, float * __restrict__ mixes) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x, sg = seg[t];
    const float * prev = t > seg_start[sg] ? h + (size_t) (t - 1) * W : state + (size_t) seg_slot[sg] * state_stride + shift_off;
    const float * cur = h + (size_t) t * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float a = cur[c], d = prev[c] - a;
        for (int s = 0; s < n_mix; s++) mixes[((size_t) t * n_mix + s) * W + c] = fmaf(d, mu[(size_t) s * W + c], a);
    }
}
__global__ void __launch_bounds__(256) token_shift_tail_kernel(const float * __restrict__ h, const int32_t * __restrict__ seg_start, const int32_t * __restrict__ seg_len,
                                                               const int32_t * __restrict__ seg_slot, float * __restrict__ state, size_t state_stride, size_t shift_off, int W) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int sg = blockIdx.x;
    const float * last = h + (size_t) (seg_start[sg] + seg_len[sg] - 1) * W;
    float * dst = state + (size_t) seg_slot[sg] * state_stride + shift_off;
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[c] = last[c];
}
int pib_token_shift(const float * h, const float * mu, int n_mix, const pib_hbatch & b, float * state, size_t state_stride, size_t shift_off, int W, float * mixes, cudaStream_t st) {
    pib_launch(token_shift_kernel, dim3(b.T), dim3(256), (size_t) 0, st, h, mu, n_mix, b.seg, b.seg_start, b.seg_slot, (const float *) state, state_stride, shift_off, W, mixes);
    CKL();
    pib_launch(token_shift_tail_kernel, dim3(b.S), dim3(256), (size_t) 0, st, h, b.seg_start, b.seg_len, b.seg_slot, state, state_stride, shift_off, W);
    CKL();
    return PIB_OK;
}

// elementwise, in place on rows [T][n] with pitch ld: op 0 tanh(z); op 1 the decay exp(-exp(z + bias[i]))
__global__ void rows_act_kernel(float * __restrict__ z, int ld, int n, int T, int op, const float * __restrict__ bias) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t) T * n) return;
    const int t = (int) (i / n), c = (int) (i % n);
    float * p = z + (size_t) t * ld + c;
    *p = op == 0 ? tanhf(*p) : expf(-expf(*p + bias[c]));
}
int pib_rows_act(float * z, int ld, int n, int T, int op, const float * bias, cudaStream_t st) {
    const int64_t tot = (int64_t) T * n;
    pib_launch(rows_act_kernel, dim3((unsigned) ((tot + 255) / 256)), dim3(256), (size_t) 0, st, z, ld, n, T, op, bias);
    CKL();
    return PIB_OK;
}

// ---- the gated delta rule: what follows the convolution ----------------------------------------------------------------------------
// cv[t] = [q (G*D) | k (G*D) | v (H*V)] after convolution and silu: q and k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q
// also times D^-1/2.  proj[t] holds the raw gate logits b (H) at b_off and a (H) at a_off: bg[t] = [sigmoid(b) (H) | exp(-exp(a_log) softplus(a + dt_bias)) (H)]
__global__ void __launch_bounds__(128) delta_prep_kernel(float * __restrict__ cv, int ldc, int G, int D, int H, const float * __restrict__ proj, int ldp, int b_off, int a_off,
                                                         const float * __restrict__ a_log, const float * __restrict__ dt_bias, float * __restrict__ bg) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float * r = cv + (size_t) t * ldc;
    const float qs = 1.0f / sqrtf((float) D);
    for (int hh = warp; hh < 2 * G; hh += nw) {
        float * x = r + (size_t) hh * D;
        float s = 0.f;
        for (int i = lane; i < D; i += 32) s = fmaf(x[i], x[i], s);
        const float inv = (hh < G ? qs : 1.0f) / sqrtf(warp_sum(s) + 1e-6f);
        for (int i = lane; i < D; i += 32) x[i] *= inv;
    }
    const float * p = proj + (size_t) t * ldp;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        bg[(size_t) t * 2 * H + i] = mk_sigmoid(p[b_off + i]);
        const float z = p[a_off + i] + dt_bias[i];
        const float sp = z > 20.f ? z : log1pf(expf(z));
        bg[(size_t) t * 2 * H + H + i] = expf(-expf(a_log[i]) * sp);
    }
}
int pib_delta_prep(float * cv, int ldc, const pib_hlayer & L, const float * proj, int ldp, int b_off, int a_off, float * bg, int T, cudaStream_t st) {
    pib_launch(delta_prep_kernel, dim3(T), dim3(128), (size_t) 0, st, cv, ldc, L.kv_heads, L.dim, L.heads, proj, ldp, b_off, a_off, (const float *) L.a_log, (const float *) L.dt_bias, bg);
    CKL();
    return PIB_OK;
}

// ---- the recurrences -----------------------------------------------------------------------------------------------------------------
// grid (segment, head, tile of LS_VT value columns), 16 * LS_VT threads: the 16 lanes of a half-warp share one column of the head's
// [D][V] matrix, lane `part` keeping rows part, part + 16, ... in registers (columns are independent).  A token's inputs come through
// shared memory in chunks of tokens, the next chunk in flight (cp.async) while this one is walked; the matrix is read from the slot at
// the segment's start and left there at its end.
//   MODE 0 (time mixing):  o = sum_d a_d (s_d + u_d k_d v),  s_d <- w_d s_d + k_d v                         row = [a D | k D | w D | v LS_VT | dot]
//   MODE 1 (delta rule):   s_d <- g s_d,  e = beta (v - sum_d s_d k_d),  o = sum_d s_d a_d + e sum_d k_d a_d,  s_d <- s_d + k_d e
//                                                                                                           row = [a D | k D | v LS_VT | g, beta | dot]
//   MODE 2 (constant decay): s_d <- c s_d + k_d v,  o = sum_d a_d s_d  (read after the write; c one number per head)   row = [a D | k D | v LS_VT | dot]
//   MODE 3 (one decay per head and token, Mamba-2): s_d <- c s_d + (dt k_d) v,  o = sum_d a_d s_d + u v  (read after the write; u one number per head)
//                                                                                                           row = [a D | k D | v LS_VT | c, dt | dot]
// What does not depend on the matrix or the column -- dot = sum_d a_d u_d k_d (MODE 0), sum_d a_d k_d (MODE 1) -- is formed once per token
// when its chunk has landed; in MODE 1 the read-out is taken from the sums over the matrix before the write (one round of shuffles for
// both sums), and the next token's rows are already in registers while the sums of this one cross the lanes.
// FULL: D == 16 RPT, no row guards.
#define LS_VT    8
struct ls_args {
    const float * a; int lda, a_hs;          // query-like rows: a[t * lda + group * a_hs + d]
    const float * k; int ldk, k_hs;
    const float * w; int ldw;                // MODE 0: decay rows w[t * ldw + h * D + d];   MODE 1: bg rows [beta (H) | g (H)], ldw = 2 H;   MODE 2: decay [H];   MODE 3: rows [dt (H) | c (H)]
    const float * v; int ldv;                // v[t * ldv + h * V + j]
    const float * u;                         // MODE 0: bonus [H][D];   MODE 3: skip [H]
    int H, G, D, V, chunk;
    const int32_t * seg_start, * seg_len, * seg_slot;
    float * state; size_t state_stride, state_off;
    float * out;                             // [T][H][V]
    int vec16;                               // set by lin_scan: the operand rows start on 16-byte boundaries and D is a multiple of 4 (staged in 16-byte pieces)
};
__device__ __forceinline__ float ls_sum16(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    x += __shfl_xor_sync(0xffffffffu, x, 4);
    x += __shfl_xor_sync(0xffffffffu, x, 8);
    return x;
}
template <int RPT, int MODE, bool FULL>
__global__ void __launch_bounds__(16 * LS_VT) lin_scan_kernel(ls_args A) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float hs[];
    const int sg = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * LS_VT, part = threadIdx.x & 15, vl = threadIdx.x >> 4, vd = v0 + vl;
    const int D = FULL ? 16 * RPT : A.D, V = A.V, H = A.H, grp = h / (H / A.G), CH = A.chunk;
    const int s0 = A.seg_start[sg], n = A.seg_len[sg];
    const int vbase = MODE == 0 ? 3 * D : 2 * D, dot_off = vbase + LS_VT + ((MODE == 1 || MODE == 3) ? 2 : 0), row_f = (dot_off + 4) & ~3;
    const float cdec = MODE == 2 ? A.w[h] : 0.f, skip = MODE == 3 ? A.u[h] : 0.f;
    const bool vok = vd < V;
    float * S = A.state + (size_t) A.seg_slot[sg] * A.state_stride + A.state_off + (size_t) h * D * V;
    float s[RPT], ub[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int d = part + 16 * r;
        s[r] = ((FULL || d < D) && vok) ? S[(size_t) d * V + vd] : 0.f;
        ub[r] = (MODE == 0 && (FULL || d < D)) ? A.u[(size_t) h * D + d] : 0.f;
    }
    auto fetch = [&](int c0, int buf) {
        const int nc = min(CH, n - c0);
        if (A.vec16) {
            // the chunk's operand rows as one list of 16-byte pieces (token, operand, piece) spread over the threads, then the tokens' few
            // scalars the same way: a thread forms an address per copy, not per token
            const uint32_t base = (uint32_t) __cvta_generic_to_shared(hs + (size_t) buf * CH * row_f);
            const int nv = D >> 2, NP = (MODE == 0 ? 3 : 2) * nv;
            for (int p = threadIdx.x; p < nc * NP; p += blockDim.x) {
                const int t = p / NP, e = p - t * NP, which = e / nv, i = e - which * nv;
                const size_t tt = (size_t) (s0 + c0 + t);
                const float * src = which == 0 ? A.a + tt * A.lda + (size_t) grp * A.a_hs : which == 1 ? A.k + tt * A.ldk + (size_t) grp * A.k_hs : A.w + tt * A.ldw + (size_t) h * D;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + 4u * (uint32_t) (t * row_f + which * D + 4 * i)), "l"(src + 4 * i) : "memory");
            }
            constexpr int NS = LS_VT + ((MODE == 1 || MODE == 3) ? 2 : 0);
            for (int p = threadIdx.x; p < nc * NS; p += blockDim.x) {
                const int t = p / NS, j = p - t * NS;
                const size_t tt = (size_t) (s0 + c0 + t);
                const uint32_t dst = base + 4u * (uint32_t) (t * row_f + vbase + j);
                if (j < LS_VT) {
                    if (v0 + j < V) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(A.v + tt * A.ldv + (size_t) h * V + v0 + j) : "memory");
                } else {
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(A.w + tt * A.ldw + (j == LS_VT ? H : 0) + h) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
        for (int t = 0; t < nc; t++) {
            const size_t tt = (size_t) (s0 + c0 + t);
            const float * ar = A.a + tt * A.lda + (size_t) grp * A.a_hs;
            const float * kr = A.k + tt * A.ldk + (size_t) grp * A.k_hs;
            const uint32_t dst = (uint32_t) __cvta_generic_to_shared(hs + (size_t) (buf * CH + t) * row_f);
            for (int e = threadIdx.x; e < D; e += blockDim.x) {
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * e), "l"(ar + e) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * (D + e)), "l"(kr + e) : "memory");
                if (MODE == 0) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * (2 * D + e)), "l"(A.w + tt * A.ldw + (size_t) h * D + e) : "memory");
            }
            if (threadIdx.x < LS_VT && v0 + (int) threadIdx.x < V)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * (vbase + threadIdx.x)), "l"(A.v + tt * A.ldv + (size_t) h * V + v0 + threadIdx.x) : "memory");
            if ((MODE == 1 || MODE == 3) && threadIdx.x >= 32 && threadIdx.x < 34) {       // g, then beta (MODE 3: the decay, then dt)
                const int which = threadIdx.x - 32;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * (vbase + LS_VT + which)), "l"(A.w + tt * A.ldw + (which == 0 ? H : 0) + h) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n > 0) fetch(0, 0);
    int buf = 0;
    float * op = A.out + (size_t) s0 * H * V + (size_t) h * V + vd;
    const int ostride = H * V;
    for (int c0 = 0; c0 < n; c0 += CH, buf ^= 1) {
        const int nc = min(CH, n - c0);
        if (c0 + CH < n) { fetch(c0 + CH, buf ^ 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else             asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        float * rows = hs + (size_t) buf * CH * row_f;
        for (int t0 = 0; t0 < nc; t0 += LS_VT) {             // the part of a token's step that needs neither the matrix nor the column
            const int  t = t0 + vl;                          // (both halves of a warp take every trip: the shuffles below name all 32 lanes)
            const bool live = t < nc;
            const float * rp = rows + (size_t) (live ? t : 0) * row_f + part;
            float p = 0.f;
#pragma unroll
            for (int r = 0; r < RPT; r++) if (FULL || part + 16 * r < D) p = fmaf(MODE == 0 ? rp[16 * r] * ub[r] : rp[16 * r], rp[D + 16 * r], p);
            p = ls_sum16(p);
            if (live && part == 0) rows[(size_t) t * row_f + dot_off] = p;
        }
        __syncthreads();
        const float * qp = rows + part;
        float aa[RPT], kk[RPT], ww[RPT];
#pragma unroll
        for (int r = 0; r < RPT; r++) {
            const bool ok = FULL || part + 16 * r < D;
            aa[r] = ok ? qp[16 * r] : 0.f; kk[r] = ok ? qp[D + 16 * r] : 0.f; ww[r] = (MODE == 0 && ok) ? qp[2 * D + 16 * r] : 0.f;
        }
#pragma unroll 2
        for (int t = 0; t < nc; t++, op += ostride) {
            const float * sc = qp - part + vbase;            // this token's scalars
            const float * qn = t + 1 < nc ? qp + row_f : qp; // the next token's rows (the last token reads its own again)
            const float v = vok ? sc[vl] : 0.f, dot = sc[dot_off - vbase];
            float an[RPT], kn[RPT], wn[RPT];
            if (MODE == 0) {
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < RPT; r++) { acc = fmaf(aa[r], s[r], acc); s[r] = fmaf(ww[r], s[r], kk[r] * v); }
#pragma unroll
                for (int r = 0; r < RPT; r++) {
                    const bool ok = FULL || part + 16 * r < D;
                    an[r] = ok ? qn[16 * r] : 0.f; kn[r] = ok ? qn[D + 16 * r] : 0.f; wn[r] = ok ? qn[2 * D + 16 * r] : 0.f;
                }
                acc = ls_sum16(acc);
                if (part == 0 && vok) *op = fmaf(v, dot, acc);
            } else if (MODE == 2) {
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < RPT; r++) { acc = fmaf(aa[r], s[r], acc); s[r] = fmaf(cdec, s[r], kk[r] * v); }
#pragma unroll
                for (int r = 0; r < RPT; r++) {
                    const bool ok = FULL || part + 16 * r < D;
                    an[r] = ok ? qn[16 * r] : 0.f; kn[r] = ok ? qn[D + 16 * r] : 0.f; wn[r] = 0.f;
                }
                acc = ls_sum16(acc);
                if (part == 0 && vok) *op = fmaf(cdec, acc, v * dot);       // sum_d a_d (c s_d + k_d v)
            } else if (MODE == 3) {
                const float dec = sc[LS_VT], kv = sc[LS_VT + 1] * v;
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < RPT; r++) { acc = fmaf(aa[r], s[r], acc); s[r] = fmaf(dec, s[r], kk[r] * kv); }
#pragma unroll
                for (int r = 0; r < RPT; r++) {
                    const bool ok = FULL || part + 16 * r < D;
                    an[r] = ok ? qn[16 * r] : 0.f; kn[r] = ok ? qn[D + 16 * r] : 0.f; wn[r] = 0.f;
                }
                acc = ls_sum16(acc);
                if (part == 0 && vok) *op = fmaf(dec, acc, fmaf(kv, dot, skip * v));      // sum_d a_d (c s_d + dt k_d v) + u v
            } else {
                const float g = sc[LS_VT], beta = sc[LS_VT + 1];
                float sk = 0.f, sa = 0.f;
#pragma unroll
                for (int r = 0; r < RPT; r++) { s[r] *= g; sk = fmaf(s[r], kk[r], sk); sa = fmaf(s[r], aa[r], sa); }
#pragma unroll
                for (int r = 0; r < RPT; r++) {
                    const bool ok = FULL || part + 16 * r < D;
                    an[r] = ok ? qn[16 * r] : 0.f; kn[r] = ok ? qn[D + 16 * r] : 0.f; wn[r] = 0.f;
                }
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) { sk += __shfl_xor_sync(0xffffffffu, sk, o); sa += __shfl_xor_sync(0xffffffffu, sa, o); }
                const float e = beta * (v - sk);
#pragma unroll
                for (int r = 0; r < RPT; r++) s[r] = fmaf(kk[r], e, s[r]);
                if (part == 0 && vok) *op = fmaf(e, dot, sa);
            }
#pragma unroll
            for (int r = 0; r < RPT; r++) { aa[r] = an[r]; kk[r] = kn[r]; ww[r] = wn[r]; }
            qp = qn;
        }
        __syncthreads();                           // everyone is done with this buffer before the fetch after next refills it
    }
#pragma unroll
    for (int r = 0; r < RPT; r++) { const int d = part + 16 * r; if ((FULL || d < D) && vok) S[(size_t) d * V + vd] = s[r]; }
}

static int lin_scan(int mode, ls_args & A, int S, cudaStream_t st) {
    if (A.D > 256) { pib_set_error("recurrence: dim %d not supported (up to 256)", A.D); return PIB_ERR_UNSUPP; }
    dim3 grid((unsigned) S, (unsigned) A.H, (unsigned) ((A.V + LS_VT - 1) / LS_VT));
    const size_t row_f = ((size_t) (mode == 0 ? 3 * A.D : 2 * A.D) + LS_VT + ((mode == 1 || mode == 3) ? 2 : 0) + 4) & ~(size_t) 3;
    {   // 16-byte staging copies need every operand row to start on a 16-byte boundary
        static const int on = getenv("PIB_SCAN_VEC") ? atoi(getenv("PIB_SCAN_VEC")) : 1;
        auto al = [](const void * p) { return ((uintptr_t) p & 15) == 0; };
        A.vec16 = on && A.D % 4 == 0 && al(A.a) && al(A.k) && A.lda % 4 == 0 && A.ldk % 4 == 0 && A.a_hs % 4 == 0 && A.k_hs % 4 == 0 &&
                  (mode != 0 || (al(A.w) && A.ldw % 4 == 0));
    }
    // chunks of 32 tokens halve the barriers per token, but their double buffer must not push part of the grid into a second wave
    const size_t smem32 = row_f * 4 * 2 * 32;
    const size_t per_sm = smem32 <= 100 * 1024 ? (size_t) (227 * 1024) / (smem32 + 1024) : 0;
    A.chunk = per_sm > 0 && (size_t) grid.x * grid.y * grid.z <= per_sm * (size_t) pib_num_sms() ? 32 : 16;
    const size_t smem = (size_t) 2 * A.chunk * row_f * 4;
#define LS_GO(RPT, MODE, FULL) do { if (smem > 48 * 1024) cudaFuncSetAttribute(lin_scan_kernel<RPT, MODE, FULL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem); \
                                    pib_launch(lin_scan_kernel<RPT, MODE, FULL>, dim3(grid), dim3(16 * LS_VT), (size_t) smem, st, A); } while (0)
#define LS_PICK(MODE) do { if (A.D == 64) LS_GO(4, MODE, true); else if (A.D == 128) LS_GO(8, MODE, true); else if (A.D <= 32) LS_GO(2, MODE, false); \
                           else if (A.D <= 64) LS_GO(4, MODE, false); else if (A.D <= 128) LS_GO(8, MODE, false); else LS_GO(16, MODE, false); } while (0)
    if (mode == 0) LS_PICK(0); else if (mode == 1) LS_PICK(1); else if (mode == 2) LS_PICK(2); else LS_PICK(3);
#undef LS_PICK
#undef LS_GO
    CKL();
    return PIB_OK;
}

// rkvg[t] = [r | k | v | g] (H*D each), wdec[t] = decays (H*D)
int pib_wkv_scan(const float * rkvg, int ld, const float * wdec, int ldw, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, float * out, cudaStream_t st) {
    const int HD = L.heads * L.dim;
    ls_args A;
    A.a = rkvg; A.lda = ld; A.a_hs = L.dim; A.k = rkvg + HD; A.ldk = ld; A.k_hs = L.dim; A.w = wdec; A.ldw = ldw; A.v = rkvg + 2 * HD; A.ldv = ld; A.u = L.bonus;
    A.H = L.heads; A.G = L.heads; A.D = L.dim; A.V = L.dim; A.seg_start = b.seg_start; A.seg_len = b.seg_len; A.seg_slot = b.seg_slot;
    A.state = state; A.state_stride = state_stride; A.state_off = L.state_off; A.out = out;
    return lin_scan(0, A, b.S, st);
}
// cv[t] = [q (G*D) | k (G*D) | v (H*V)] prepared by pib_delta_prep, bg[t] = [beta (H) | g (H)]
int pib_delta_scan(const float * cv, int ldc, const float * bg, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, float * out, cudaStream_t st) {
    const int GD = L.kv_heads * L.dim;
    ls_args A;
    A.a = cv; A.lda = ldc; A.a_hs = L.dim; A.k = cv + GD; A.ldk = ldc; A.k_hs = L.dim; A.w = bg; A.ldw = 2 * L.heads; A.v = cv + 2 * GD; A.ldv = ldc; A.u = nullptr;
    A.H = L.heads; A.G = L.kv_heads; A.D = L.dim; A.V = L.vdim; A.seg_start = b.seg_start; A.seg_len = b.seg_len; A.seg_slot = b.seg_slot;
    A.state = state; A.state_stride = state_stride; A.state_off = L.state_off; A.out = out;
    return lin_scan(1, A, b.S, st);
}

// ---- a long segment of the constant-decay recurrence in parts --------------------------------------------------------------------------
// With a constant decay the tokens of a segment need not be walked in one chain.  The segment is cut into P parts; part 0 starts from the
// slot's matrix, every other part from zeros, and all parts are walked at once by lin_scan_kernel (P times the blocks: the recurrence is
// bound by dependent issue at low occupancy, not by work).  With L_p the matrix part p ends with and n_p its length, the matrix in front of
// part p is F_(p-1), F_0 = L_0, F_p = c^(n_p) F_(p-1) + L_p, and what token tau of part p >= 1 still lacks is c^(tau+1) F_(p-1)^T q: one small
// fp32 product per part and head.  The slot's matrix becomes F_(P-1).
//   buf (floats): L [P][E] | F [P][E], E = H * D * V; then the parts' table (int32): start [P] | length [P] | index [P]
__global__ void decay_split_prepare_kernel(const int32_t * __restrict__ seg_start, const int32_t * __restrict__ seg_slot, const float * __restrict__ state, size_t state_stride,
                                           size_t state_off, int E, int P, int T, int per, float * __restrict__ Lm, int32_t * __restrict__ table) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < P) { table[i] = seg_start[0] + (int) i * per; table[P + i] = min(per, T - (int) i * per); table[2 * P + i] = (int) i; }
    if (i >= (int64_t) P * E) return;
    Lm[i] = i < E ? state[(size_t) seg_slot[0] * state_stride + state_off + i] : 0.f;
}
// cum (optional, pitch ldc): decays that differ from token to token -- cum[t][h] is the product of head h's decays from the start of t's
// part up to and with t, so a part's last row is the decay over the whole part
__global__ void decay_split_combine_kernel(const float * __restrict__ Lm, float * __restrict__ F, int E, int DV, int P, const int32_t * __restrict__ table,
                                           const float * __restrict__ decay, const float * __restrict__ cum, int ldc, const int32_t * __restrict__ seg_slot,
                                           float * __restrict__ state, size_t state_stride, size_t state_off) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const float l2 = cum ? 0.f : log2f(decay[e / DV]);
    float f = Lm[e];
    F[e] = f;
    for (int p = 1; p < P; p++) {
        const float c = cum ? cum[(size_t) (table[p] + table[P + p] - 1) * ldc + e / DV] : exp2f((float) table[P + p] * l2);
        f = fmaf(c, f, Lm[(size_t) p * E + e]);
        F[(size_t) p * E + e] = f;
    }
    state[(size_t) seg_slot[0] * state_stride + state_off + e] = f;
}
// grid (tiles of DF_TT tokens, heads x tiles of DF_VT columns, parts 1 .. P-1): out[t][h][v] += c^(tau+1) sum_d q[t][h][d] F_(p-1)[h][d][v]
// (with cum: cum[t][h] in place of c^(tau+1)); the H heads read the query rows of G groups
#define DF_TT 64
#define DF_VT 64
__global__ void __launch_bounds__(256) decay_split_fixup_kernel(const float * __restrict__ q, int ldq, const float * __restrict__ F, int E, int H, int G, int D, int V,
                                                                const int32_t * __restrict__ table, int P, const float * __restrict__ decay, const float * __restrict__ cum,
                                                                int ldc, float * __restrict__ out) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ __align__(16) float fs[];   // F tile [Dp][DF_VT], then query rows [DF_TT][Dp]; Dp = D rounded up to 4, the pad zeros
    const int nvt = (V + DF_VT - 1) / DF_VT, p = blockIdx.z + 1, h = blockIdx.y / nvt, v0 = (blockIdx.y % nvt) * DF_VT, t0 = blockIdx.x * DF_TT;
    const int start = table[p], len = table[P + p], Dp = (D + 3) & ~3;
    if (t0 >= len) return;
    float * qs = fs + (size_t) Dp * DF_VT;
    const float * Fp = F + (size_t) (p - 1) * E + (size_t) h * D * V;
    for (int i = threadIdx.x; i < Dp * DF_VT; i += blockDim.x) { const int d = i / DF_VT, j = i % DF_VT; fs[i] = (d < D && v0 + j < V) ? Fp[(size_t) d * V + v0 + j] : 0.f; }
    for (int i = threadIdx.x; i < DF_TT * Dp; i += blockDim.x) {
        const int t = i / Dp, d = i % Dp;
        qs[i] = (t0 + t < len && d < D) ? q[(size_t) (start + t0 + t) * ldq + (size_t) (h / (H / G)) * D + d] : 0.f;
    }
    __syncthreads();
    // a thread owns 8 tokens x 2 columns; the 8 tokens of a warp are the same for all its lanes (their query values are broadcast, four
    // states per load), the columns are vj and vj + 32
    const int vj = threadIdx.x & 31, tg = threadIdx.x >> 5;
    float acc0[8], acc1[8];
#pragma unroll
    for (int i = 0; i < 8; i++) { acc0[i] = 0.f; acc1[i] = 0.f; }
    const float * qr = qs + (size_t) tg * 8 * Dp;
    for (int d = 0; d < Dp; d += 4) {
        float f0[4], f1[4];
#pragma unroll
        for (int k = 0; k < 4; k++) { f0[k] = fs[(d + k) * DF_VT + vj]; f1[k] = fs[(d + k) * DF_VT + vj + 32]; }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float4 qv = *reinterpret_cast<const float4 *>(qr + (size_t) i * Dp + d);
            acc0[i] = fmaf(qv.x, f0[0], acc0[i]); acc0[i] = fmaf(qv.y, f0[1], acc0[i]); acc0[i] = fmaf(qv.z, f0[2], acc0[i]); acc0[i] = fmaf(qv.w, f0[3], acc0[i]);
            acc1[i] = fmaf(qv.x, f1[0], acc1[i]); acc1[i] = fmaf(qv.y, f1[1], acc1[i]); acc1[i] = fmaf(qv.z, f1[2], acc1[i]); acc1[i] = fmaf(qv.w, f1[3], acc1[i]);
        }
    }
    const float l2 = cum ? 0.f : log2f(decay[h]);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int t = t0 + tg * 8 + i;
        if (t >= len) continue;
        const float c = cum ? cum[(size_t) (start + t) * ldc + h] : exp2f((float) (t + 1) * l2);
        float * o = out + (size_t) (start + t) * H * V + (size_t) h * V + v0;
        if (v0 + vj < V)      o[vj] = fmaf(c, acc0[i], o[vj]);
        if (v0 + vj + 32 < V) o[vj + 32] = fmaf(c, acc1[i], o[vj + 32]);
    }
}
size_t pib_scan_split_bytes(int H, int D, int V, int parts) { return ((size_t) 2 * parts * H * D * V + 3 * (size_t) parts) * 4 + 64; }
size_t pib_decay_split_bytes(const pib_hlayer & L, int parts) { return pib_scan_split_bytes(L.heads2, L.dim2, L.vdim2, parts); }

// the parts of a segment walked at once: matrices in front of the parts, then what each token still lacks (see above).  A: the walk's
// arguments over the whole batch (one segment); mode: the recurrence; q: the read-out rows of G groups; cum / decay: see the kernels
static int scan_in_parts(int mode, ls_args A, const float * q, int ldq, const float * decay, const float * cum, int ldc, const pib_hbatch & b, float * state, size_t state_stride,
                         size_t state_off, float * split_buf, int parts, int per, cudaStream_t st) {
    if (b.S != 1) { pib_set_error("recurrence in parts: the batch must be one segment"); return PIB_ERR_ARG; }
    const int H = A.H, D = A.D, V = A.V, E = H * D * V;
    float * Lm = split_buf, * F = split_buf + (size_t) parts * E;
    int32_t * table = reinterpret_cast<int32_t *>(split_buf + (size_t) 2 * parts * E);
    const int64_t n = (int64_t) parts * E;
    pib_launch(decay_split_prepare_kernel, dim3((unsigned) ((n + 255) / 256)), dim3(256), (size_t) 0, st, b.seg_start, b.seg_slot, (const float *) state, state_stride, state_off, E,
               parts, b.T, per, Lm, table);
    CKL();
    A.seg_start = table; A.seg_len = table + parts; A.seg_slot = table + 2 * parts; A.state = Lm; A.state_stride = (size_t) E; A.state_off = 0;
    int rc = lin_scan(mode, A, parts, st);
    if (rc != PIB_OK) return rc;
    pib_launch(decay_split_combine_kernel, dim3((unsigned) ((E + 255) / 256)), dim3(256), (size_t) 0, st, (const float *) Lm, F, E, D * V, parts, (const int32_t *) table,
               decay, cum, ldc, b.seg_slot, state, state_stride, state_off);
    CKL();
    const size_t smem = (size_t) ((D + 3) & ~3) * (DF_VT + DF_TT) * 4;
    if (smem > 200 * 1024) { pib_set_error("recurrence in parts: dim %d", D); return PIB_ERR_UNSUPP; }
    if (smem > 48 * 1024) cudaFuncSetAttribute(decay_split_fixup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
    dim3 grid((unsigned) ((per + DF_TT - 1) / DF_TT), (unsigned) (H * ((V + DF_VT - 1) / DF_VT)), (unsigned) (parts - 1));
    pib_launch(decay_split_fixup_kernel, dim3(grid), dim3(256), (size_t) smem, st, q, ldq, (const float *) F, E, H, A.G, D, V, (const int32_t *) table, parts, decay, cum, ldc, A.out);
    CKL();
    return PIB_OK;
}

// linear attention with one constant decay per head: rows proj[t] hold q (H*D) at q_off, k (H*D) at k_off, v (H*V) at v_off, activations applied.
// parts >= 2 (only for a batch that is ONE segment): the segment is walked as `parts` parts of `per` tokens at once; split_buf holds
// pib_decay_split_bytes(L, parts) bytes
int pib_decay_scan(const float * proj, int ldp, int q_off, int k_off, int v_off, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, float * out,
                   cudaStream_t st, float * split_buf, int parts, int per) {
    ls_args A;
    A.a = proj + q_off; A.lda = ldp; A.a_hs = L.dim2; A.k = proj + k_off; A.ldk = ldp; A.k_hs = L.dim2; A.w = L.decay; A.ldw = 0; A.v = proj + v_off; A.ldv = ldp; A.u = nullptr;
    A.H = L.heads2; A.G = L.heads2; A.D = L.dim2; A.V = L.vdim2; A.seg_start = b.seg_start; A.seg_len = b.seg_len; A.seg_slot = b.seg_slot;
    A.state = state; A.state_stride = state_stride; A.state_off = L.state_off; A.out = out;
    if (parts < 2 || !split_buf) return lin_scan(2, A, b.S, st);
    return scan_in_parts(2, A, proj + q_off, ldp, L.decay, nullptr, 0, b, state, state_stride, L.state_off, split_buf, parts, per, st);
}

// cum[t][h] <- exp(sum of the logarithms of head h's decays from the start of t's part up to and with t); on entry the column holds the
// logarithms.  One thread per (part, head).
__global__ void cum_decay_kernel(float * __restrict__ cum, int ldc, int H, int T, int per, int P) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P * H) return;
    const int p = i / H, h = i % H, t1 = min(T, (p + 1) * per);
    float s = 0.f;
    for (int t = p * per; t < t1; t += 8) {                    // eight rows' loads in flight at once: the chain is the additions only
        float l[8];
#pragma unroll
        for (int i = 0; i < 8; i++) l[i] = t + i < t1 ? cum[(size_t) (t + i) * ldc + h] : 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) { s += l[i]; if (t + i < t1) cum[(size_t) (t + i) * ldc + h] = expf(s); }
    }
}

// Mamba-2: xbc[t] = [x (H*V) | B (G*N) | C (G*N)] after convolution and silu, dg[t] = [dt (H) | decay (H) | log decay (H)]; the matrices are
// [H][N][V].  parts >= 2 (only for a batch that is ONE segment): the segment is walked as `parts` parts of `per` tokens at once, as for a
// constant decay, with the running products of the decays inside a part (they take the third column's place) where that has powers of c
int pib_mamba2_scan(const float * xbc, int ldc, float * dg, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, float * out, cudaStream_t st,
                    float * split_buf, int parts, int per) {
    const int I = L.heads * L.vdim, GN = L.kv_heads * L.n_state, H = L.heads;
    ls_args A;
    A.a = xbc + I + GN; A.lda = ldc; A.a_hs = L.n_state; A.k = xbc + I; A.ldk = ldc; A.k_hs = L.n_state; A.w = dg; A.ldw = 3 * H; A.v = xbc; A.ldv = ldc; A.u = L.ssm_d;
    A.H = H; A.G = L.kv_heads; A.D = L.n_state; A.V = L.vdim; A.seg_start = b.seg_start; A.seg_len = b.seg_len; A.seg_slot = b.seg_slot;
    A.state = state; A.state_stride = state_stride; A.state_off = L.state_off; A.out = out;
    if (parts < 2 || !split_buf) return lin_scan(3, A, b.S, st);
    pib_launch(cum_decay_kernel, dim3((unsigned) ((parts * H + 127) / 128)), dim3(128), (size_t) 0, st, dg + 2 * H, 3 * H, H, b.T, per, parts);
    CKL();
    return scan_in_parts(3, A, xbc + I + GN, ldc, nullptr, dg + 2 * H, 3 * H, b, state, state_stride, L.state_off, split_buf, parts, per, st);
}

// one warp per (token, head): o <- o / sqrt(mean(o^2) + eps) * w[(h * w_hs) + i] * silu(gate[t * ldg + h * V + i])
__global__ void gated_head_norm_kernel(float * __restrict__ o, int n_rows, int H, int V, const float * __restrict__ w, int w_hs, const float * __restrict__ gate, int ldg, float eps) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const int t = row / H, h = row % H;
    float * r = o + (size_t) row * V;
    const float * g = gate + (size_t) t * ldg + (size_t) h * V;
    const float * wr = w + (size_t) h * w_hs;
    float s = 0.f;
    for (int i = lane; i < V; i += 32) s = fmaf(r[i], r[i], s);
    const float inv = 1.0f / sqrtf(warp_sum(s) / V + eps);
    for (int i = lane; i < V; i += 32) r[i] = r[i] * inv * wr[i] * mk_silu(g[i]);
}
int pib_gated_head_norm(float * o, int T, int H, int V, const float * w, int w_hs, const float * gate, int ldg, float eps, cudaStream_t st) {
    const int n_rows = T * H;
    pib_launch(gated_head_norm_kernel, dim3((n_rows + 7) / 8), dim3(256), (size_t) 0, st, o, n_rows, H, V, w, w_hs, gate, ldg, eps);
    CKL();
    return PIB_OK;
}

// ---- clamped gated experts ---------------------------------------------------------------------------------------------------------
// rows [n_rows][ld] = [gate (F) | up (F)] of an expert's input h; with a weight per row the expert sees w h, and since both products are
// linear in h the weight multiplies them here.  a = min(w gate, limit), b = clamp(w up, -limit, limit); the row's first F entries become
// a sigmoid(1.702 a) (b + 1).  scale_of: row -> index into scale (null: the row itself).
__global__ void glu_clamp_kernel(float * __restrict__ gu, int ld, int F, float limit, const float * __restrict__ scale, const int32_t * __restrict__ scale_of, int n_rows) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t) n_rows * F) return;
    const int row = (int) (i / F), c = (int) (i % F);
    float * r = gu + (size_t) row * ld;
    const float w = scale ? scale[scale_of ? scale_of[row] : row] : 1.0f;
    const float a = fminf(w * r[c], limit), b = fminf(fmaxf(w * r[F + c], -limit), limit);
    r[c] = a * mk_sigmoid(1.702f * a) * (b + 1.0f);
}
int pib_glu_clamp(float * gu, int ld, int F, float limit, const float * scale, const int32_t * scale_of, int n_rows, cudaStream_t st) {
    const int64_t tot = (int64_t) n_rows * F;
    if (tot <= 0) return PIB_OK;
    pib_launch(glu_clamp_kernel, dim3((unsigned) ((tot + 255) / 256)), dim3(256), (size_t) 0, st, gu, ld, F, limit, scale, scale_of, n_rows);
    CKL();
    return PIB_OK;
}

// ---- the parallel layer's sum ---------------------------------------------------------------------------------------------------------
// x[t] += mixer[t] + shared[t] * sigmoid(sgl[t * ldsg]) + sum_k edn[inv[t * top + k]]   (each part optional; k ascending)
__global__ void parallel_sum_kernel(float * __restrict__ x, const float * __restrict__ mixer, const float * __restrict__ shared, const float * __restrict__ sgl, int ldsg,
                                    const float * __restrict__ edn, const int32_t * __restrict__ inv, int top, int W) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x;
    const float sg = shared ? (sgl ? mk_sigmoid(sgl[(size_t) t * ldsg]) : 1.0f) : 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = mixer ? mixer[(size_t) t * W + c] : 0.f;
        if (shared) acc = fmaf(shared[(size_t) t * W + c], sg, acc);
        if (edn) for (int k = 0; k < top; k++) acc += edn[(size_t) inv[(size_t) t * top + k] * W + c];
        x[(size_t) t * W + c] += acc;
    }
}
int pib_parallel_sum(float * x, const float * mixer, const float * shared, const float * sgl, int ldsg, const float * edn, const int32_t * inv, int top, int T, int W, cudaStream_t st) {
    pib_launch(parallel_sum_kernel, dim3(T), dim3(256), (size_t) 0, st, x, mixer, shared, sgl, ldsg, edn, inv, top, W);
    CKL();
    return PIB_OK;
}
