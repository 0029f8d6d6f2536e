// hybrid_kernels.cu -- the per-token and per-sequence kernels of layer-list models (hybrid.cuh).  Everything here computes in fp32:
// norms, rotations, attention scores and weights, gates and the recurrence, the router.
//
//   LayerNorm (weight, no bias) on a sublayer's output, added to the residual stream
//   causal convolution over time on any run of channels (in front of a mixer, or on projected q | k | v), its last taps-1 inputs kept per sequence
//   latent attention: per token one cached row [c | k_rot]; queries are folded through W_uk ("absorbed"), so a score is
//       (q_lat . c + q_rot . k_rot) * scale, softmax over a sliding window plus one learned sink logit per head, and the
//       output is sum_j p_j c_j (folded through W_uv by the caller)
//   HGRN2: S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T, o_t = S_t^T q_t, per head, state in fp32 per sequence
//   PolyNorm, mixture-of-experts routing (softmax, top-k, renormalise), grouping of (token, expert) pairs by expert
#include "hybrid.cuh"

#include <algorithm>

#include <cuda_bf16.h>

#define CKL() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) { pib_set_error("%s:%d: launch failed: %s", __FILE__, __LINE__, cudaGetErrorString(e__)); return PIB_ERR_CUDA; } } while (0)

// sum over the block (any block size that is a multiple of 32, up to 1024); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float * red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}

// ---- LayerNorm ---------------------------------------------------------------------------------------------------------------
// out[t] (+)= (in[t] - mean) / sqrt(mean((in[t] - mean)^2) + eps) * w     one block per token, the row staged in shared memory
__device__ __forceinline__ void ln_row(const float * row, const float * __restrict__ w, float eps, int W, float * __restrict__ out, bool accumulate, float * red) {
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) s += row[i];
    const float mean = block_sum(s, red) / W;
    float q = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) { const float d = row[i] - mean; q += d * d; }
    const float inv = 1.0f / sqrtf(block_sum(q, red) / W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = (row[i] - mean) * inv * w[i];
        out[i] = accumulate ? out[i] + v : v;
    }
}

__global__ void __launch_bounds__(256) layer_norm_kernel(const float * __restrict__ in, const float * __restrict__ w, float eps, int W, float * out, int accumulate) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float srow[];
    __shared__ float red[32];
    const float * r = in + (size_t) blockIdx.x * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) srow[i] = r[i];
    __syncthreads();
    ln_row(srow, w, eps, W, out + (size_t) blockIdx.x * W, accumulate != 0, red);
}

template <typename WT>
__global__ void __launch_bounds__(256) embed_ln_kernel(const WT * __restrict__ embd, const int32_t * __restrict__ tok, const float * __restrict__ w, float eps, int W,
                                                       float * __restrict__ x) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float srow[];
    __shared__ float red[32];
    const WT * r = embd + (size_t) tok[blockIdx.x] * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) srow[i] = (float) r[i];
    __syncthreads();
    ln_row(srow, w, eps, W, x + (size_t) blockIdx.x * W, false, red);
}

int pib_embed_ln(const pib_weight * embd, const int32_t * tok, const float * w, float eps, int T, int W, float * x, cudaStream_t st) {
    if (embd->type == PIB_TYPE_BF16) pib_launch(embed_ln_kernel<__nv_bfloat16>, dim3(T), dim3(256), (size_t) ((size_t) W * 4), st, (const __nv_bfloat16 *) embd->base, tok, w, eps, W, x);
    else                             pib_launch(embed_ln_kernel<float>, dim3(T), dim3(256), (size_t) ((size_t) W * 4), st, (const float *) embd->base, tok, w, eps, W, x);
    CKL();
    return PIB_OK;
}

int pib_layer_norm(const float * in, const float * w, float eps, int T, int W, float * out, int accumulate, cudaStream_t st) {
    pib_launch(layer_norm_kernel, dim3(T), dim3(256), (size_t) ((size_t) W * 4), st, in, w, eps, W, out, accumulate);
    CKL();
    return PIB_OK;
}

// ---- causal convolution with a per-sequence tail ---------------------------------------------------------------------------------
// out[t][c] = (flags & 1 ? u[t][c] : 0) + (bias ? bias[c] : 0) + sum_j w[c][j] * in(t - taps + 1 + j)[c], then silu if flags & 2; in() is this batch's u inside the
// token's segment, the slot's tail ([taps-1][C]) before it.  u rows have pitch ldu, out rows pitch ldo; C channels.
#define CANON_MAX_TAPS 16
enum { CONV_ADD_INPUT = 1, CONV_SILU = 2, CONV_MOVE_TAIL = 4 };
__global__ void __launch_bounds__(256) canon_kernel(const float * __restrict__ x, int ldu, const float * __restrict__ w, int taps, const int32_t * __restrict__ seg,
                                                    const int32_t * __restrict__ seg_start, const int32_t * __restrict__ seg_slot,
                                                    float * __restrict__ state, size_t state_stride, size_t tail_off, int W, float * __restrict__ h, int ldo, int flags,
                                                    const float * __restrict__ bias) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x, sg = seg[t], s0 = seg_start[sg];
    float * tail = state + (size_t) seg_slot[sg] * state_stride + tail_off;
    const bool single = (flags & CONV_MOVE_TAIL) != 0;    // a batch of decoded tokens only: this block is the tail's only reader and moves it on itself
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += blockDim.x * gridDim.y) {       // channels are independent: a token's may be spread over several blocks
        float acc = (flags & CONV_ADD_INPUT) ? x[(size_t) t * ldu + c] : 0.f;
        if (bias) acc += bias[c];
        for (int j = 0; j < taps; j++) {
            const int tau = t - (taps - 1) + j;
            const float v = tau >= s0 ? x[(size_t) tau * ldu + c] : tail[(size_t) (taps - 1 + tau - s0) * W + c];
            acc = fmaf(w[(size_t) c * taps + j], v, acc);
            if (single && j > 0) tail[(size_t) (j - 1) * W + c] = v;      // row j - 1 was read in the trip before: every row moves up one place
        }
        if (flags & CONV_SILU) acc = acc / (1.0f + expf(-acc));
        h[(size_t) t * ldo + c] = acc;
    }
}

// after canon_kernel, when some segment has more than one token: the last taps-1 inputs of every segment become its slot's tail (old tail
// rows move up when the segment is shorter)
__global__ void __launch_bounds__(256) canon_tail_kernel(const float * __restrict__ x, int ldu, int taps, const int32_t * __restrict__ seg_start, const int32_t * __restrict__ seg_len,
                                                         const int32_t * __restrict__ seg_slot, float * __restrict__ state, size_t state_stride, size_t tail_off, int W) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int sg = blockIdx.x, s0 = seg_start[sg], s1 = s0 + seg_len[sg];
    float * tail = state + (size_t) seg_slot[sg] * state_stride + tail_off;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v[CANON_MAX_TAPS];
#pragma unroll
        for (int k = 0; k < CANON_MAX_TAPS; k++) {
            if (k < taps - 1) {
                const int tau = s1 - (taps - 1) + k;
                v[k] = tau >= s0 ? x[(size_t) tau * ldu + c] : tail[(size_t) (taps - 1 + tau - s0) * W + c];
            }
        }
#pragma unroll
        for (int k = 0; k < CANON_MAX_TAPS; k++) if (k < taps - 1) tail[(size_t) k * W + c] = v[k];
    }
}

// the general form: C channels of rows u (pitch ldu) -> out (pitch ldo); add_input: out += u; silu: activation on the way out
int pib_chan_conv(const float * u, int ldu, const float * w, int taps, const pib_hbatch & b, float * state, size_t state_stride, size_t tail_off, int C, float * out, int ldo,
                  int add_input, int silu, cudaStream_t st, const float * bias) {
    if (taps > CANON_MAX_TAPS || taps < 1) { pib_set_error("convolution: %d taps (1 to %d)", taps, CANON_MAX_TAPS); return PIB_ERR_UNSUPP; }
    // T == S: every segment is one token; its block moves the tail on itself and no tail kernel follows.  (In a batch that also holds longer
    // segments the tail kernel handles every segment, so no block may have moved a tail before it.)
    const int flags = (add_input ? CONV_ADD_INPUT : 0) | (silu ? CONV_SILU : 0) | (b.T == b.S ? CONV_MOVE_TAIL : 0);
    // few tokens (decode steps): a token's channels go to several blocks, so that more than a handful of SMs have loads in flight
    const unsigned ny = b.T > 32 ? 1u : (unsigned) std::min(16, (C + 255) / 256);
    pib_launch(canon_kernel, dim3((unsigned) b.T, ny), dim3(256), (size_t) (0), st, u, ldu, w, taps, b.seg, b.seg_start, b.seg_slot, state, state_stride, tail_off, C, out, ldo, flags, bias);
    CKL();
    if (taps > 1 && b.T > b.S) { pib_launch(canon_tail_kernel, dim3(b.S), dim3(256), (size_t) (0), st, u, ldu, taps, b.seg_start, b.seg_len, b.seg_slot, state, state_stride, tail_off, C); CKL(); }
    return PIB_OK;
}
// h = x + conv(x) over the model's width, in front of a mixer
int pib_canon_conv(const float * x, const float * w, int taps, const pib_hbatch & b, float * state, size_t state_stride, size_t tail_off, int W, float * h,
                   cudaStream_t st) {
    return pib_chan_conv(x, W, w, taps, b, state, state_stride, tail_off, W, h, W, 1, 0, st);
}

// ---- position -> cell table of each state slot -----------------------------------------------------------------------------------
__global__ void cellmap_kernel(int32_t * __restrict__ cellmap, int n_ctx, const int32_t * __restrict__ pos, const int32_t * __restrict__ cell,
                               const int32_t * __restrict__ slot, int T) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < T) cellmap[(size_t) slot[t] * n_ctx + pos[t]] = cell[t];
}
int pib_cellmap_set(int32_t * cellmap, int n_ctx, const pib_hbatch & b, cudaStream_t st) {
    pib_launch(cellmap_kernel, dim3((b.T + 255) / 256), dim3(256), (size_t) (0), st, cellmap, n_ctx, b.pos, b.cell, b.slot, b.T);
    CKL();
    return PIB_OK;
}

// coordinate i of a vector whose first rot_dims coordinates turn by the angles cs (pairs (i, i + rot_dims / 2) or (2 i, 2 i + 1))
__device__ __forceinline__ float rot_coord(const float * __restrict__ v, int i, int rot_dims, int pairs, const float2 * __restrict__ cs) {
    if (i >= rot_dims) return v[i];
    if (pairs == PIB_PAIR_ADJACENT) { const float2 c = cs[i >> 1]; return (i & 1) ? v[i] * c.x + v[i - 1] * c.y : v[i] * c.x - v[i + 1] * c.y; }
    const int half = rot_dims / 2;
    return i < half ? v[i] * cs[i].x - v[i + half] * cs[i].y : v[i] * cs[i - half].x + v[i - half] * cs[i - half].y;
}

// ---- latent attention: norms of the two latents, rotation of the shared key part, cache write --------------------------------------
// proj[t] = [W_dq h (q_rank) | W_dkv h (kv_rank + rot_dim)]; cq[t] = RMSnorm(first part) * dq_norm; with a cache of its own the layer
// writes cache[cell[t]] = [RMSnorm(next kv_rank) * dkv_norm | rotate(last rot_dim, pos[t])].  A layer without a query latent (q_rank 0)
// has its query rows in front instead, kv_off floats wide, and only the cache row is formed.
__global__ void __launch_bounds__(128) latent_prep_kernel(const float * __restrict__ proj, int ldp, int q_rank, int kv_off, int kv_rank, int rot_dim, int rot_dims, int pairs,
                                                          const float * __restrict__ dq_norm, const float * __restrict__ dkv_norm, float eps,
                                                          const int32_t * __restrict__ pos, const int32_t * __restrict__ cell,
                                                          const float2 * __restrict__ rope, float * __restrict__ cq, float * __restrict__ cache, int cache_row) {
    pib_pdl_wait();
    pib_pdl_trigger();
    __shared__ float red[32];
    const int     t = blockIdx.x;
    const float * p = proj + (size_t) t * ldp;
    float s = 0.f;
    if (q_rank > 0) {
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) s += p[i] * p[i];
        const float rq = 1.0f / sqrtf(block_sum(s, red) / q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t) t * q_rank + i] = p[i] * rq * dq_norm[i];
    }
    if (!cache) return;
    const float * d = p + kv_off;
    s = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) s += d[i] * d[i];
    const float rc = 1.0f / sqrtf(block_sum(s, red) / kv_rank + eps);
    float * row = cache + (size_t) cell[t] * cache_row;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) row[i] = d[i] * rc * dkv_norm[i];
    const float *  k = d + kv_rank;
    const float2 * cs = rope + (size_t) pos[t] * (rot_dims / 2);
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) row[kv_rank + i] = rot_coord(k, i, rot_dims, pairs, cs);
}

int pib_latent_prep(const float * proj, int ldp, int kv_off, const pib_hlayer & L, const float * dq_norm, const float * dkv_norm, float eps, const pib_hbatch & b,
                    const float2 * rope, int rope_n_pos, float * cq, float * cache, int cache_row, cudaStream_t st) {
    (void) rope_n_pos;
    pib_launch(latent_prep_kernel, dim3(b.T), dim3(128), (size_t) (0), st, proj, ldp, L.q_rank, kv_off, L.kv_rank, L.rot_dim, L.rot_dims, L.rot_pairs, dq_norm, dkv_norm, eps, b.pos, b.cell, rope, cq, cache, cache_row);
    CKL();
    return PIB_OK;
}

// ---- latent attention proper ---------------------------------------------------------------------------------------------------
// grid (token, head group); a block holds HPB heads x KS key shares, one warp each.  A warp walks its share of the window
// [max(0, p - window + 1), p], keeps a running maximum / denominator / weighted sum of latent rows (RPL registers per lane), and the
// shares of a head are merged in shared memory.  The sink enters as one more logit with no row: the running state starts at
// (max = sink, denominator = 1, sum = 0).
template <int RPL>
__global__ void __launch_bounds__(512) latent_attn_kernel(const float * __restrict__ q, int ldq, const float * __restrict__ qlat, int H, int D, int rot_dim, int rot_dims, int pairs, int R,
                                                          float scale, int window, const float * __restrict__ sink, const int32_t * __restrict__ pos,
                                                          const int32_t * __restrict__ slot, const float2 * __restrict__ rope, const float * __restrict__ cache,
                                                          int cache_row, const int32_t * __restrict__ cellmap, int n_ctx, int HPB, int KS, float * __restrict__ ctx,
                                                          const int32_t * __restrict__ skip) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float sm[];                 // [HPB * KS][R + 2] partial states, then [HPB][rot_dim] rotated queries
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (skip && skip[t]) return;                  // this token's segment goes through the matmul form (pib_latent_attention_mm)
    const int hl = warp / KS, ks = warp % KS, h = blockIdx.y * HPB + hl;
    const int p = pos[t], lo = max(0, p - window + 1);
    float * qr_s = sm + (size_t) HPB * KS * (R + 2) + (size_t) hl * rot_dim;
    const bool live = h < H;
    if (live && ks == 0) {
        const float *  qr = q + (size_t) t * ldq + (size_t) h * (D + rot_dim) + D;
        const float2 * cs = rope + (size_t) p * (rot_dims / 2);
        for (int i = lane; i < rot_dim; i += 32) qr_s[i] = rot_coord(qr, i, rot_dims, pairs, cs);
    }
    __syncthreads();
    float ql[RPL], acc[RPL];
    float m = -INFINITY, l = 0.f;
    if (live) {
        const float * qlp = qlat + ((size_t) t * H + h) * R;
#pragma unroll
        for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; ql[i] = r < R ? qlp[r] : 0.f; acc[i] = 0.f; }
        if (ks == 0 && sink) { m = sink[h]; l = 1.f; }
        const int32_t * map = cellmap + (size_t) slot[t] * n_ctx;
        for (int j = lo + ks; j <= p; j += KS) {
            const float * row = cache + (size_t) map[j] * cache_row;
            float c[RPL], s = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; c[i] = r < R ? row[r] : 0.f; s = fmaf(ql[i], c[i], s); }
            for (int i = lane; i < rot_dim; i += 32) s = fmaf(qr_s[i], row[R + i], s);
            s = warp_sum(s) * scale;
            const float mn = fmaxf(m, s), a = expf(m - mn), e = expf(s - mn);         // m == -inf only before the first key: a = 0
            l = l * a + e;
#pragma unroll
            for (int i = 0; i < RPL; i++) acc[i] = fmaf(acc[i], a, e * c[i]);
            m = mn;
        }
        float * part = sm + (size_t) warp * (R + 2);
#pragma unroll
        for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; if (r < R) part[r] = acc[i]; }
        if (lane == 0) { part[R] = m; part[R + 1] = l; }
    }
    __syncthreads();
    if (live && ks == 0) {
        const float * base = sm + (size_t) (hl * KS) * (R + 2);
        float M = -INFINITY;
        for (int k = 0; k < KS; k++) M = fmaxf(M, base[(size_t) k * (R + 2) + R]);
        float Lsum = 0.f, o[RPL];
#pragma unroll
        for (int i = 0; i < RPL; i++) o[i] = 0.f;
        for (int k = 0; k < KS; k++) {
            const float * pk = base + (size_t) k * (R + 2);
            const float   mk = pk[R];
            if (mk == -INFINITY) continue;           // a share that saw no key
            const float f = expf(mk - M);
            Lsum = fmaf(pk[R + 1], f, Lsum);
#pragma unroll
            for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; if (r < R) o[i] = fmaf(pk[r], f, o[i]); }
        }
        const float inv = 1.0f / Lsum;
        float * out = ctx + ((size_t) t * H + h) * R;
#pragma unroll
        for (int i = 0; i < RPL; i++) { const int r = i * 32 + lane; if (r < R) out[r] = o[i] * inv; }
    }
}

int pib_latent_attention(const float * q, int ldq, const float * qlat, const pib_hlayer & L, const pib_hbatch & b, const float2 * rope, int rope_n_pos,
                         const float * cache, int cache_row, const int32_t * cellmap, int n_ctx, float * ctx, const int32_t * skip, cudaStream_t st) {
    (void) rope_n_pos;
    const int H = L.heads, R = L.kv_rank;
    // few tokens (decoding): one head per CTA and 16 key shares, so that a step still fills some of the machine
    const int HPB = (long long) b.T * H <= 1024 ? 1 : (H < 4 ? H : 4);
    int KS = 16 / HPB;
    if (L.window < 64) KS = 1;
    while (KS > 1 && (size_t) HPB * KS * (R + 2) * 4 > 160 * 1024) KS >>= 1;
    const size_t smem = ((size_t) HPB * KS * (R + 2) + (size_t) HPB * L.rot_dim) * 4;
    dim3 grid((unsigned) b.T, (unsigned) ((H + HPB - 1) / HPB));
    const int threads = HPB * KS * 32;
#define LA_GO(RPL) do {                                                                                                            \
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_attn_kernel<RPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem); \
        pib_launch(latent_attn_kernel<RPL>, dim3(grid), dim3(threads), (size_t) (smem), st, q, ldq, qlat, H, L.dim, L.rot_dim, L.rot_dims, L.rot_pairs, R, L.scale, L.window, (const float *) L.sink, b.pos,  \
                                                             b.slot, rope, cache, cache_row, cellmap, n_ctx, HPB, KS, ctx, skip); \
    } while (0)
    if (R <= 128) LA_GO(4); else if (R <= 256) LA_GO(8); else if (R <= 512) LA_GO(16);
    else { pib_set_error("latent attention: kv_rank %d (max 512)", R); return PIB_ERR_UNSUPP; }
#undef LA_GO
    CKL();
    return PIB_OK;
}

// ---- latent attention as matmuls (long portions, served mode) ----------------------------------------------------------------------
// For a block of consecutive tokens of one segment the scores against the block's key range [j0, j0 + NK) are one matmul, the masked
// softmax with the sink one pass over the score rows, and the weighted sums of latent rows a second matmul.  These kernels prepare the
// operands: the keys' rows as bfloat16 [NK][R + rot_dim] and, transposed and twice side by side, [R][2 NKp] (NKp = NK rounded up to 8, the pad zero;
// twice because a weight enters the value matmul as its bfloat16 part plus the remainder of that rounding), and the
// queries as rows [(token, head)][R + rot_dim] = scale * [W_uk^T q | rotated q part].
__global__ void __launch_bounds__(128) lat_gather_kernel(const float * __restrict__ cache, int cache_row, const int32_t * __restrict__ map, int j0, int NK, int NKp, int R,
                                                         int RK, __nv_bfloat16 * __restrict__ Kb, __nv_bfloat16 * __restrict__ Vt) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int j = blockIdx.x;
    if (j < NK) {
        const float * row = cache + (size_t) map[j0 + j] * cache_row;
        for (int i = threadIdx.x; i < RK; i += blockDim.x) {
            const __nv_bfloat16 v = __float2bfloat16_rn(row[i]);
            Kb[(size_t) j * RK + i] = v;
            if (i < R) { Vt[(size_t) i * 2 * NKp + j] = v; Vt[(size_t) i * 2 * NKp + NKp + j] = v; }
        }
    } else {
        for (int i = threadIdx.x; i < R; i += blockDim.x) { Vt[(size_t) i * 2 * NKp + j] = __float2bfloat16_rn(0.f); Vt[(size_t) i * 2 * NKp + NKp + j] = __float2bfloat16_rn(0.f); }
    }
}
__global__ void __launch_bounds__(128) lat_qcat_kernel(const float * __restrict__ q, int ldq, const float * __restrict__ qlat, int H, int D, int rot_dim, int rot_dims, int pairs, int R,
                                                       float scale, const int32_t * __restrict__ pos, const float2 * __restrict__ rope, int t0, float * __restrict__ Qc) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = t0 + blockIdx.x, h = blockIdx.y, RK = R + rot_dim;
    float *       out = Qc + ((size_t) blockIdx.x * H + h) * RK;
    const float * ql = qlat + ((size_t) t * H + h) * R;
    for (int i = threadIdx.x; i < R; i += blockDim.x) out[i] = ql[i] * scale;
    const float *  qr = q + (size_t) t * ldq + (size_t) h * (D + rot_dim) + D;
    const float2 * cs = rope + (size_t) pos[t] * (rot_dims / 2);
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) out[R + i] = rot_coord(qr, i, rot_dims, pairs, cs) * scale;
}
// one score row per (token, head), in place: keys outside [p - window + 1, p] (chunk mask: outside [p - p % window, p]) and the pad get weight 0, the sink (optional) one share of
// the denominator.  Rows come in groups of rows_per_z (one group per problem of the score matmul), inside a group `rep` heads per token:
// token t0 + (row % rows_per_z) / rep, head (row / rows_per_z) * rep + (row % rows_per_z) % rep.
__global__ void __launch_bounds__(256) lat_softmax_kernel(float * __restrict__ S, __nv_bfloat16 * __restrict__ P, int NKp, int NK, int j0, int window,
                                                          const int32_t * __restrict__ pos, int t0, int rows_per_z, int rep, const float * __restrict__ sink, int mask) {
    pib_pdl_wait();
    pib_pdl_trigger();
    __shared__ float red[32];
    const int row = blockIdx.x, rz = row % rows_per_z, t = t0 + rz / rep, h = (row / rows_per_z) * rep + rz % rep, p = pos[t];
    float *   s = S + (size_t) row * NKp;
    __nv_bfloat16 * pw = P + (size_t) row * 2 * NKp;   // [weights' bfloat16 part | what the rounding left]: the value matmul sees both, so the weights keep fp32 accuracy
    const int lo = (mask == PIB_MASK_CHUNK ? p - p % window : max(0, p - window + 1)) - j0, hi = p - j0;            // valid columns [lo, hi]
    const float sk = sink ? sink[h] : -INFINITY;
    float m = sk;
    for (int j = lo + (int) threadIdx.x; j <= hi; j += blockDim.x) m = fmaxf(m, s[j]);
    m = warp_max(m);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    for (int i = 0; i < (int) (blockDim.x >> 5); i++) m = fmaxf(m, red[i]);
    float sum = 0.f;
    for (int j = threadIdx.x; j < NKp; j += blockDim.x) {
        const float e = (j >= lo && j <= hi) ? expf(s[j] - m) : 0.f;
        s[j] = e;
        sum += e;
    }
    const float inv = 1.0f / (block_sum(sum, red) + (sink ? expf(sk - m) : 0.f));
    for (int j = threadIdx.x; j < NKp; j += blockDim.x) {
        const float p = s[j] * inv;
        const __nv_bfloat16 hi16 = __float2bfloat16_rn(p);
        pw[j] = hi16;
        pw[NKp + j] = __float2bfloat16_rn(p - __bfloat162float(hi16));
    }
    (void) NK; (void) hi;
}
int pib_window_softmax(float * S, void * P, int NKp, int NK, int j0, int window, const int32_t * pos, int t0, int n_rows, int rows_per_z, int rep, const float * sink,
                       cudaStream_t st, int mask) {
    pib_launch(lat_softmax_kernel, dim3(n_rows), dim3(256), (size_t) (0), st, S, (__nv_bfloat16 *) P, NKp, NK, j0, window, pos, t0, rows_per_z, rep, sink, mask);
    CKL();
    return PIB_OK;
}

// bfloat16 weight rows back to fp32 rows (same pitch), for the few-row matmul kernels
__global__ void lat_widen_kernel(const __nv_bfloat16 * __restrict__ P, int n, float * __restrict__ S) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const __nv_bfloat16 * p = P + (size_t) blockIdx.x * n;
    float * s = S + (size_t) blockIdx.x * n;
    for (int j = threadIdx.x; j < n; j += blockDim.x) s[j] = __bfloat162float(p[j]);
}

// the block of `nq` tokens starting at batch row t0 (positions p0 ..), keys [j0, j0 + NK): ctx rows [(token, head)][R] of those tokens
int pib_latent_attention_mm(const float * q, int ldq, const float * qlat, const pib_hlayer & L, const pib_hbatch & b, const float2 * rope, const float * cache, int cache_row,
                            const int32_t * map, int t0, int nq, int j0, int NK, void * Kb, void * Vt, float * Qc, float * S, void * P, float * ctx, cudaStream_t st) {
    const int H = L.heads, R = L.kv_rank, RK = R + L.rot_dim, NKp = (NK + 7) & ~7;
    pib_launch(lat_gather_kernel, dim3(NKp), dim3(128), (size_t) (0), st, cache, cache_row, map, j0, NK, NKp, R, RK, (__nv_bfloat16 *) Kb, (__nv_bfloat16 *) Vt);
    CKL();
    pib_launch(lat_qcat_kernel, dim3(dim3((unsigned) nq, (unsigned) H)), dim3(128), (size_t) (0), st, q, ldq, qlat, H, L.dim, L.rot_dim, L.rot_dims, L.rot_pairs, R, L.scale, b.pos, rope, t0, Qc);
    CKL();
    pib_mm a;
    a.W = Kb; a.wtype = PIB_TYPE_BF16; a.ldw = RK; a.X = Qc; a.ldx = RK; a.Y = S; a.ldy = NKp; a.M = nq * H; a.N = NK; a.K = RK;
    int rc = pib_dense_mm(a, st);
    if (rc != PIB_OK) return rc;
    if ((rc = pib_window_softmax(S, P, NKp, NK, j0, L.window, b.pos, t0, nq * H, nq * H, H, L.sink, st)) != PIB_OK) return rc;
    pib_mm v;
    v.W = Vt; v.wtype = PIB_TYPE_BF16; v.ldw = 2 * NKp; v.Y = ctx + (size_t) t0 * H * R; v.ldy = R; v.M = nq * H; v.N = R; v.K = 2 * NKp;
    if (nq * H > 16) { v.X = (const float *) P; v.ldx = 2 * NKp; v.x_bf16 = 1; return pib_dense_mm(v, st); }
    // a last block of very few rows goes to the row kernel, which reads fp32: widen the weights again
    pib_launch(lat_widen_kernel, dim3((unsigned) (nq * H)), dim3(256), (size_t) 0, st, (const __nv_bfloat16 *) P, 2 * NKp, S);
    CKL();
    v.X = S; v.ldx = 2 * NKp;
    return pib_dense_mm(v, st);
}

// ---- HGRN2 ----------------------------------------------------------------------------------------------------------------------
// in place on the projection rows [q | f | v]: q <- silu(q), f <- lower + (1 - lower) * sigmoid(f + bias)
__global__ void hgrn2_gate_kernel(float * __restrict__ qfv, int ld, const float * __restrict__ f_bias, const float * __restrict__ lower, int T, int HD) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t) T * HD) return;
    const int t = (int) (i / HD), c = (int) (i % HD);
    float *   r = qfv + (size_t) t * ld;
    const float qv = r[c];
    r[c] = qv / (1.0f + expf(-qv));
    const float lo = lower[c], g = 1.0f / (1.0f + expf(-(r[HD + c] + f_bias[c])));
    r[HD + c] = lo + (1.0f - lo) * g;
}
int pib_hgrn2_gates(float * qfv, int ld, const float * f_bias, const float * lower, int T, int HD, cudaStream_t st) {
    const int64_t n = (int64_t) T * HD;
    pib_launch(hgrn2_gate_kernel, dim3((unsigned) ((n + 255) / 256)), dim3(256), (size_t) (0), st, qfv, ld, f_bias, lower, T, HD);
    CKL();
    return PIB_OK;
}

// grid (segment, head, tile of HG_VT value columns), 16 * HG_VT threads: the 16 lanes of a half-warp share one column of the head's
// matrix, lane `part` keeping rows part, part + 16, part + 32, ... in registers (columns are independent, so a head is spread over
// vdim / HG_VT CTAs and the machine holds several warps per scheduler; neighbouring lanes read neighbouring words of shared memory, no
// bank conflicts).  A step is s <- v + f (s - v) (= f s + (1 - f) v) and a dot product with q, reduced over the 16 lanes by shuffles.
// The tokens' q, f and v come through shared memory in chunks of HG_CHUNK tokens, the next chunk in flight (cp.async) while this one is
// walked; the matrix is read from the slot at the start of the segment and left there at its end.  FULL: dim == 16 RPT, no row guards.
#define HG_CHUNK 16
#define HG_VT    8
template <int RPT, bool FULL>
__global__ void __launch_bounds__(16 * HG_VT) hgrn2_scan_kernel(const float * __restrict__ qfv, int ld, int H, int D, int V, const int32_t * __restrict__ seg_start,
                                                                const int32_t * __restrict__ seg_len, const int32_t * __restrict__ seg_slot, float * __restrict__ state,
                                                                size_t state_stride, size_t state_off, float * __restrict__ out) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float hs[];                  // 2 x [HG_CHUNK][2 D + HG_VT]: the chunk being walked and the one in flight
    const int sg = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * HG_VT, part = threadIdx.x & 15, vl = threadIdx.x >> 4, vd = v0 + vl;
    const int s0 = seg_start[sg], n = seg_len[sg], HD = H * D, row_f = 2 * D + HG_VT;
    const bool vok = vd < V;
    float *   S = state + (size_t) seg_slot[sg] * state_stride + state_off + (size_t) h * D * V;
    float s[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) { const int d = part + 16 * r; s[r] = ((FULL || d < D) && vok) ? S[(size_t) d * V + vd] : 0.f; }
    auto fetch = [&](int c0, int buf) {
        const int nc = min(HG_CHUNK, n - c0);
        for (int t = 0; t < nc; t++) {
            const float * row = qfv + (size_t) (s0 + c0 + t) * ld + (size_t) h * D;
            const uint32_t dst = (uint32_t) __cvta_generic_to_shared(hs + (buf * HG_CHUNK + t) * row_f);
            for (int e = threadIdx.x; e < D; e += blockDim.x) {
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * e), "l"(row + e) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * (D + e)), "l"(row + HD + e) : "memory");
            }
            if (threadIdx.x < HG_VT && v0 + (int) threadIdx.x < V)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * (2 * D + threadIdx.x)), "l"(qfv + (size_t) (s0 + c0 + t) * ld + 2 * HD + (size_t) h * V + v0 + threadIdx.x) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n > 0) fetch(0, 0);
    int buf = 0;
    float * op = out + (size_t) s0 * H * V + (size_t) h * V + vd;
    const int ostride = H * V;
    for (int c0 = 0; c0 < n; c0 += HG_CHUNK, buf ^= 1) {
        const int nc = min(HG_CHUNK, n - c0);
        if (c0 + HG_CHUNK < n) { fetch(c0 + HG_CHUNK, buf ^ 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else                   asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float * qp = hs + buf * HG_CHUNK * row_f + part;
#pragma unroll 4
        for (int t = 0; t < nc; t++, qp += row_f, op += ostride) {
            const float v = vok ? qp[2 * D + vl - part] : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < RPT; r++) {
                if (FULL || part + 16 * r < D) {
                    s[r] = fmaf(qp[D + 16 * r], s[r] - v, v);
                    acc = fmaf(qp[16 * r], s[r], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            if (part == 0 && vok) *op = acc;
        }
        __syncthreads();                           // everyone is done with this buffer before the fetch after next refills it
    }
#pragma unroll
    for (int r = 0; r < RPT; r++) { const int d = part + 16 * r; if ((FULL || d < D) && vok) S[(size_t) d * V + vd] = s[r]; }
}

// one warp per (token, head): o <- o / sqrt(mean(o^2) + eps) * w
__global__ void head_rmsnorm_kernel(float * __restrict__ o, int n_rows, int V, const float * __restrict__ w, float eps) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    float * r = o + (size_t) row * V;
    float s = 0.f;
    for (int i = lane; i < V; i += 32) s += r[i] * r[i];
    const float inv = 1.0f / sqrtf(warp_sum(s) / V + eps);
    for (int i = lane; i < V; i += 32) r[i] = r[i] * inv * w[i];
}

int pib_hgrn2_scan(const float * qfv, int ld, const pib_hlayer & L, const pib_hbatch & b, float * state, size_t state_stride, const float * onorm, float eps,
                   float * out, cudaStream_t st) {
    const int H = L.heads, D = L.dim, V = L.vdim;
    if (D > 256) { pib_set_error("hgrn2: dim %d not supported (up to 256)", D); return PIB_ERR_UNSUPP; }
    dim3 grid((unsigned) b.S, (unsigned) H, (unsigned) ((V + HG_VT - 1) / HG_VT));
    const size_t smem = (size_t) 2 * HG_CHUNK * (2 * D + HG_VT) * 4;
#define HG_GO(RPT, FULL) pib_launch(hgrn2_scan_kernel<RPT, FULL>, dim3(grid), dim3(16 * HG_VT), (size_t) (smem), st, qfv, ld, H, D, V, b.seg_start, b.seg_len, b.seg_slot, state, \
                                    state_stride, L.state_off, out)
    if (D == 64)       HG_GO(4, true);
    else if (D == 128) HG_GO(8, true);
    else if (D <= 64)  HG_GO(4, false);
    else if (D <= 128) HG_GO(8, false);
    else               HG_GO(16, false);
#undef HG_GO
    CKL();
    const int n_rows = b.T * H;
    pib_launch(head_rmsnorm_kernel, dim3((n_rows + 7) / 8), dim3(256), (size_t) (0), st, out, n_rows, V, onorm, eps);
    CKL();
    return PIB_OK;
}

// ---- PolyNorm: z <- a N(z) + b N(z^2) + c N(z^3) + e, N(u) = u / sqrt(mean(u^2) + eps) over the token's row ---------------------------
__global__ void __launch_bounds__(256) polynorm_kernel(float * __restrict__ z, int F, float a, float b, float c, float e, float eps) {
    pib_pdl_wait();
    pib_pdl_trigger();
    __shared__ float red[32];
    float * r = z + (size_t) blockIdx.x * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) { const float v = r[i], v2 = v * v; s2 += v2; s4 += v2 * v2; s6 += v2 * v2 * v2; }
    const float n1 = a / sqrtf(block_sum(s2, red) / F + eps);
    const float n2 = b / sqrtf(block_sum(s4, red) / F + eps);
    const float n3 = c / sqrtf(block_sum(s6, red) / F + eps);
    for (int i = threadIdx.x; i < F; i += blockDim.x) { const float v = r[i]; r[i] = fmaf(v, n1, fmaf(v * v, n2, fmaf(v * v * v, n3, e))); }
}
int pib_polynorm(float * z, int T, int F, const float * act4, float eps, cudaStream_t st) {
    pib_launch(polynorm_kernel, dim3(T), dim3(256), (size_t) (0), st, z, F, act4[0], act4[1], act4[2], act4[3], eps);
    CKL();
    return PIB_OK;
}

// ---- mixture of experts ------------------------------------------------------------------------------------------------------------
// one warp per token: the `top` largest logits (ties: the lower index).  mode PIB_ROUTE_SOFTMAX_RENORM: scores = softmax over the E
// logits, weights = score / (sum of the chosen + 1e-20); PIB_ROUTE_SIGMOID: weights = sigmoid(logit) of the chosen, as they are (the
// order of the logits is the order of their sigmoids)
#define MOE_MAX_TOP 16
__global__ void moe_route_kernel(const float * __restrict__ logits, int T, int E, int top, int mode, int32_t * __restrict__ ids, float * __restrict__ wts) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const float * z = logits + (size_t) t * E;
    float mx = -INFINITY;
    for (int i = lane; i < E; i += 32) mx = fmaxf(mx, z[i]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < E; i += 32) sum += expf(z[i] - mx);
    sum = warp_sum(sum);
    int   chosen[MOE_MAX_TOP];
    float score[MOE_MAX_TOP], tot = 0.f;
    for (int k = 0; k < top; k++) {
        float bv = -INFINITY;
        int   bi = 0x7fffffff;
        for (int i = lane; i < E; i += 32) {
            bool taken = false;
            for (int j = 0; j < k; j++) taken |= chosen[j] == i;
            const float v = z[i];
            if (!taken && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int   oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        chosen[k] = bi;
        score[k]  = mode == PIB_ROUTE_SIGMOID ? 1.0f / (1.0f + expf(-bv)) : expf(bv - mx) / sum;
        tot += score[k];
    }
    if (lane == 0)
        for (int k = 0; k < top; k++) { ids[(size_t) t * top + k] = chosen[k]; wts[(size_t) t * top + k] = mode == PIB_ROUTE_SIGMOID ? score[k] : score[k] / (tot + 1e-20f); }
}
int pib_moe_route(const float * logits, int T, int E, int top, int mode, int32_t * ids, float * wts, cudaStream_t st) {
    if (top > MOE_MAX_TOP || top > E) { pib_set_error("router: top %d of %d experts (max %d)", top, E, MOE_MAX_TOP); return PIB_ERR_UNSUPP; }
    pib_launch(moe_route_kernel, dim3((T + 7) / 8), dim3(256), (size_t) (0), st, logits, T, E, top, mode, ids, wts);
    CKL();
    return PIB_OK;
}

// pairs (token, k) grouped by expert, inside an expert in pair order: counts[e]; offs[e] = first sorted position of expert e;
// perm[sorted position] = pair; inv[pair] = sorted position.  No atomics: the order, and so every sum formed from it, is fixed.
__global__ void __launch_bounds__(256) moe_count_kernel(const int32_t * __restrict__ ids, int n_pairs, int32_t * __restrict__ counts) {
    pib_pdl_wait();
    pib_pdl_trigger();
    __shared__ float red[32];
    const int e = blockIdx.x;
    int n = 0;
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) n += ids[i] == e;
    const float tot = block_sum((float) n, red);          // exact below 2^24 pairs
    if (threadIdx.x == 0) counts[e] = (int32_t) tot;
}
__global__ void __launch_bounds__(256) moe_fill_kernel(const int32_t * __restrict__ ids, int n_pairs, int E, const int32_t * __restrict__ counts,
                                                       int32_t * __restrict__ offs, int32_t * __restrict__ perm, int32_t * __restrict__ inv) {
    pib_pdl_wait();
    pib_pdl_trigger();
    __shared__ int wsum[8];
    __shared__ int base_s;
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        int o = 0;
        for (int i = 0; i < e; i++) o += counts[i];
        base_s = o;
        offs[e] = o;
        if (e == E - 1) offs[E] = o + counts[e];
    }
    __syncthreads();
    int base = base_s;
    for (int i0 = 0; i0 < n_pairs; i0 += 256) {
        const int  i = i0 + threadIdx.x;
        const bool mine = i < n_pairs && ids[i] == e;
        const unsigned bal = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) wsum[warp] = __popc(bal);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < 8; w++) { if (w < warp) before += wsum[w]; total += wsum[w]; }
        if (mine) {
            const int p = base + before + __popc(bal & ((1u << lane) - 1u));
            perm[p] = i;
            inv[i]  = p;
        }
        base += total;
        __syncthreads();
    }
}
int pib_moe_sort(const int32_t * ids, int n_pairs, int E, int32_t * counts, int32_t * offs, int32_t * perm, int32_t * inv, cudaStream_t st) {
    if (n_pairs >= (1 << 24)) { pib_set_error("router: %d pairs in one batch", n_pairs); return PIB_ERR_UNSUPP; }
    pib_launch(moe_count_kernel, dim3(E), dim3(256), (size_t) (0), st, ids, n_pairs, counts);
    CKL();
    pib_launch(moe_fill_kernel, dim3(E), dim3(256), (size_t) (0), st, ids, n_pairs, E, counts, offs, perm, inv);
    CKL();
    return PIB_OK;
}

// y[t] = shared[t] + sum_k w[t][k] * edn[inv[t * top + k]]   (k in ascending order)
__global__ void moe_combine_kernel(const float * __restrict__ shared, const float * __restrict__ edn, const float * __restrict__ wts, const int32_t * __restrict__ inv,
                                   int top, int W, float * __restrict__ y) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = shared ? shared[(size_t) t * W + c] : 0.f;
        for (int k = 0; k < top; k++) acc = fmaf(wts[(size_t) t * top + k], edn[(size_t) inv[(size_t) t * top + k] * W + c], acc);
        y[(size_t) t * W + c] = acc;
    }
}
int pib_moe_combine(const float * shared, const float * edn, const float * wts, const int32_t * inv, int T, int top, int W, float * y, cudaStream_t st) {
    pib_launch(moe_combine_kernel, dim3(T), dim3(256), (size_t) (0), st, shared, edn, wts, inv, top, W, y);
    CKL();
    return PIB_OK;
}
