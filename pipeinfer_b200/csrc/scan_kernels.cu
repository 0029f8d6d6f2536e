// scan_kernels.cu -- more parts for layer-list models (hybrid.cuh), all fp32:
//
//   the pre-norm frame: the residual sum, an RMS norm whose weight is ONE number and the token shift h_t + (h_{t-1} - h_t) * mu in one
//       pass; embedding rows kept beside the stream for layers that are walked again; the opening [stream ; embedding] of a walk
//   the selective state-space scan: per channel c and state n  S <- exp(dt_c A[c][n]) S + dt_c u_c B_n,  y_c = sum_n S C_n + D_c u_c,
//       dt = softplus(raw + bias), the output gated by silu(z)
//   the two-branch mixer's per-token work: biases, rotation ("rotate half" pairing) of the first rot_dims coordinates of every query /
//       key head, unit RMS per head, cache write [key | unrotated key as the value], silu on the linear branch's q | k | v; and after
//       both branches: head gates on the softmax branch, RMS norm over all heads times sigmoid gates on the linear branch, both
//       scaled into one row for the shared output matmul
#include "hybrid.cuh"

#include <cuda_bf16.h>

#define CKL() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) { pib_set_error("%s:%d: launch failed: %s", __FILE__, __LINE__, cudaGetErrorString(e__)); return PIB_ERR_CUDA; } } while (0)

__device__ __forceinline__ float sk_block_sum(float v, float * red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}
__device__ __forceinline__ float sk_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float sk_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sk_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---- the pre-norm frame ------------------------------------------------------------------------------------------------------------
// x'[t] = (xin ? xin[t] : 0) + (y ? y[t] : 0) + (bias ? bias : 0), stored to xout when xout is given (a buffer other than xin: the block of
// token t + 1 forms x'[t] from the same inputs).  n[t] = x'[t] / sqrt(mean(x'[t]^2) + eps) * g.  Without mu h[t] = n[t]; with mu
// h[t] = n[t] + (n[t - 1] - n[t]) * mu, where n[t - 1] of a segment's first token is the slot's row (zeros at a sequence's start).
__global__ void __launch_bounds__(256) prenorm_shift_kernel(const float * __restrict__ xin, const float * __restrict__ y, const float * __restrict__ bias, float * __restrict__ xout,
                                                            float g, float eps, const float * __restrict__ mu, const int32_t * __restrict__ seg,
                                                            const int32_t * __restrict__ seg_start, const int32_t * __restrict__ seg_len, const int32_t * __restrict__ seg_slot,
                                                            float * __restrict__ state, size_t state_stride, size_t shift_off, int W, float * __restrict__ h) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float srow[];               // [2][W]: this token's row, the previous token's
    __shared__ float red[32];
    const int t = blockIdx.x;
    const bool inside = mu && t > seg_start[seg[t]];        // the previous token is in this batch
    float s0 = 0.f, s1 = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = bias ? bias[i] : 0.f, u = v;
        if (xin) { v += xin[(size_t) t * W + i]; if (inside) u += xin[(size_t) (t - 1) * W + i]; }
        if (y)   { v += y[(size_t) t * W + i];   if (inside) u += y[(size_t) (t - 1) * W + i]; }
        srow[i] = v; srow[W + i] = u;
        s0 = fmaf(v, v, s0); s1 = fmaf(u, u, s1);
        if (xout) xout[(size_t) t * W + i] = v;
    }
    const float inv0 = g / sqrtf(sk_block_sum(s0, red) / W + eps);
    float inv1 = 0.f;
    if (inside) inv1 = g / sqrtf(sk_block_sum(s1, red) / W + eps);
    float * prev = mu ? state + (size_t) seg_slot[seg[t]] * state_stride + shift_off : nullptr;
    const bool single = mu && seg_len[seg[t]] == 1;          // a decoded token: this block is the only reader of the slot's row and leaves its own there
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float n = srow[i] * inv0;
        float o = n;
        if (mu) { const float pn = inside ? srow[W + i] * inv1 : prev[i]; o = fmaf(pn - n, mu[i], n); }
        h[(size_t) t * W + i] = o;
        if (single) prev[i] = n;
    }
}
// after prenorm_shift_kernel, when some segment has more than one token (its first token's block reads the slot's row, so its last token's
// block cannot replace it in the same launch): the normed (unshifted) row of every segment's last token becomes its slot's previous row
__global__ void __launch_bounds__(256) prenorm_tail_kernel(const float * __restrict__ xin, const float * __restrict__ y, const float * __restrict__ bias, float g, float eps,
                                                           const int32_t * __restrict__ seg_start, const int32_t * __restrict__ seg_len, const int32_t * __restrict__ seg_slot,
                                                           float * __restrict__ state, size_t state_stride, size_t shift_off, int W) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float srow[];
    __shared__ float red[32];
    const int sg = blockIdx.x, t = seg_start[sg] + seg_len[sg] - 1;
    float s0 = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = bias ? bias[i] : 0.f;
        if (xin) v += xin[(size_t) t * W + i];
        if (y)   v += y[(size_t) t * W + i];
        srow[i] = v;
        s0 = fmaf(v, v, s0);
    }
    const float inv0 = g / sqrtf(sk_block_sum(s0, red) / W + eps);
    float * dst = state + (size_t) seg_slot[sg] * state_stride + shift_off;
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = srow[i] * inv0;
}
int pib_prenorm_shift(const float * xin, const float * y, const float * bias, float * xout, float g, float eps, const float * mu, const pib_hbatch & b, float * state,
                      size_t state_stride, size_t shift_off, int W, float * h, cudaStream_t st) {
    if (xout && xout == xin) { pib_set_error("pre-norm: the updated stream needs a buffer of its own"); return PIB_ERR_ARG; }
    pib_launch(prenorm_shift_kernel, dim3(b.T), dim3(256), (size_t) 2 * W * 4, st, xin, y, bias, xout, g, eps, mu, b.seg, b.seg_start, b.seg_len, b.seg_slot, state, state_stride,
               shift_off, W, h);
    CKL();
    if (mu && b.T > b.S) {            // T == S: every segment is one token, the blocks have left their rows themselves
        pib_launch(prenorm_tail_kernel, dim3(b.S), dim3(256), (size_t) W * 4, st, xin, y, bias, g, eps, b.seg_start, b.seg_len, b.seg_slot, state, state_stride, shift_off, W);
        CKL();
    }
    return PIB_OK;
}

// x[t] = embedding row of tok[t]; with cat ([T][2 W]) the row is also kept in cat's second half
template <typename WT>
__global__ void __launch_bounds__(256) embed_pair_kernel(const WT * __restrict__ embd, const int32_t * __restrict__ tok, int W, float * __restrict__ x, float * __restrict__ cat) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const WT * r = embd + (size_t) tok[blockIdx.x] * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = (float) r[i];
        x[(size_t) blockIdx.x * W + i] = v;
        if (cat) cat[(size_t) blockIdx.x * 2 * W + W + i] = v;
    }
}
int pib_embed_pair(const pib_weight * embd, const int32_t * tok, int T, int W, float * x, float * cat, cudaStream_t st) {
    if (embd->type == PIB_TYPE_BF16) pib_launch(embed_pair_kernel<__nv_bfloat16>, dim3(T), dim3(256), (size_t) 0, st, (const __nv_bfloat16 *) embd->base, tok, W, x, cat);
    else                             pib_launch(embed_pair_kernel<float>, dim3(T), dim3(256), (size_t) 0, st, (const float *) embd->base, tok, W, x, cat);
    CKL();
    return PIB_OK;
}
// cat[t][0 .. W) = xin[t] + y[t] + bias (each optional): the stream as a walk's opening reads it, beside the embedding row
__global__ void __launch_bounds__(256) concat_stream_kernel(const float * __restrict__ xin, const float * __restrict__ y, const float * __restrict__ bias, int W, float * __restrict__ cat) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = bias ? bias[i] : 0.f;
        if (xin) v += xin[t * W + i];
        if (y)   v += y[t * W + i];
        cat[t * 2 * W + i] = v;
    }
}
int pib_concat_stream(const float * xin, const float * y, const float * bias, int T, int W, float * cat, cudaStream_t st) {
    pib_launch(concat_stream_kernel, dim3(T), dim3(256), (size_t) 0, st, xin, y, bias, W, cat);
    CKL();
    return PIB_OK;
}

// ---- selective state-space scan --------------------------------------------------------------------------------------------------------
// grid (segment, tile of SS_THREADS / P channels), SS_THREADS threads: the P lanes of a channel keep states part, part + P, ... in
// registers (P = 16 from 16 states on: one state per lane at 16, so that a layer of a few thousand channels fills the machine with warps;
// measured at 16 states and 4 096 channels: 4 lanes 0.89 ms, 8 lanes 0.54 ms, 16 lanes 0.46 ms per 2 048 tokens).  A chunk of SS_TC tokens is staged in shared memory (dt with its bias and softplus applied once per channel and token),
// walked token by token, and its outputs leave in whole rows, gated by silu(z) on the way out.  The states are read from the slot at
// the segment's start and left there at its end.
#define SS_THREADS 128
#define SS_TC      16
struct ss_args {
    const float * u; int ldu;                // after convolution and silu
    const float * dtr; int lddt;             // W_dt (.) before bias and softplus
    const float * bc; int ldbc;              // [B (N) | C (N)]
    const float * z; int ldz;                // gate rows
    const float * dt_bias, * A, * Dk;        // [inner], [inner][N] (negative), [inner]
    int inner, N;
    const int32_t * seg_start, * seg_len, * seg_slot;
    float * state; size_t state_stride, state_off;
    float * out;                             // [T][inner]
};
template <int P, int NPL>
__global__ void __launch_bounds__(SS_THREADS) ssm_scan_kernel(ss_args a) {
    pib_pdl_wait();
    pib_pdl_trigger();
    constexpr int CH = SS_THREADS / P, TB = NPL <= 2 ? 4 : NPL <= 8 ? 2 : 1;
    extern __shared__ float sm[];
    const int N = a.N, sg = blockIdx.x, c0 = blockIdx.y * CH, cl = threadIdx.x / P, part = threadIdx.x % P, c = c0 + cl;
    float * dts = sm, * us = dts + SS_TC * CH, * zs = us + SS_TC * CH, * ys = zs + SS_TC * CH, * Bs = ys + SS_TC * CH, * Cs = Bs + SS_TC * N;
    const int s0 = a.seg_start[sg], n = a.seg_len[sg];
    const bool cok = c < a.inner;
    float * S = a.state + (size_t) a.seg_slot[sg] * a.state_stride + a.state_off + (size_t) (cok ? c : 0) * N;
    float s[NPL], Ar[NPL];
#pragma unroll
    for (int r = 0; r < NPL; r++) {
        const int k = part + P * r;
        const bool ok = cok && k < N;
        s[r] = ok ? S[k] : 0.f;
        Ar[r] = ok ? a.A[(size_t) c * N + k] : 0.f;
    }
    const float Dc = cok ? a.Dk[c] : 0.f;
    for (int t0 = 0; t0 < n; t0 += SS_TC) {
        const int nc = min(SS_TC, n - t0);
        for (int i = threadIdx.x; i < nc * CH; i += blockDim.x) {
            const int tt = i / CH, cc = i % CH, ch = c0 + cc;
            const size_t row = (size_t) (s0 + t0 + tt);
            const bool ok = ch < a.inner;
            dts[i] = ok ? sk_softplus(a.dtr[row * a.lddt + ch] + a.dt_bias[ch]) : 0.f;
            us[i]  = ok ? a.u[row * a.ldu + ch] : 0.f;
            zs[i]  = ok ? a.z[row * a.ldz + ch] : 0.f;
        }
        for (int i = threadIdx.x; i < nc * N; i += blockDim.x) {
            const int tt = i / N, k = i % N;
            const float * r = a.bc + (size_t) (s0 + t0 + tt) * a.ldbc;
            Bs[i] = r[k]; Cs[i] = r[N + k];
        }
        __syncthreads();
        // TB tokens at a time: their decays exp(dt A) and inputs dt u B do not depend on the states, so they are formed side by side; only
        // the fused multiply-adds on the states run one after the other
        for (int tb = 0; tb < nc; tb += TB) {
            float dA[TB][NPL], dB[TB][NPL], uu[TB];
#pragma unroll
            for (int j = 0; j < TB; j++) {
                const int tt = min(tb + j, nc - 1);
                const float dt = dts[tt * CH + cl], u = us[tt * CH + cl], du = dt * u;
                const float * Bt = Bs + tt * N + part;
                uu[j] = u;
#pragma unroll
                for (int r = 0; r < NPL; r++) {
                    const bool ok = part + P * r < N;
                    dA[j][r] = 1.0f + expm1f(dt * Ar[r]);             // the decay rounded once: over a thousand steps expf's last-place errors would add up
                    dB[j][r] = ok ? du * Bt[P * r] : 0.f;
                }
            }
            float acc[TB];
#pragma unroll
            for (int j = 0; j < TB; j++) {
                const int tt = min(tb + j, nc - 1);
                const float * Ct = Cs + tt * N + part;
                acc[j] = 0.f;
                if (tb + j < nc) {
#pragma unroll
                    for (int r = 0; r < NPL; r++) {
                        s[r] = fmaf(dA[j][r], s[r], dB[j][r]);
                        if (part + P * r < N) acc[j] = fmaf(s[r], Ct[P * r], acc[j]);
                    }
                }
            }
#pragma unroll
            for (int o = 1; o < P; o <<= 1)
#pragma unroll
                for (int j = 0; j < TB; j++) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
            if (part < TB && tb + part < nc) {                 // lane j of the channel stores token j's sum
                float v = acc[0];
#pragma unroll
                for (int j = 1; j < TB; j++) if (part == j) v = acc[j];
                float uj = uu[0];
#pragma unroll
                for (int j = 1; j < TB; j++) if (part == j) uj = uu[j];
                ys[(tb + part) * CH + cl] = fmaf(Dc, uj, v);
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nc * CH; i += blockDim.x) {
            const int tt = i / CH, ch = c0 + i % CH;
            if (ch < a.inner) a.out[(size_t) (s0 + t0 + tt) * a.inner + ch] = ys[i] * sk_silu(zs[i]);
        }
    }
#pragma unroll
    for (int r = 0; r < NPL; r++) { const int k = part + P * r; if (cok && k < N) S[k] = s[r]; }
}
int pib_ssm_scan(const float * u, int ldu, const float * dtr, int lddt, const float * bc, int ldbc, const float * z, int ldz, const pib_hlayer & L, const pib_hbatch & b,
                 float * state, size_t state_stride, float * out, cudaStream_t st) {
    const int N = L.n_state;
    if (N < 1 || N > 256) { pib_set_error("state-space scan: %d states per channel (1 to 256)", N); return PIB_ERR_UNSUPP; }
    ss_args a = { u, ldu, dtr, lddt, bc, ldbc, z, ldz, L.dt_bias, L.ssm_a, L.ssm_d, L.inner, N, b.seg_start, b.seg_len, b.seg_slot, state, state_stride, L.state_off, out };
    const int P = N >= 16 ? 16 : N >= 8 ? 8 : 4, CH = SS_THREADS / P, per = (N + P - 1) / P;
    dim3 grid((unsigned) b.S, (unsigned) ((L.inner + CH - 1) / CH));
    const size_t smem = (size_t) (4 * SS_TC * CH + 2 * SS_TC * N) * 4;
#define SS_GO(P, NPL) do { if (smem > 48 * 1024) cudaFuncSetAttribute(ssm_scan_kernel<P, NPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem); \
                           pib_launch(ssm_scan_kernel<P, NPL>, dim3(grid), dim3(SS_THREADS), (size_t) smem, st, a); } while (0)
    if (P == 4)      { if (per <= 1) SS_GO(4, 1); else SS_GO(4, 2); }
    else if (P == 8) { if (per <= 1) SS_GO(8, 1); else SS_GO(8, 2); }
    else if (per <= 1) SS_GO(16, 1); else if (per <= 2) SS_GO(16, 2); else if (per <= 4) SS_GO(16, 4); else if (per <= 8) SS_GO(16, 8); else SS_GO(16, 16);
#undef SS_GO
    CKL();
    return PIB_OK;
}

// ---- two-branch mixer: what follows the projections ---------------------------------------------------------------------------------------
// proj[t] = [q (H*D) | k (G*D) | head gates (H) | q2 | k2 | v2 | gates2] before any bias.  One warp per query / key head: add the bias, keep
// the key as the VALUE of the token's cell, rotate the first rot_dims coordinates (i pairs with i + rot_dims / 2), divide by the root mean
// square over D; queries go to q[t][h], keys to the cell: [keys (G*D) | values (G*D)].  The other threads' share: silu in place on q2 | k2 | v2.
__global__ void __launch_bounds__(256) dual_prep_kernel(float * __restrict__ proj, int ldp, int H, int G, int D, int rot_dims, const float * __restrict__ bias, float eps,
                                                        int act_off, int act_n, const int32_t * __restrict__ pos, const int32_t * __restrict__ cell,
                                                        const float2 * __restrict__ rope, float * __restrict__ q, float * __restrict__ cache, int cache_row) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float sm[];                 // per warp [2][D]
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float * r = proj + (size_t) t * ldp;
    float * row = cache + (size_t) cell[t] * cache_row;
    const int half = rot_dims / 2;
    const float2 * cs = rope + (size_t) pos[t] * half;
    float * raw = sm + (size_t) warp * 2 * D, * rot = raw + D;
    for (int hh = warp; hh < H + G; hh += nw) {
        const float * src = r + (size_t) hh * D;
        const float * b = bias + (size_t) hh * D;
        for (int i = lane; i < D; i += 32) {
            const float v = src[i] + b[i];
            raw[i] = v;
            if (hh >= H) row[(size_t) G * D + (size_t) (hh - H) * D + i] = v;
        }
        __syncwarp();
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) {
            float v;
            if (i < half)          v = raw[i] * cs[i].x - raw[i + half] * cs[i].y;
            else if (i < rot_dims) v = raw[i] * cs[i - half].x + raw[i - half] * cs[i - half].y;
            else                   v = raw[i];
            rot[i] = v;
            ss = fmaf(v, v, ss);
        }
        const float inv = 1.0f / sqrtf(warp_sum(ss) / D + eps);
        float * dst = hh < H ? q + ((size_t) t * H + hh) * D : row + (size_t) (hh - H) * D;
        for (int i = lane; i < D; i += 32) dst[i] = rot[i] * inv;
        __syncwarp();
    }
    for (int i = threadIdx.x; i < act_n; i += blockDim.x) r[act_off + i] = sk_silu(r[act_off + i]);
}
int pib_dual_prep(float * proj, int ldp, const pib_hlayer & L, float eps, const pib_hbatch & b, const float2 * rope, float * q, float * cache, int cache_row, cudaStream_t st) {
    const int H = L.heads, G = L.kv_heads, D = L.dim, act_off = (H + G) * D + H, act_n = L.heads2 * (2 * L.dim2 + L.vdim2);
    const size_t smem = (size_t) 8 * 2 * D * 4;
    if (smem > 48 * 1024) cudaFuncSetAttribute(dual_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
    pib_launch(dual_prep_kernel, dim3(b.T), dim3(256), (size_t) smem, st, proj, ldp, H, G, D, L.rot_dims, (const float *) L.proj_bias, eps, act_off, act_n, b.pos, b.cell, rope, q,
               cache, cache_row);
    CKL();
    return PIB_OK;
}

// out[t] = [ sa * a[t][h][:] * sigmoid(proj[t][ga_off + h])  (H*V)  |  sb * bo[t] / rms(bo[t]) * w * sigmoid(proj[t][gb_off + :])  (H2*V2) ]
__global__ void __launch_bounds__(256) dual_gate_kernel(const float * __restrict__ a, const float * __restrict__ bo, const float * __restrict__ proj, int ldp, int ga_off, int gb_off,
                                                        int H, int V, int NB, const float * __restrict__ w, float sa, float sb, float eps, float * __restrict__ out) {
    pib_pdl_wait();
    pib_pdl_trigger();
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    const float * p = proj + t * ldp;
    float * o = out + t * ((size_t) H * V + NB);
    for (int i = threadIdx.x; i < H * V; i += blockDim.x) o[i] = sa * a[t * H * V + i] * sk_sigmoid(p[ga_off + i / V]);
    const float * br = bo + t * NB;
    float ss = 0.f;
    for (int i = threadIdx.x; i < NB; i += blockDim.x) ss = fmaf(br[i], br[i], ss);
    const float inv = sb / sqrtf(sk_block_sum(ss, red) / NB + eps);
    for (int i = threadIdx.x; i < NB; i += blockDim.x) o[(size_t) H * V + i] = br[i] * inv * w[i] * sk_sigmoid(p[gb_off + i]);
}
int pib_dual_gate(const float * a, const float * bo, const float * proj, int ldp, int ga_off, int gb_off, const pib_hlayer & L, float eps, int T, float * out, cudaStream_t st) {
    pib_launch(dual_gate_kernel, dim3(T), dim3(256), (size_t) 0, st, a, bo, proj, ldp, ga_off, gb_off, L.heads, L.vdim, L.heads2 * L.vdim2, (const float *) L.onorm, L.mix_a, L.mix_b,
               eps, out);
    CKL();
    return PIB_OK;
}
