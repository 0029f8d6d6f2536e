// stream_kernels.cu -- parts for layer-list models (hybrid.cuh) with several residual streams, all fp32:
//
//   hyper-connections: every token carries S streams X_s [W].  A sublayer reads u = sum_s in_s X_s through a LayerNorm with weight and
//       bias, and its output y is written back as X_t <- sum_s mix[s][t] X_s + out_t y.  One kernel does the write of the sublayer before
//       and the read + norm of the next one, so the streams cross memory once per sublayer.
//   rotation tables with YaRN-scaled frequencies
//   Mamba-2: step sizes and decays per head and token; the gate silu(z) in front of an RMS norm over equal parts of the channels
//   differential attention: biases + rotation + cache write of q | k | v rows with several maps per head; a1 - lambda a2 and the unit RMS
#include "hybrid.cuh"

#include <math.h>

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
__device__ __forceinline__ float sk_silu(float z) { return z / (1.0f + expf(-z)); }

// ---- hyper-connections ------------------------------------------------------------------------------------------------------------------
// X [T][S][W].  hc_prev (with y): [in (S) | out (S) | mix (S x S, [from][to])] of the sublayer whose output y [T][W] is still to be
// written; hc_in: the read weights of the sublayer that follows (null: every stream counts once, the model's output); h [T][W] receives
// LayerNorm(u) * w + bias (null: only the write is done).  One block per token; a thread owns its columns in all streams.
template <int MAXS>
__global__ void __launch_bounds__(MAXS <= 4 ? 1024 : 256) hyper_norm_kernel(float * __restrict__ X, int S, const float * __restrict__ y, const float * __restrict__ hc_prev,
                                                         const float * __restrict__ hc_in, const float * __restrict__ w, const float * __restrict__ bias, float eps, int W,
                                                         float * __restrict__ h) {
    pib_pdl_wait();
    pib_pdl_trigger();
    extern __shared__ float srow[];                      // u [W]
    __shared__ float red[32];
    __shared__ float cin[MAXS], cout[MAXS], cmix[MAXS * MAXS];
    if (threadIdx.x < S) {
        cin[threadIdx.x]  = hc_in ? hc_in[threadIdx.x] : 1.0f;
        cout[threadIdx.x] = y ? hc_prev[S + threadIdx.x] : 0.f;
    }
    if (y) for (int i = threadIdx.x; i < S * S; i += blockDim.x) cmix[i] = hc_prev[2 * S + i];
    __syncthreads();
    float * xr = X + (size_t) blockIdx.x * S * W;
    const float * yr = y ? y + (size_t) blockIdx.x * W : nullptr;
    float sum = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float xs[MAXS];
#pragma unroll
        for (int s = 0; s < MAXS; s++) xs[s] = s < S ? xr[(size_t) s * W + c] : 0.f;
        if (yr) {
            const float yv = yr[c];
            float xn[MAXS];
#pragma unroll
            for (int t = 0; t < MAXS; t++) {
                float a = 0.f;
                if (t < S) {
#pragma unroll
                    for (int s = 0; s < MAXS; s++) if (s < S) a = fmaf(cmix[s * S + t], xs[s], a);
                    a = fmaf(cout[t], yv, a);
                    xr[(size_t) t * W + c] = a;
                }
                xn[t] = a;
            }
#pragma unroll
            for (int s = 0; s < MAXS; s++) xs[s] = xn[s];
        }
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < MAXS; s++) if (s < S) u = fmaf(cin[s], xs[s], u);
        srow[c] = u;
        sum += u;
    }
    if (!h) return;
    const float mean = sk_block_sum(sum, red) / W;
    float q = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = srow[c] - mean; q = fmaf(d, d, q); }
    const float inv = 1.0f / sqrtf(sk_block_sum(q, red) / W + eps);
    float * hr = h + (size_t) blockIdx.x * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) hr[c] = fmaf((srow[c] - mean) * inv, w[c], bias ? bias[c] : 0.f);
}
int pib_hyper_norm(float * X, int S, const float * y, const float * hc_prev, const float * hc_in, const float * w, const float * bias, float eps, int T, int W, float * h,
                   cudaStream_t st) {
    if (S < 1 || S > 16) { pib_set_error("hyper-connections: %d streams (1 to 16)", S); return PIB_ERR_UNSUPP; }
    // a decode step has one CTA per sequence: more threads keep more of the row's loads in flight (prompts fill the GPU with 256-thread CTAs)
    const int threads = T > 32 ? 256 : W >= 2048 ? 1024 : W >= 1024 ? 512 : 256;
    if (S <= 4) pib_launch(hyper_norm_kernel<4>, dim3(T), dim3(threads), (size_t) W * 4, st, X, S, y, hc_prev, hc_in, w, bias, eps, W, h);
    else        pib_launch(hyper_norm_kernel<16>, dim3(T), dim3(256), (size_t) W * 4, st, X, S, y, hc_prev, hc_in, w, bias, eps, W, h);
    CKL();
    return PIB_OK;
}

// ---- rotation tables --------------------------------------------------------------------------------------------------------------------
// tab [n_pos][dims / 2] = {cos, sin} (p * f_i) * magnitude, every angle from its own power, in double
void pib_rope_table(std::vector<float2> & tab, int n_pos, const pib_hybrid::Rope & r) {
    const int half = r.dims / 2;
    tab.assign((size_t) n_pos * (size_t) half, make_float2(1.f, 0.f));
    if (half <= 0) return;
    std::vector<double> f((size_t) half);
    double mag = 1.0;
    for (int i = 0; i < half; i++) f[(size_t) i] = pow((double) r.base, -2.0 * i / (double) r.dims);
    if (r.factor > 0) {
        const double two_pi = 6.283185307179586476925286766559;
        auto dim_of = [&](double turns) { return r.dims * log(r.original / (two_pi * turns)) / (2.0 * log((double) r.base)); };
        const double lo = std::max(floor(dim_of(r.fast)), 0.0), hi = std::min(ceil(dim_of(r.slow)), (double) (r.dims - 1));
        for (int i = 0; i < half; i++) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
            f[(size_t) i] = f[(size_t) i] / r.factor * ramp + f[(size_t) i] * (1.0 - ramp);
        }
        mag = 0.1 * log(r.factor) + 1.0;
    }
    for (int p = 0; p < n_pos; p++)
        for (int i = 0; i < half; i++) {
            const double a = (double) p * f[(size_t) i];
            tab[(size_t) p * half + i] = make_float2((float) (cos(a) * mag), (float) (sin(a) * mag));
        }
}

// ---- Mamba-2 ------------------------------------------------------------------------------------------------------------------------------
// dg[t] = [dt (H) | decay (H) | log decay (H)]: dt = softplus(proj[t][dt_off + h] + dt_bias[h]), decay = exp(-exp(a_log[h]) dt)
__global__ void mamba2_prep_kernel(const float * __restrict__ proj, int ldp, int dt_off, int H, const float * __restrict__ dt_bias, const float * __restrict__ a_log, int T,
                                   float * __restrict__ dg) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * H) return;
    const int t = i / H, h = i % H;
    const float z = proj[(size_t) t * ldp + dt_off + h] + dt_bias[h];
    const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
    const float ld = -expf(a_log[h]) * dt;
    dg[(size_t) t * 3 * H + h] = dt;
    dg[(size_t) t * 3 * H + H + h] = expf(ld);
    dg[(size_t) t * 3 * H + 2 * H + h] = ld;
}
int pib_mamba2_prep(const float * proj, int ldp, int dt_off, const pib_hlayer & L, int T, float * dg, cudaStream_t st) {
    pib_launch(mamba2_prep_kernel, dim3((unsigned) ((T * L.heads + 255) / 256)), dim3(256), (size_t) 0, st, proj, ldp, dt_off, L.heads, (const float *) L.dt_bias,
               (const float *) L.a_log, T, dg);
    CKL();
    return PIB_OK;
}

// y [T][C] <- (y silu(z)) / sqrt(mean over the part + eps) * w, the C channels in `groups` equal parts; z rows have pitch ldz.  Grid (token, part).
__global__ void __launch_bounds__(1024) gated_group_norm_kernel(float * __restrict__ y, const float * __restrict__ z, int ldz, int C, int gs, const float * __restrict__ w, float eps) {
    pib_pdl_wait();
    pib_pdl_trigger();
    __shared__ float red[32];
    float *       yr = y + (size_t) blockIdx.x * C + (size_t) blockIdx.y * gs;
    const float * zr = z + (size_t) blockIdx.x * ldz + (size_t) blockIdx.y * gs;
    const float * wr = w + (size_t) blockIdx.y * gs;
    float s = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) { const float v = yr[i] * sk_silu(zr[i]); yr[i] = v; s = fmaf(v, v, s); }
    const float inv = 1.0f / sqrtf(sk_block_sum(s, red) / gs + eps);
    for (int i = threadIdx.x; i < gs; i += blockDim.x) yr[i] = yr[i] * inv * wr[i];
}
int pib_gated_group_norm(float * y, const float * z, int ldz, int T, int C, int groups, const float * w, float eps, cudaStream_t st) {
    if (groups < 1 || C % groups) { pib_set_error("grouped norm: %d channels in %d parts", C, groups); return PIB_ERR_ARG; }
    const int gs = C / groups, threads = T > 32 ? 256 : gs >= 2048 ? 1024 : gs >= 1024 ? 512 : 256;     // decode steps: more of a part's loads in flight
    pib_launch(gated_group_norm_kernel, dim3((unsigned) T, (unsigned) groups), dim3(threads), (size_t) 0, st, y, z, ldz, C, gs, w, eps);
    CKL();
    return PIB_OK;
}

// ---- attention with several maps per head ---------------------------------------------------------------------------------------------------
// proj[t] = [q (H * maps * D) | k (G * maps * D) | v (G * V)]; bias over all rows (null: none).  Within every D-wide chunk of q and k the
// first rot_dims coordinates turn by the token's angles.  q[t] gets the query rows, the token's cell [k | v].
__global__ void __launch_bounds__(1024) qkv_rope_kernel(const float * __restrict__ proj, int ldp, int nq, int nk, int nv, int D, int rot_dims, int pairs, const float * __restrict__ bias,
                                                       const int32_t * __restrict__ pos, const int32_t * __restrict__ cell, const float2 * __restrict__ rope,
                                                       float * __restrict__ q, float * __restrict__ cache, int cache_row) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int t = blockIdx.x, half = rot_dims / 2;
    const float *  p = proj + (size_t) t * ldp;
    const float2 * cs = rope + (size_t) pos[t] * half;
    float * row = cache + (size_t) cell[t] * cache_row;
    for (int e = threadIdx.x; e < nq + nk + nv; e += blockDim.x) {
        float v = p[e] + (bias ? bias[e] : 0.f);
        if (e < nq + nk) {
            const int i = e % D;
            if (i < rot_dims) {
                int j, pe;
                bool first;
                if (pairs == PIB_PAIR_ADJACENT) { j = i >> 1; first = !(i & 1); pe = first ? e + 1 : e - 1; }
                else                            { first = i < half; j = first ? i : i - half; pe = first ? e + half : e - half; }
                const float o = p[pe] + (bias ? bias[pe] : 0.f);
                v = first ? v * cs[j].x - o * cs[j].y : v * cs[j].x + o * cs[j].y;
            }
        }
        if (e < nq) q[(size_t) t * nq + e] = v; else row[e - nq] = v;
    }
}
int pib_qkv_rope(const float * proj, int ldp, const pib_hlayer & L, const pib_hbatch & b, const float2 * rope, float * q, float * cache, int cache_row, cudaStream_t st) {
    const int n_all = (L.heads + L.kv_heads) * L.maps * L.dim + L.kv_heads * L.vdim, threads = b.T > 32 ? 256 : n_all >= 2048 ? 1024 : n_all >= 1024 ? 512 : 256;
    pib_launch(qkv_rope_kernel, dim3(b.T), dim3(threads), (size_t) 0, st, proj, ldp, L.heads * L.maps * L.dim, L.kv_heads * L.maps * L.dim, L.kv_heads * L.vdim, L.dim, L.rot_dims,
               L.rot_pairs, (const float *) L.proj_bias, b.pos, b.cell, rope, q, cache, cache_row);
    CKL();
    return PIB_OK;
}

// a [T][H][2][V] (the two maps' outputs) -> out [T][H][V] = o / sqrt(mean(o^2) + eps) * diff_out, o = a1 - diff_lambda a2.  One warp per (token, head).
__global__ void diff_combine_kernel(const float * __restrict__ a, int n_rows, int V, float lambda, float out_scale, float eps, float * __restrict__ out) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const float * a1 = a + (size_t) row * 2 * V, * a2 = a1 + V;
    float * o = out + (size_t) row * V;
    float s = 0.f;
    for (int i = lane; i < V; i += 32) { const float d = fmaf(-lambda, a2[i], a1[i]); s = fmaf(d, d, s); }
    const float inv = out_scale / sqrtf(warp_sum(s) / V + eps);
    for (int i = lane; i < V; i += 32) o[i] = fmaf(-lambda, a2[i], a1[i]) * inv;
}
int pib_diff_combine(const float * a, const pib_hlayer & L, float eps, int T, float * out, cudaStream_t st) {
    const int n_rows = T * L.heads;
    pib_launch(diff_combine_kernel, dim3((unsigned) ((n_rows + 7) / 8)), dim3(256), (size_t) 0, st, a, n_rows, L.vdim, L.diff_lambda, L.diff_out, eps, out);
    CKL();
    return PIB_OK;
}
