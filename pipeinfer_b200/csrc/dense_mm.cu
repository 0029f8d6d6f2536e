// dense_mm.cu -- matmuls with dense (unquantised) weights: Y[m][n] = sum_k X[m][k] * W[n][k], weights bfloat16 or float32 rows.
//
// Two arithmetic modes, chosen per call:
//   * served mode: X is rounded to bfloat16 when it is staged (the operand precision of the tensor cores), W is bfloat16, every
//     product is accumulated in fp32;
//   * exact mode: W float32, X float32, fmaf chains in k order -- true 32-bit, no reduced-precision matrix mode.
// One launch covers Z independent problems (heads of an attention layer, experts of a mixture) that differ by constant
// strides; with `zrange` problem z owns a run of rows of a sorted list (tokens grouped by expert) and rows may be gathered
// through an index list.
//
// Kernels: mm_tile_kernel (any shape; 64 x 64 x 16 tiles, 4 x 4 outputs per thread), for up to MV_MAXB rows mv_rows_kernel
// (one warp per weight row, 16-byte weight loads: the weights are read once at the speed of memory), and for up to 32 float32 outputs
// over many rows mm_few_cols_kernel (a warp per row: a router's logits, where 64-wide output tiles would leave most of the machine idle).
#include "hybrid.cuh"

#include <cuda_bf16.h>

#define MM_BM 64
#define MM_BN 64
#define MM_BK 16
#define MV_MAXB 16

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float ld_w(const float * p) { return *p; }
__device__ __forceinline__ float ld_w(const __nv_bfloat16 * p) { return __bfloat162float(*p); }

struct mm_dev {
    const void * W; int64_t ldw, wz;
    const float * X; int64_t ldx, xz; const int32_t * xrows; int xdiv;
    float * Y; int64_t ldy, yz;
    int M, N, K;
    const int32_t * zrange;
    float e0, e1;
};

template <typename WT, bool ROUND, int EPI>
__global__ void __launch_bounds__(256) mm_tile_kernel(mm_dev a) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int z = blockIdx.z;
    int row0 = 0, row1 = a.M;
    if (a.zrange) { row0 = a.zrange[z]; row1 = a.zrange[z + 1]; }
    const int m0 = row0 + blockIdx.x * MM_BM;
    if (m0 >= row1) return;
    const int n0 = blockIdx.y * MM_BN;
    const WT *    W = reinterpret_cast<const WT *>(a.W) + (size_t) z * a.wz;
    const float * X = a.X + (size_t) z * a.xz;
    float *       Y = a.Y + (size_t) z * a.yz;
    __shared__ float Xs[MM_BK][MM_BM + 4];
    __shared__ float Ws[MM_BK][MM_BN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    // rows this thread stages: element (r, kk) with kk = tid % 16, r = tid / 16 + 16 * l
    int64_t xoff[4];
    bool    xok[4], wok[4];
#pragma unroll
    for (int l = 0; l < 4; l++) {
        const int r = (tid >> 4) + 16 * l;
        const int m = m0 + r;
        xok[l] = m < row1;
        const int src = xok[l] ? (a.xrows ? a.xrows[m] / a.xdiv : m) : 0;
        xoff[l] = (int64_t) src * a.ldx;
        wok[l] = n0 + r < a.N;
    }
    const int kk = tid & 15;
    for (int k0 = 0; k0 < a.K; k0 += MM_BK) {
        const bool kok = k0 + kk < a.K;
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const int r = (tid >> 4) + 16 * l;
            float xv = (xok[l] && kok) ? X[xoff[l] + k0 + kk] : 0.f;
            if (ROUND) xv = round_bf16(xv);
            Xs[kk][r] = xv;
            Ws[kk][r] = (wok[l] && kok) ? ld_w(W + (size_t) (n0 + r) * a.ldw + k0 + kk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MM_BK; k++) {
            float xa[4], wb[4];
#pragma unroll
            for (int i = 0; i < 4; i++) xa[i] = Xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wb[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(xa[i], wb[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= row1) continue;
        if (EPI == PIB_EPI_GLU_PAIR) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < a.N) Y[(size_t) m * a.ldy + (n >> 1)] = pib_glu_pair<ROUND>(acc[i][j], acc[i][j + 1], a.e0);
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            Y[(size_t) m * a.ldy + n] = pib_epilogue<EPI, ROUND>(acc[i][j], a.e0, a.e1);
        }
    }
}

// ---- few rows (decoding): one warp per weight row n, lanes stride over k in 16-byte pieces, B <= MV_MAXB rows of X at once ----
template <typename WT> struct wvec;
template <> struct wvec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16 * p, float * o) {
        const int4 r = ld_stream_v4(p);
        const uint32_t u[4] = { (uint32_t) r.x, (uint32_t) r.y, (uint32_t) r.z, (uint32_t) r.w };
#pragma unroll
        for (int i = 0; i < 4; i++) { o[2 * i] = __uint_as_float(u[i] << 16); o[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
    }
};
template <> struct wvec<float> {
    static constexpr int N = 4;
    __device__ static void load(const float * p, float * o) {
        const int4 r = ld_stream_v4(p);
        o[0] = __int_as_float(r.x); o[1] = __int_as_float(r.y); o[2] = __int_as_float(r.z); o[3] = __int_as_float(r.w);
    }
};

// the rows [row0, row1) of problem z (at most B of them) against weight row n
template <typename WT, bool ROUND, int EPI, int B>
__device__ __forceinline__ void mv_rows_body(const mm_dev & a, bool xvec, int z, int n, int lane, int row0, int row1) {
    constexpr int NR = EPI == PIB_EPI_GLU_PAIR ? 2 : 1;        // paired outputs: the warp walks the pair's two weight rows one after the other
    const float * X = a.X + (size_t) z * a.xz;
    float *       Y = a.Y + (size_t) z * a.yz;
    constexpr int V = wvec<WT>::N;
    const float * xr[B];
#pragma unroll
    for (int b = 0; b < B; b++) {
        const int m = row0 + b < row1 ? row0 + b : row0;
        xr[b] = X + (int64_t) (a.xrows ? a.xrows[m] / a.xdiv : m) * a.ldx;
    }
    float res[NR][B];
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const WT * W = reinterpret_cast<const WT *>(a.W) + (size_t) z * a.wz + (size_t) (n * NR + r) * a.ldw;
        float acc[B];
#pragma unroll
        for (int b = 0; b < B; b++) acc[b] = 0.f;
        const int Kv = a.K - a.K % V;
        // few rows: the loop is bound by the weight bytes a warp has in flight, so more trips are opened at once
#pragma unroll (B <= 2 ? 4 : 2)
        for (int k = lane * V; k < Kv; k += 32 * V) {
            float w[V];
            wvec<WT>::load(W + k, w);
#pragma unroll
            for (int b = 0; b < B; b++) {
                float xv[V];
                if (xvec) {             // rows of X start on 16-byte boundaries (checked on the host): 128-bit loads
#pragma unroll
                    for (int i = 0; i < V; i += 4) *reinterpret_cast<float4 *>(xv + i) = *reinterpret_cast<const float4 *>(xr[b] + k + i);
                } else {
#pragma unroll
                    for (int i = 0; i < V; i++) xv[i] = xr[b][k + i];
                }
#pragma unroll
                for (int i = 0; i < V; i++) acc[b] = fmaf(ROUND ? round_bf16(xv[i]) : xv[i], w[i], acc[b]);
            }
        }
        for (int k = Kv + lane; k < a.K; k += 32) {
            const float w = ld_w(W + k);
#pragma unroll
            for (int b = 0; b < B; b++) { float xv = xr[b][k]; if (ROUND) xv = round_bf16(xv); acc[b] = fmaf(xv, w, acc[b]); }
        }
#pragma unroll
        for (int b = 0; b < B; b++) res[r][b] = warp_sum(acc[b]);
    }
#pragma unroll
    for (int b = 0; b < B; b++) {
        if (lane == 0 && row0 + b < row1)
            Y[(size_t) (row0 + b) * a.ldy + n] = EPI == PIB_EPI_GLU_PAIR ? pib_glu_pair<ROUND>(res[0][b], res[NR - 1][b], a.e0) : pib_epilogue<EPI, ROUND>(res[0][b], a.e0, a.e1);
    }
}

// B = the most rows any problem can own (the batch's total).  A grouped problem (zrange) usually owns fewer -- an expert of a decode
// step has one or two of the batch's pairs -- and takes the instance that fits its own count, so that it stays bound by its weights' bytes
// and not by B times the arithmetic.  Every row's sum is formed in the same order whichever instance runs.
template <typename WT, bool ROUND, int EPI, int B>
__global__ void __launch_bounds__(256) mv_rows_kernel(mm_dev a, bool xvec) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int z = blockIdx.z;
    int row0 = 0, row1 = a.M;
    if (a.zrange) { row0 = a.zrange[z]; row1 = a.zrange[z + 1]; }
    if (row1 - row0 > B) row1 = row0 + B;            // the host only picks this kernel when every z has at most B rows
    if (row0 >= row1) return;
    const int lane = threadIdx.x & 31, n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= (EPI == PIB_EPI_GLU_PAIR ? a.N / 2 : a.N)) return;
    const int cnt = row1 - row0;
    if (B > 1 && a.zrange && cnt < B) {
        if (cnt == 1)                { mv_rows_body<WT, ROUND, EPI, 1>(a, xvec, z, n, lane, row0, row1); return; }
        if (B > 2 && cnt <= 2)       { mv_rows_body<WT, ROUND, EPI, 2>(a, xvec, z, n, lane, row0, row1); return; }
        if (B > 4 && cnt <= 4)       { mv_rows_body<WT, ROUND, EPI, (B > 4 ? 4 : B)>(a, xvec, z, n, lane, row0, row1); return; }
        if (B > 8 && cnt <= 8)       { mv_rows_body<WT, ROUND, EPI, (B > 8 ? 8 : B)>(a, xvec, z, n, lane, row0, row1); return; }
    }
    mv_rows_body<WT, ROUND, EPI, B>(a, xvec, z, n, lane, row0, row1);
}

// ---- few outputs, many rows (a router's logits over a prompt): one warp per row m, lanes stride over k, NB accumulators per lane ----
// float32 weights and activations, no rounding; the weight matrix (N x K floats) stays in L1 / L2 while every warp walks it.
template <int NB>
__global__ void __launch_bounds__(256) mm_few_cols_kernel(mm_dev a) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int lane = threadIdx.x & 31, m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (m >= a.M) return;
    const float * W = reinterpret_cast<const float *>(a.W);
    const float * x = a.X + (size_t) m * a.ldx;
    float acc[NB];
#pragma unroll
    for (int n = 0; n < NB; n++) acc[n] = 0.f;
    for (int k = lane; k < a.K; k += 32) {
        const float xv = x[k];
#pragma unroll
        for (int n = 0; n < NB; n++) if (n < a.N) acc[n] = fmaf(xv, W[(size_t) n * a.ldw + k], acc[n]);
    }
#pragma unroll
    for (int n = 0; n < NB; n++) {
        const float v = warp_sum(acc[n]);
        if (lane == 0 && n < a.N) a.Y[(size_t) m * a.ldy + n] = v;
    }
}

template <typename WT, bool ROUND, int EPI>
static int launch_mm(const pib_mm & a, const mm_dev & d, cudaStream_t st) {
    const int  V = wvec<WT>::N;
    // the row kernel wants aligned 16-byte weight loads: row stride, z stride and base all multiples of the vector
    const bool vec_ok = a.ldw % V == 0 && a.wz % V == 0 && ((uintptr_t) a.W & 15) == 0;
    // few rows in all (with zrange: no problem z can own more than the total): a warp per weight row; problems without rows leave at once
    if (a.M <= MV_MAXB && vec_ok) {
        dim3 grid((unsigned) (((EPI == PIB_EPI_GLU_PAIR ? a.N / 2 : a.N) + 7) / 8), 1, (unsigned) a.Z);
        const bool xvec = a.ldx % 4 == 0 && a.xz % 4 == 0 && ((uintptr_t) a.X & 15) == 0;
        if (a.M == 1)      pib_launch(mv_rows_kernel<WT, ROUND, EPI, 1>, dim3(grid), dim3(256), (size_t) (0), st, d, xvec);
        else if (a.M == 2) pib_launch(mv_rows_kernel<WT, ROUND, EPI, 2>, dim3(grid), dim3(256), (size_t) (0), st, d, xvec);
        else if (a.M <= 4) pib_launch(mv_rows_kernel<WT, ROUND, EPI, 4>, dim3(grid), dim3(256), (size_t) (0), st, d, xvec);
        else if (a.M <= 8) pib_launch(mv_rows_kernel<WT, ROUND, EPI, 8>, dim3(grid), dim3(256), (size_t) (0), st, d, xvec);
        else               pib_launch(mv_rows_kernel<WT, ROUND, EPI, MV_MAXB>, dim3(grid), dim3(256), (size_t) (0), st, d, xvec);
    } else {
        dim3 grid((unsigned) ((a.M + MM_BM - 1) / MM_BM), (unsigned) ((a.N + MM_BN - 1) / MM_BN), (unsigned) a.Z);
        pib_launch(mm_tile_kernel<WT, ROUND, EPI>, dim3(grid), dim3(256), (size_t) (0), st, d);
    }
    PIB_CHECK(cudaGetLastError());
    return PIB_OK;
}

int pib_dense_mm_tc(const pib_mm & a, cudaStream_t st);     // dense_mma.cu: bfloat16 tensor-core tiles; PIB_ERR_UNSUPP when the shape does not fit

int pib_dense_mm(const pib_mm & a, cudaStream_t st) {
    if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.Z <= 0) return PIB_OK;
    if (a.exact && a.wtype != PIB_TYPE_F32) { pib_set_error("dense matmul: exact mode needs float32 weights"); return PIB_ERR_ARG; }
    if (a.wtype == PIB_TYPE_BF16 && !a.exact) {
        const int rc = pib_dense_mm_tc(a, st);
        if (rc != PIB_ERR_UNSUPP) return rc;
    }
    if (a.x_bf16) { pib_set_error("dense matmul: bfloat16 activations need the tensor-core path (more than 16 rows, strides multiples of 8)"); return PIB_ERR_UNSUPP; }
    mm_dev d = { a.W, a.ldw, a.wz, a.X, a.ldx, a.xz, a.xrows, a.xdiv < 1 ? 1 : a.xdiv, a.Y, a.ldy, a.yz, a.M, a.N, a.K, a.zrange, a.e0, a.e1 };
    if (a.wtype == PIB_TYPE_F32 && a.exact && a.N <= 32 && a.M > MV_MAXB && a.Z == 1 && !a.xrows && !a.zrange && a.epi == PIB_EPI_NONE) {
        dim3 grid((unsigned) ((a.M + 7) / 8));
        if (a.N <= 8)       pib_launch(mm_few_cols_kernel<8>, dim3(grid), dim3(256), (size_t) 0, st, d);
        else if (a.N <= 16) pib_launch(mm_few_cols_kernel<16>, dim3(grid), dim3(256), (size_t) 0, st, d);
        else                pib_launch(mm_few_cols_kernel<32>, dim3(grid), dim3(256), (size_t) 0, st, d);
        PIB_CHECK(cudaGetLastError());
        return PIB_OK;
    }
    if (a.epi == PIB_EPI_GLU_PAIR && (a.N & 1)) { pib_set_error("dense matmul: paired outputs need an even number of weight rows"); return PIB_ERR_ARG; }
#define MM_GO(WT, ROUND) (a.epi == PIB_EPI_RELU2 ? launch_mm<WT, ROUND, PIB_EPI_RELU2>(a, d, st) : a.epi == PIB_EPI_XIELU ? launch_mm<WT, ROUND, PIB_EPI_XIELU>(a, d, st) : \
                          a.epi == PIB_EPI_GLU_PAIR ? launch_mm<WT, ROUND, PIB_EPI_GLU_PAIR>(a, d, st) : \
                                                    launch_mm<WT, ROUND, PIB_EPI_NONE>(a, d, st))
    if (a.wtype == PIB_TYPE_BF16) return MM_GO(__nv_bfloat16, true);
    if (a.wtype == PIB_TYPE_F32) return a.exact ? MM_GO(float, false) : MM_GO(float, true);
#undef MM_GO
    pib_set_error("dense matmul: weight type %d", a.wtype);
    return PIB_ERR_UNSUPP;
}

pib_weight * pib_dense_upload(int type, const void * host, int64_t N, int64_t K) {
    if ((type != PIB_TYPE_BF16 && type != PIB_TYPE_F32) || N <= 0 || K <= 0) { pib_set_error("dense weight: type %d, %lld x %lld", type, (long long) N, (long long) K); return nullptr; }
    pib_weight * w = (pib_weight *) calloc(1, sizeof(pib_weight));
    w->type = type; w->N = N; w->K = K;
    w->bytes = (size_t) N * K * (type == PIB_TYPE_BF16 ? 2 : 4);
    if (cudaMalloc(&w->base, w->bytes + 256) != cudaSuccess) {
        pib_set_error("dense weight: cudaMalloc of %zu bytes failed", w->bytes);
        cudaGetLastError(); free(w);
        return nullptr;
    }
    w->owns = 1;
    if (host && cudaMemcpy(w->base, host, w->bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        pib_set_error("dense weight: upload failed: %s", cudaGetErrorString(cudaGetLastError()));
        pib_weight_free(w);
        return nullptr;
    }
    return w;
}

// host-buffer convenience for the parity tests: every operand in host memory, shapes and strides as in pib_mm (elements).
// W: bfloat16 bits (wtype PIB_TYPE_BF16) or float32; zrange / xrows may be null; e0, e1: the epilogue's constants.
extern "C" int pib_dense_mm_host(int wtype, const void * W, int64_t w_elems, int64_t ldw, int64_t wz, const float * X, int64_t x_elems, int64_t ldx, int64_t xz,
                                 const int32_t * xrows, int xdiv, float * Y, int64_t y_elems, int64_t ldy, int64_t yz, int M, int N, int K, int Z,
                                 const int32_t * zrange, int epi, int exact, float e0, float e1) {
    const size_t wb = (size_t) w_elems * (wtype == PIB_TYPE_BF16 ? 2 : 4);
    void * dW = nullptr; float * dX = nullptr, * dY = nullptr; int32_t * dR = nullptr, * dZ = nullptr;
    int rc = PIB_OK;
    if (cudaMalloc(&dW, wb + 256) != cudaSuccess || cudaMalloc(&dX, (size_t) x_elems * 4 + 256) != cudaSuccess || cudaMalloc(&dY, (size_t) y_elems * 4 + 256) != cudaSuccess ||
        cudaMalloc(&dR, (size_t) M * 4 + 256) != cudaSuccess || cudaMalloc(&dZ, (size_t) (Z + 1) * 4 + 256) != cudaSuccess) rc = PIB_ERR_NOMEM;
    if (rc == PIB_OK) {
        cudaMemcpy(dW, W, wb, cudaMemcpyHostToDevice);
        cudaMemcpy(dX, X, (size_t) x_elems * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(dY, Y, (size_t) y_elems * 4, cudaMemcpyHostToDevice);
        if (xrows) cudaMemcpy(dR, xrows, (size_t) M * 4, cudaMemcpyHostToDevice);
        if (zrange) cudaMemcpy(dZ, zrange, (size_t) (Z + 1) * 4, cudaMemcpyHostToDevice);
        pib_mm a;
        a.W = dW; a.wtype = wtype; a.ldw = ldw; a.wz = wz; a.X = dX; a.ldx = ldx; a.xz = xz; a.xrows = xrows ? dR : nullptr; a.xdiv = xdiv;
        a.Y = dY; a.ldy = ldy; a.yz = yz; a.M = M; a.N = N; a.K = K; a.Z = Z; a.zrange = zrange ? dZ : nullptr; a.epi = epi; a.exact = exact; a.e0 = e0; a.e1 = e1;
        rc = pib_dense_mm(a, nullptr);
        if (rc == PIB_OK && wtype == PIB_TYPE_BF16 && !exact) { pib_dense_mm_check(nullptr, 1); }
        if (rc == PIB_OK && cudaDeviceSynchronize() != cudaSuccess) { pib_set_error("dense matmul: %s", cudaGetErrorString(cudaGetLastError())); rc = PIB_ERR_CUDA; }
        if (rc == PIB_OK && wtype == PIB_TYPE_BF16 && !exact) rc = pib_dense_mm_check(nullptr, 0);
        if (rc == PIB_OK) cudaMemcpy(Y, dY, (size_t) y_elems * 4, cudaMemcpyDeviceToHost);
    } else pib_set_error("dense matmul: out of memory for the test buffers");
    for (void * p : { dW, (void *) dX, (void *) dY, (void *) dR, (void *) dZ }) if (p) cudaFree(p);
    return rc;
}
