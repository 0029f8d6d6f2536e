// dense_mma.cu -- the dense matmul on the tensor cores: Y[m][n] = sum_k bf16(X[m][k]) * W[n][k], W bfloat16 rows, fp32 accumulation.
//
// More than DT_ROWS_MAX rows (prompt portions): dense_tc_kernel, tcgen05.  A CTA owns 128 weight rows x NB tokens of one problem z:
//   warp 0       one lane streams both operands by TMA (cp.async.bulk.tensor.3d, 128-byte swizzle): the weight tile [128 n][64 k] and
//                the activation tile [NB m][64 k] of every k-step land in one stage and complete one mbarrier
//   warp 1       allocates tensor memory; one lane issues tcgen05.mma.cta_group::1.kind::f16 (bf16 x bf16 -> fp32, M 128, N NB, 4 x K 16 per
//                k-step) and commits each stage back to the producer, the last one to the epilogue
//   warps 2..5   read the accumulators (tcgen05.ld.32x32b: a lane is a weight row, a column a token) and store Y, optionally relu^2
// The activations are fp32 in the layer buffers (a producer that can write bfloat16 rows itself passes them as they are: x_bf16);
// otherwise dense_cast_kernel writes them once as bfloat16 rows (gathered through the row list
// of a grouped problem, so that every expert's tokens are neighbours) -- the TMA source.  Tails in K, N and M are zero-filled by TMA
// and masked at the store.  Tensor maps are 3-D {k, row, z}: heads of an attention layer and experts of a mixture are the z axis.
// Every mbarrier wait is bounded: a wait that runs out raises the CTA's abort flag and an error word that the host reads.
//
// Up to DT_ROWS_MAX rows (decoding) the weights are the limit (memory-bound): those calls stay with the row kernels of dense_mm.cu.
#include <cuda.h>
#include <cuda_bf16.h>

#include <map>
#include <mutex>
#include <utility>

#include "hybrid.cuh"

#define DT_BM        128
#define DT_BK        64
#define DT_THREADS   192
#define DT_SPIN      (1u << 22)
#define DT_ROWS_MAX  16

__device__ __forceinline__ uint32_t dt_smem(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void dt_mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void dt_mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
// bounded: false when the phase did not complete within DT_SPIN polls or another role gave up
__device__ __forceinline__ bool dt_mbar_wait(uint32_t bar, uint32_t parity, volatile int * abort_s) {
    for (uint32_t it = 0; it < DT_SPIN; it++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 63) == 63 && *abort_s) return false;
    }
    *abort_s = 1;
    return false;
}
__device__ __forceinline__ void dt_tma_3d(uint32_t dst, const CUtensorMap * map, uint32_t bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t dt_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t) 1 << 16;
    d |= (uint64_t) (1024 >> 4) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) 2 << 61;
    return d;
}
__device__ __forceinline__ void dt_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void dt_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- fp32 rows -> bfloat16 rows [Zs][M][Kp] (Kp = K rounded up to 8, the tail zero), gathered through xrows ---------------------------
__global__ void dense_cast_kernel(const float * __restrict__ X, int64_t ldx, int64_t xz, const int32_t * __restrict__ xrows, int xdiv, int M, int K, int Kp,
                                  __nv_bfloat16 * __restrict__ out) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int m = blockIdx.x, z = blockIdx.y;
    const float * src = X + (size_t) z * xz + (size_t) (xrows ? xrows[m] / xdiv : m) * ldx;
    __nv_bfloat16 * dst = out + ((size_t) z * M + m) * Kp;
    for (int k = threadIdx.x * 2; k < Kp; k += blockDim.x * 2) {
        const float a = k < K ? src[k] : 0.f, b = k + 1 < K ? src[k + 1] : 0.f;
        *reinterpret_cast<__nv_bfloat162 *>(dst + k) = __floats2bfloat162_rn(a, b);
    }
}

template <int NB> struct dt_cfg {
    static constexpr int STAGES  = NB <= 64 ? 4 : 3;
    static constexpr int A_BYTES = DT_BM * DT_BK * 2, B_BYTES = NB * DT_BK * 2;
    static constexpr int TM_COLS = NB < 32 ? 32 : NB;
    static constexpr size_t SMEM = (size_t) STAGES * (A_BYTES + B_BYTES) + (2 * STAGES + 1) * 8 + 32 + 1024;
};

template <int NB, int EPI>
__global__ void __launch_bounds__(DT_THREADS)
dense_tc_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap, int M, int N, int K, const int32_t * __restrict__ zrange,
                int x_has_z, float * __restrict__ Y, int64_t ldy, int64_t yz, int * __restrict__ err, float e0, float e1) {
    pib_pdl_wait();
    pib_pdl_trigger();
    const int z = blockIdx.z;
    int row0 = 0, row1 = M;
    if (zrange) { row0 = zrange[z]; row1 = zrange[z + 1]; }
    const int m0 = row0 + blockIdx.y * NB;
    if (m0 >= row1) return;                                    // the whole CTA leaves before any barrier or allocation exists
    const int n0 = blockIdx.x * DT_BM;
    using C = dt_cfg<NB>;
    extern __shared__ __align__(1024) uint8_t dt_dsm[];
    uint8_t *  sA  = dt_dsm + ((1024u - (dt_smem(dt_dsm) & 1023u)) & 1023u);
    uint8_t *  sB  = sA + C::STAGES * C::A_BYTES;
    uint64_t * bar = reinterpret_cast<uint64_t *>(sB + C::STAGES * C::B_BYTES);          // full[S], empty[S], accumulators ready
    uint32_t * tmem_slot = reinterpret_cast<uint32_t *>(bar + 2 * C::STAGES + 1);
    volatile int * abort_s = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar_f = dt_smem(bar), bar_e = bar_f + C::STAGES * 8, bar_t = bar_f + 2 * C::STAGES * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_ksteps = (K + DT_BK - 1) / DT_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { dt_mbar_init(bar_f + s * 8, 1); dt_mbar_init(bar_e + s * 8, 1); }
        dt_mbar_init(bar_t, 1);
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dt_smem(tmem_slot)), "r"((uint32_t) C::TM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kt = 0; kt < n_ksteps; kt++) {
                const int s = kt % C::STAGES;
                if (kt >= C::STAGES && !dt_mbar_wait(bar_e + s * 8, ((kt / C::STAGES) - 1) & 1, abort_s)) break;
                dt_mbar_expect_tx(bar_f + s * 8, C::A_BYTES + C::B_BYTES);
                dt_tma_3d(dt_smem(sA + s * C::A_BYTES), &wmap, bar_f + s * 8, kt * DT_BK, n0, z);
                dt_tma_3d(dt_smem(sB + s * C::B_BYTES), &xmap, bar_f + s * 8, kt * DT_BK, m0, x_has_z ? z : 0);
            }
        }
    } else if (warp == 1) {
        // instruction descriptor: fp32 accumulators, bfloat16 x bfloat16, both operands K-major, N = NB, M = 128
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (NB >> 3) << 17) | ((uint32_t) (DT_BM >> 4) << 24);
        if (lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < n_ksteps && ok; kt++) {
                const int s = kt % C::STAGES;
                ok = dt_mbar_wait(bar_f + s * 8, (kt / C::STAGES) & 1, abort_s);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ad = dt_desc(dt_smem(sA + s * C::A_BYTES)), bd = dt_desc(dt_smem(sB + s * C::B_BYTES));
#pragma unroll
                for (int k = 0; k < DT_BK / 16; k++) dt_mma(tmem_d, ad + 2 * k, bd + 2 * k, idesc, (kt | k) != 0);
                dt_commit(bar_e + s * 8);
            }
            if (ok) dt_commit(bar_t);
        }
    } else {
        const bool ok = dt_mbar_wait(bar_t, 0, abort_s);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q4 = warp & 3, orow = n0 + q4 * 32 + lane;
        float * Yz = Y + (size_t) z * yz;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < NB; c0 += 32) {
                if (m0 + c0 >= row1) break;
                uint32_t v[32];
                const uint32_t taddr = tmem_d + ((uint32_t) (q4 * 32) << 16) + (uint32_t) c0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                               "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                               "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                               "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                             : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (EPI == PIB_EPI_GLU_PAIR) {           // a pair's two weight rows sit in neighbouring lanes: the even lane writes the pair's output
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float mine = __uint_as_float(v[j]), other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        const int m = m0 + c0 + j;
                        if (!(lane & 1) && orow + 1 < N && m < row1) Yz[(size_t) m * ldy + (orow >> 1)] = pib_glu_pair<true>(mine, other, e0);
                    }
                } else if (orow < N) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int m = m0 + c0 + j;
                        if (m < row1) {
                            Yz[(size_t) m * ldy + orow] = pib_epilogue<EPI, true>(__uint_as_float(v[j]), e0, e1);
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_s) {
        // a wait ran out: say so, give copies and MMAs still in flight time to land (bounded), then free the tensor memory
        if (threadIdx.x == 0) atomicExch(err, 1 + (int) blockIdx.x);
        for (int i = 0; i < 2000; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t) C::TM_COLS) : "memory");
}

// ---- host side --------------------------------------------------------------------------------------------------------------------
typedef CUresult (*dt_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static dt_encode_fn dt_encode() {
    static dt_encode_fn fn = nullptr;
    if (!fn) {
        cudaDriverEntryPointQueryResult st;
        void * p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) == cudaSuccess && st == cudaDriverEntryPointSuccess) fn = (dt_encode_fn) p;
    }
    return fn;
}

// per (device, stream): the bfloat16 staging of the activations and the error word of the kernels' bounded waits
struct dt_scratch { __nv_bfloat16 * xs = nullptr; size_t cap = 0; int * err = nullptr; int * err_host = nullptr; };
static dt_scratch * dt_scratch_of(cudaStream_t st, size_t bytes) {
    static std::map<std::pair<int, cudaStream_t>, dt_scratch> all;
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    dt_scratch & s = all[std::make_pair(dev, st)];
    if (!s.err) {
        if (cudaMalloc(&s.err, 4) != cudaSuccess || cudaMemset(s.err, 0, 4) != cudaSuccess || cudaMallocHost(&s.err_host, 4) != cudaSuccess) { cudaGetLastError(); s.err = nullptr; return nullptr; }
        *s.err_host = 0;
    }
    if (bytes > s.cap) {
        cudaStreamSynchronize(st);
        if (s.xs) cudaFree(s.xs);
        s.cap = bytes + bytes / 2;
        if (cudaMalloc(&s.xs, s.cap) != cudaSuccess) { cudaGetLastError(); s.xs = nullptr; s.cap = 0; return nullptr; }
    }
    return &s;
}

static int dt_map3(CUtensorMap * map, const void * base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes, uint64_t s2_bytes, uint32_t box1) {
    dt_encode_fn enc = dt_encode();
    if (!enc) { pib_set_error("dense matmul: cuTensorMapEncodeTiled not available"); return PIB_ERR_UNSUPP; }
    const cuuint64_t gdim[3] = { d0, d1, d2 };
    const cuuint64_t gstr[2] = { s1_bytes, s2_bytes };
    const cuuint32_t box[3]  = { DT_BK, box1, 1 };
    const cuuint32_t estr[3] = { 1, 1, 1 };
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { pib_set_error("dense matmul: cuTensorMapEncodeTiled failed (%d)", (int) r); return PIB_ERR_UNSUPP; }
    return PIB_OK;
}

template <int NB>
static int dt_launch(const pib_mm & a, const CUtensorMap & wmap, const CUtensorMap & xmap, int x_has_z, int * err, cudaStream_t st) {
    using C = dt_cfg<NB>;
    static bool configured = false;
    if (!configured) {
        PIB_CHECK(cudaFuncSetAttribute(dense_tc_kernel<NB, PIB_EPI_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) C::SMEM));
        PIB_CHECK(cudaFuncSetAttribute(dense_tc_kernel<NB, PIB_EPI_RELU2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) C::SMEM));
        PIB_CHECK(cudaFuncSetAttribute(dense_tc_kernel<NB, PIB_EPI_XIELU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) C::SMEM));
        PIB_CHECK(cudaFuncSetAttribute(dense_tc_kernel<NB, PIB_EPI_GLU_PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) C::SMEM));
        configured = true;
    }
    dim3 grid((unsigned) ((a.N + DT_BM - 1) / DT_BM), (unsigned) ((a.M + NB - 1) / NB), (unsigned) a.Z);
    if (a.epi == PIB_EPI_RELU2)      pib_launch(dense_tc_kernel<NB, PIB_EPI_RELU2>, dim3(grid), dim3(DT_THREADS), (size_t) (C::SMEM), st, wmap, xmap, a.M, a.N, a.K, a.zrange, x_has_z, a.Y, a.ldy, a.yz, err, a.e0, a.e1);
    else if (a.epi == PIB_EPI_XIELU) pib_launch(dense_tc_kernel<NB, PIB_EPI_XIELU>, dim3(grid), dim3(DT_THREADS), (size_t) (C::SMEM), st, wmap, xmap, a.M, a.N, a.K, a.zrange, x_has_z, a.Y, a.ldy, a.yz, err, a.e0, a.e1);
    else if (a.epi == PIB_EPI_GLU_PAIR) pib_launch(dense_tc_kernel<NB, PIB_EPI_GLU_PAIR>, dim3(grid), dim3(DT_THREADS), (size_t) (C::SMEM), st, wmap, xmap, a.M, a.N, a.K, a.zrange, x_has_z, a.Y, a.ldy, a.yz, err, a.e0, a.e1);
    else                             pib_launch(dense_tc_kernel<NB, PIB_EPI_NONE>, dim3(grid), dim3(DT_THREADS), (size_t) (C::SMEM), st, wmap, xmap, a.M, a.N, a.K, a.zrange, x_has_z, a.Y, a.ldy, a.yz, err, a.e0, a.e1);
    PIB_CHECK(cudaGetLastError());
    return PIB_OK;
}

static bool dt_enabled() { static const int on = getenv("PIB_DENSE_TC") ? atoi(getenv("PIB_DENSE_TC")) : 1; return on != 0; }

int pib_dense_mm_tc(const pib_mm & a, cudaStream_t st) {
    if (!dt_enabled() || a.wtype != PIB_TYPE_BF16) return PIB_ERR_UNSUPP;
    if (a.M <= DT_ROWS_MAX) return PIB_ERR_UNSUPP;                       // few rows: the memory-bound kernels of dense_mm.cu
    // TMA wants 16-byte aligned bases and strides
    if (((uintptr_t) a.W & 15) || a.ldw % 8 || a.wz % 8 || a.K < 16) return PIB_ERR_UNSUPP;
    const int  Kp = (a.K + 7) & ~7;
    const bool grouped = a.zrange != nullptr;
    const int  Zs = grouped ? 1 : a.Z;
    if (a.x_bf16 && (grouped || a.xrows || a.ldx % 8 || ((uintptr_t) a.X & 15) || (a.Z > 1 && a.xz % 8))) return PIB_ERR_UNSUPP;
    dt_scratch * sc = dt_scratch_of(st, a.x_bf16 ? 0 : (size_t) Zs * a.M * Kp * 2 + 256);
    if (!sc || (!a.x_bf16 && !sc->xs)) return PIB_ERR_UNSUPP;
    if (!a.x_bf16) pib_launch(dense_cast_kernel, dim3(dim3((unsigned) a.M, (unsigned) Zs)), dim3(128), (size_t) (0), st, a.X, a.ldx, a.xz, a.xrows, a.xdiv < 1 ? 1 : a.xdiv, a.M, a.K, Kp, sc->xs);
    PIB_CHECK(cudaGetLastError());
    // the token tile: as wide as the rows of one problem allow (grouped problems: the average share of an expert)
    const int per = grouped ? (a.M + a.Z - 1) / a.Z : a.M;
    const int NB = per <= 32 ? 32 : per <= 64 ? 64 : 128;
    CUtensorMap wmap, xmap;
    int rc = dt_map3(&wmap, a.W, (uint64_t) a.K, (uint64_t) a.N, (uint64_t) a.Z, (uint64_t) a.ldw * 2, (uint64_t) (a.Z > 1 ? a.wz : (int64_t) a.N * a.ldw) * 2, DT_BM);
    if (rc == PIB_OK && a.x_bf16) rc = dt_map3(&xmap, a.X, (uint64_t) a.K, (uint64_t) a.M, (uint64_t) a.Z, (uint64_t) a.ldx * 2, (uint64_t) (a.Z > 1 ? a.xz : (int64_t) a.M * a.ldx) * 2, (uint32_t) NB);
    else if (rc == PIB_OK) rc = dt_map3(&xmap, sc->xs, (uint64_t) Kp, (uint64_t) a.M, (uint64_t) Zs, (uint64_t) Kp * 2, (uint64_t) a.M * Kp * 2, (uint32_t) NB);
    if (rc != PIB_OK) return rc;
    switch (NB) {
        case 32:  return dt_launch<32>(a, wmap, xmap, grouped ? 0 : 1, sc->err, st);
        case 64:  return dt_launch<64>(a, wmap, xmap, grouped ? 0 : 1, sc->err, st);
        default:  return dt_launch<128>(a, wmap, xmap, grouped ? 0 : 1, sc->err, st);
    }
}

// the error word of this stream's tensor-core matmuls.  enqueue = 1: copy it to pinned memory in stream order (no wait);
// enqueue = 0: read that copy (the caller has waited for the stream, or for an event behind the copy); 0 = no kernel gave up on a wait
int pib_dense_mm_check(cudaStream_t st, int enqueue) {
    dt_scratch * sc = dt_scratch_of(st, 0);
    if (!sc) return PIB_OK;
    if (enqueue) return cudaMemcpyAsync(sc->err_host, sc->err, 4, cudaMemcpyDeviceToHost, st) == cudaSuccess ? PIB_OK : PIB_ERR_CUDA;
    if (*sc->err_host) { pib_set_error("dense matmul: a tensor-core kernel gave up on a barrier wait (CTA %d)", *sc->err_host - 1); return PIB_ERR_CUDA; }
    return PIB_OK;
}
