"""GPU: the dense (bfloat16 / float32 weight) matmul of pipeinfer_b200/csrc/dense_mm.cu + dense_mma.cu against numpy: the
float32 path exactly up to summation order, the bfloat16 paths against the product of the bfloat16-rounded operands in float64.
Shapes cover the row kernel (few rows), the SIMT tiles (odd sizes) and the tcgen05 tiles (many rows), plain, one problem per
head, and grouped by expert with gathered rows and the relu^2 epilogue."""
import ctypes as C

import numpy as np
import pytest

from tests.rapisun_oracle import bf16_round

pytestmark = pytest.mark.gpu
BF16, F32 = 30, 0


def bf16_bits(a):
    return (np.asarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def mm(W, X, M, N, K, Z=1, ldw=None, wz=0, ldx=None, xz=0, ldy=None, yz=0, y_elems=None, xrows=None, xdiv=1, zrange=None, epi=0, exact=False, f32=False, e0=0.0, e1=0.0):
    from pipeinfer_b200 import load
    lib = load()
    lib.init(0)
    L = lib.L
    L.pib_dense_mm_host.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int,
                                    C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float]
    Wd = np.ascontiguousarray(W, np.float32) if f32 else np.ascontiguousarray(bf16_bits(W))
    Xd = np.ascontiguousarray(X, np.float32)
    ldw, ldx, ldy = ldw or K, ldx or K, ldy or N
    Y = np.full(y_elems or M * ldy, np.nan, np.float32)
    r = np.ascontiguousarray(xrows, np.int32) if xrows is not None else None
    zr = np.ascontiguousarray(zrange, np.int32) if zrange is not None else None
    rc = L.pib_dense_mm_host(F32 if f32 else BF16, Wd.ctypes.data, Wd.size, ldw, wz, Xd.ctypes.data, Xd.size, ldx, xz,
                             r.ctypes.data if r is not None else None, xdiv, Y.ctypes.data, Y.size, ldy, yz, M, N, K, Z,
                             zr.ctypes.data if zr is not None else None, epi, 1 if exact else 0, e0, e1)
    assert rc == 0, L.pib_last_error().decode()
    return Y


@pytest.mark.parametrize("M,N,K", [(1, 450, 200), (3, 130, 72), (8, 257, 1024), (9, 64, 40), (16, 200, 104), (17, 392, 184), (100, 130, 200),
                                   (300, 1000, 520), (1100, 456, 200), (64, 104, 64), (33, 128, 24)])
def test_plain(M, N, K):
    rng = np.random.default_rng(M * 7 + N)
    W = bf16_round(rng.standard_normal((N, K)))
    X = rng.standard_normal((M, K))
    ref = bf16_round(X) @ W.T
    got = mm(W, X, M, N, K).reshape(M, N)
    np.testing.assert_allclose(got, ref, rtol=0, atol=2e-4 * np.sqrt(K))
    ref32 = X.astype(np.float32).astype(np.float64) @ W.T
    got32 = mm(W, X, M, N, K, exact=True, f32=True).reshape(M, N)
    np.testing.assert_allclose(got32, ref32, rtol=1e-5, atol=3e-6 * np.sqrt(K))


@pytest.mark.parametrize("M,F,K", [(1, 225, 200), (2, 65, 72), (7, 128, 1024), (16, 100, 104), (17, 196, 184), (100, 65, 200), (300, 500, 520), (1100, 228, 200)])
def test_paired_gated_epilogue(M, F, K):
    """weight rows interleaved (gate i, linear part i): output i = a sigmoid(1.702 a) (b + 1), a = min(g, limit), b = clamp(u, -limit, limit) -- in the row
    kernel (a warp walks both rows of a pair), the SIMT tiles and the tcgen05 tiles (a pair sits in neighbouring lanes)"""
    rng = np.random.default_rng(M * 5 + F)
    Wg, Wu = bf16_round(rng.standard_normal((F, K))), bf16_round(rng.standard_normal((F, K)))
    W = np.stack([Wg, Wu], 1).reshape(2 * F, K)
    X = rng.standard_normal((M, K)) * 0.2
    limit = 1.5

    def ref_of(x):
        g, u = np.minimum(x @ Wg.T, limit), np.clip(x @ Wu.T, -limit, limit)
        return g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)
    got = mm(W, X, M, 2 * F, K, ldy=F, epi=3, e0=limit).reshape(M, F)
    np.testing.assert_allclose(got, ref_of(bf16_round(X)), rtol=0, atol=1e-3 * np.sqrt(K))
    got32 = mm(W, X, M, 2 * F, K, ldy=F, epi=3, e0=limit, exact=True, f32=True).reshape(M, F)
    np.testing.assert_allclose(got32, ref_of(X.astype(np.float32).astype(np.float64)), rtol=1e-5, atol=3e-6 * np.sqrt(K))


@pytest.mark.parametrize("T,H,D,R", [(5, 3, 24, 56), (40, 6, 72, 104), (200, 4, 128, 256), (130, 2, 16, 40)])
def test_one_problem_per_head(T, H, D, R):
    """Y[t][h][r] = sum_d X[t][h][d] * W[h][r][d], X rows carry other columns between the heads' parts (the rotated query part)"""
    rng = np.random.default_rng(T + H)
    pad = 8
    W = bf16_round(rng.standard_normal((H, R, D)))
    X = rng.standard_normal((T, H, D + pad))
    ref = np.einsum("thd,hrd->thr", bf16_round(X[:, :, :D]), W)
    got = mm(W, X, T, R, D, Z=H, ldw=D, wz=R * D, ldx=H * (D + pad), xz=D + pad, ldy=H * R, yz=R, y_elems=T * H * R).reshape(T, H, R)
    np.testing.assert_allclose(got, ref, rtol=0, atol=2e-4 * np.sqrt(D))


@pytest.mark.parametrize("T,E,top,K,N", [(4, 6, 3, 88, 40), (70, 5, 2, 64, 24), (400, 12, 2, 200, 88), (300, 3, 3, 128, 130)])
def test_grouped_by_expert_with_gather(T, E, top, K, N):
    rng = np.random.default_rng(T + E)
    W = bf16_round(rng.standard_normal((E, N, K)))
    X = rng.standard_normal((T, K))
    ids = np.stack([rng.permutation(E)[:top] for _ in range(T)]).reshape(-1)
    perm = np.argsort(ids, kind="stable").astype(np.int32)
    offs = np.concatenate([[0], np.cumsum(np.bincount(ids, minlength=E))]).astype(np.int32)
    ref = np.zeros((T * top, N))
    for i, p in enumerate(perm):
        v = bf16_round(X[p // top]) @ W[ids[p]].T
        ref[i] = np.maximum(v, 0) ** 2
    got = mm(W, X, T * top, N, K, Z=E, ldw=K, wz=N * K, xrows=perm, xdiv=top, zrange=offs, epi=1).reshape(T * top, N)
    np.testing.assert_allclose(got, ref, rtol=2e-5, atol=1e-3 * np.sqrt(K))
