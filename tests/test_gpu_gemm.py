"""GEMV/GEMM entry points against the oracle (tests/gemm_mixed.rs, gemm_f16xf16_f32.rs, proj_wrappers.rs,
mlp_wrappers.rs of the reference use 1e-3 absolute; here |a-e| <= 1e-3 + 2e-3|e|)."""
import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu

SHAPES = [(1, 10, 37), (3, 17, 64), (1, 256, 2048), (1, 2048, 2048), (2, 1024, 4096), (1, 4096, 4096),
          (5, 520, 1032), (8, 4096, 4096), (1, 2048, 5632),
          # batched rows: the tcgen05 path (M padded to 16..256, K tails, N tails, K splits)
          (16, 128, 64), (17, 300, 200), (32, 4096, 4096), (33, 1000, 2048), (64, 1024, 512), (65, 256, 1024),
          (100, 384, 520), (128, 2048, 2048), (256, 256, 4096), (32, 4096, 14336), (4, 24, 4096)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_f32xf16_gguf(nat, O, M, N, K):
    rng = np.random.default_rng(M * 31 + N + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    da, dw, dc = nat.buf(a), nat.buf(w), nat.buf(M * N * 4)
    assert nat.lib.m40llm_gemm_f32xf16_gguf_f32(nat.ctx, da.ptr, dw.ptr, dc.ptr, M, N, K) == 0
    exp = O.gemm_f32xf16_gguf(a, w)
    assert_close(dc.download(np.float32, (M, N)), exp, what=f"gguf {M}x{N}x{K}")
    for kind in (0, 1):
        dc.upload(np.zeros(M * N, np.float32))
        assert nat.lib.m40llm_gemm_f32xf16_gguf_f32_async(nat.ctx, da.ptr, dw.ptr, dc.ptr, M, N, K, kind) == 0
        nat.sync(kind)
        assert_close(dc.download(np.float32, (M, N)), exp, what=f"gguf async kind {kind}")
    nat.free_all()


@pytest.mark.parametrize("M,N,K", [(1, 10, 37), (2, 64, 48), (1, 2048, 2048), (3, 1024, 4096), (1, 4096, 4096), (6, 136, 1000)])
def test_gemm_rowmajor_forms(nat, O, M, N, K):
    rng = np.random.default_rng(M + N * 3 + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    a16 = a.astype(np.float16)
    b = (rng.standard_normal((K, N)) * 0.05).astype(np.float16)
    da, da16, db, dc = nat.buf(a), nat.buf(a16), nat.buf(b), nat.buf(M * N * 4)
    assert nat.lib.m40llm_gemm_f16xf16_f32(nat.ctx, da16.ptr, db.ptr, dc.ptr, M, N, K) == 0
    assert_close(dc.download(np.float32, (M, N)), O.gemm_f16xf16_rowmajor(a16, b), what="f16xf16")
    assert nat.lib.m40llm_gemm_f32xf16_f32(nat.ctx, da.ptr, db.ptr, dc.ptr, M, N, K) == 0
    assert_close(dc.download(np.float32, (M, N)), O.gemm_f32xf16_rowmajor(a, b), what="f32xf16")
    dc16 = nat.buf(M * N * 2)
    assert nat.lib.m40llm_gemm_f16_storage_f32_compute(nat.ctx, da16.ptr, db.ptr, dc16.ptr, M, N, K) == 0
    got = dc16.download(np.float16, (M, N)).astype(np.float32)
    assert_close(got, O.gemm_f16_storage(a16, b).astype(np.float32), atol=2e-3, what="f16 storage")
    nat.free_all()


def test_materialize_and_f32_gemm(nat, O):
    """The reference's default decode projection: expand GGUF f16 to f32 [K][N], then SGEMM (src/infer/gemm.rs:287-362)."""
    rng = np.random.default_rng(8)
    M, N, K = 2, 200, 333
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    da, dw, dbt, dc = nat.buf(a), nat.buf(w), nat.buf(N * K * 4), nat.buf(M * N * 4)
    assert nat.lib.m40llm_materialize_gguf_f16_to_f32_colmajor_nt(nat.ctx, dw.ptr, dbt.ptr, N, K) == 0
    assert np.array_equal(dbt.download(np.float32, (K, N)), w.astype(np.float32).T)
    assert nat.lib.m40llm_gemm_f32xf32_f32(nat.ctx, da.ptr, dbt.ptr, dc.ptr, M, N, K) == 0
    assert_close(dc.download(np.float32, (M, N)), O.gemm_f32xf16_gguf(a, w), what="f32xf32")
    assert nat.lib.m40llm_gemm_f32xf32_f32_async(nat.ctx, da.ptr, dbt.ptr, dc.ptr, 0, N, K) == -2
    nat.free_all()


@pytest.mark.parametrize("M,N,K", [(1, 8, 32), (1, 64, 128), (1, 4096, 4096), (3, 1000, 1024), (1, 4096, 14336), (8, 512, 4096),
                                   # batched rows: the tcgen05 Q8_0 path (K % 256 == 0), incl. N tails, row chunks of 64
                                   (2, 128, 256), (16, 8, 256), (17, 300, 512), (32, 4096, 4096), (32, 4096, 14336), (64, 256, 1024),
                                   (65, 128, 256), (100, 520, 768), (32, 14336, 4096), (5, 200, 384),
                                   # 2-4 chained 64-row passes sharing one arena (the batch sweep's 128 and 256 rows)
                                   (128, 4096, 4096), (256, 512, 1024), (129, 256, 512), (256, 4096, 14336)])
def test_gemm_q80(nat, O, M, N, K):
    rng = np.random.default_rng(M + N + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    wq = O.q80_quantize((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    da, dw, dc = nat.buf(a), nat.buf(wq), nat.buf(M * N * 4)
    assert nat.lib.m40llm_gemm_f32xq80_gguf_f32_async(nat.ctx, da.ptr, dw.ptr, dc.ptr, M, N, K, 0) == 0
    nat.sync(0)
    assert_close(dc.download(np.float32, (M, N)), O.gemm_f32xq80_gguf(a, wq, N), what=f"q80 {M}x{N}x{K}")
    assert nat.lib.m40llm_gemm_f32xq80_gguf_f32_async(nat.ctx, da.ptr, dw.ptr, dc.ptr, M, N, 33, 0) == -2
    nat.free_all()


@pytest.mark.parametrize("rows,H,F,q80", [(1, 256, 384, True), (1, 4096, 14336, True), (4, 1024, 2816, True),
                                           (32, 4096, 14336, True), (8, 256, 512, True), (70, 512, 1024, True), (32, 2048, 5632, False),
                                           (128, 1024, 2816, True), (256, 512, 1024, True), (65, 512, 1024, True),
                                           (128, 4096, 14336, True), (256, 2048, 5632, False),
                                           (1, 2048, 5632, False), (3, 512, 1024, False)])
def test_ffn_swiglu(nat, O, rows, H, F, q80):
    """hid = silu(x.Wg) * (x.Wu); out = residual + hid.Wd  (src/infer/gemm.rs:91-163 + kernels.cu:880-891)."""
    rng = np.random.default_rng(rows + H + F)
    x = rng.standard_normal((rows, H)).astype(np.float32)
    res = rng.standard_normal((rows, H)).astype(np.float32)
    wg = (rng.standard_normal((F, H)) * 0.02).astype(np.float32)
    wu = (rng.standard_normal((F, H)) * 0.02).astype(np.float32)
    wd = (rng.standard_normal((H, F)) * 0.02).astype(np.float32)
    if q80:
        wg, wu, wd = O.q80_quantize(wg), O.q80_quantize(wu), O.q80_quantize(wd)
        hid = O.swiglu(O.gemm_f32xq80_gguf(x, wg, F), O.gemm_f32xq80_gguf(x, wu, F))
        exp = res + O.gemm_f32xq80_gguf(hid, wd, H)
        fn = nat.lib.m40llm_ffn_swiglu_q80_f32_async
    else:
        wg, wu, wd = wg.astype(np.float16), wu.astype(np.float16), wd.astype(np.float16)
        hid = O.swiglu(O.gemm_f32xf16_gguf(x, wg), O.gemm_f32xf16_gguf(x, wu))
        exp = res + O.gemm_f32xf16_gguf(hid, wd)
        fn = nat.lib.m40llm_ffn_swiglu_f16_f32_async
    dx, dr, dg, du, dd = nat.buf(x), nat.buf(res), nat.buf(wg), nat.buf(wu), nat.buf(wd)
    dh, do = nat.buf(rows * F * 4), nat.buf(rows * H * 4)
    assert fn(nat.ctx, dx.ptr, dg.ptr, du.ptr, dd.ptr, dr.ptr, dh.ptr, do.ptr, rows, H, F, 0) == 0
    nat.sync(0)
    assert_close(dh.download(np.float32, (rows, F)), hid, what="hid")
    assert_close(do.download(np.float32, (rows, H)), exp, what="ffn out")
    assert fn(nat.ctx, dx.ptr, dg.ptr, du.ptr, dd.ptr, None, dh.ptr, do.ptr, rows, H, F, 1) == 0
    nat.sync(1)
    assert_close(do.download(np.float32, (rows, H)), exp - res, what="ffn out, no residual")
    nat.free_all()


@pytest.mark.parametrize("fmt,N,K", [
    ("f16", 6144, 4096),    # groups % CTAs != 0: the tail of the matrix is cut into groups one row smaller
    ("f16", 1001, 2048),    # odd row count, fewer groups than whole deals
    ("f16", 32000, 2048),   # lm_head shape
    ("f16", 595, 512),      # barely more groups than CTAs
    ("q80", 1024, 28672),   # K > 16384: activation digits made in two rounds, ring slots over a 90 KB digit area
    ("q80", 599, 512),
    ("q80", 11008, 4096),
    ("q80", 5632, 2048),
    ("q80", 2048, 5632),
])
def test_one_row_streaming_shapes(nat, O, fmt, N, K):
    """One activation row through the weight-streaming kernel at shapes that exercise its stage bookkeeping
    (equal stage counts per CTA, late ring slots, multi-round activation preparation)."""
    rng = np.random.default_rng(N * 7 + K)
    a = rng.standard_normal((1, K)).astype(np.float32)
    a[0, ::97] *= 30.0  # wide dynamic range inside 32-blocks
    a[0, 64:96] = 0.0   # an all-zero block
    dc = nat.buf(N * 4)
    da = nat.buf(a)
    if fmt == "f16":
        w = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
        dw = nat.buf(w)
        assert nat.lib.m40llm_gemm_f32xf16_gguf_f32_async(nat.ctx, da.ptr, dw.ptr, dc.ptr, 1, N, K, 1) == 0
        exp = O.gemm_f32xf16_gguf(a, w)
    else:
        wq = O.q80_quantize((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
        dw = nat.buf(wq)
        assert nat.lib.m40llm_gemm_f32xq80_gguf_f32_async(nat.ctx, da.ptr, dw.ptr, dc.ptr, 1, N, K, 1) == 0
        exp = O.gemm_f32xq80_gguf(a, wq, N)
    nat.sync(1)
    assert_close(dc.download(np.float32, (1, N)), exp, what=f"one row {fmt} {N}x{K}")
    st = np.zeros(1, np.uint32)
    assert nat.lib.m40llm_context_take_device_status(nat.ctx, st.ctypes.data) == 0 and st[0] == 0
    nat.free_all()
