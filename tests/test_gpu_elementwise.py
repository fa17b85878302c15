"""CUDA elementwise entry points against the oracle, through the C ABI.
Mirrors tests/rmsnorm_rope.rs and tests/cuda_elementwise.rs of the reference (tolerance 1e-4 there)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,dim", [(2, 8), (1, 2048), (3, 4096), (32, 4096), (2, 4099), (1, 1)])
def test_rms_norm(nat, O, rows, dim):
    rng = np.random.default_rng(rows * 7 + dim)
    x = (rng.standard_normal((rows, dim)) * 1.7).astype(np.float32)
    w = (1 + 0.2 * rng.standard_normal(dim)).astype(np.float32)
    dx, dw, dw16, dy = nat.buf(x), nat.buf(w), nat.buf(w.astype(np.float16)), nat.buf(x.nbytes)
    assert nat.lib.m40llm_rms_norm_f32_async(nat.ctx, dx.ptr, dy.ptr, rows, dim, 1e-5) == 0
    nat.sync(1)
    np.testing.assert_allclose(dy.download(np.float32, x.shape), O.rms_norm(x, None, 1e-5), atol=1e-4, rtol=1e-5)
    assert nat.lib.m40llm_rms_norm_f32_weighted_async(nat.ctx, dx.ptr, dw.ptr, dy.ptr, rows, dim, 1e-5, 1) == 0
    nat.sync(1)
    np.testing.assert_allclose(dy.download(np.float32, x.shape), O.rms_norm(x, w, 1e-5), atol=1e-4, rtol=1e-5)
    assert nat.lib.m40llm_rms_norm_f32_weighted(nat.ctx, dx.ptr, dw16.ptr, dy.ptr, rows, dim, 1e-5, 0) == 0
    np.testing.assert_allclose(dy.download(np.float32, x.shape),
                               O.rms_norm(x, w.astype(np.float16).astype(np.float32), 1e-5), atol=1e-4, rtol=1e-5)
    assert nat.lib.m40llm_rms_norm_f32_weighted_async(nat.ctx, dx.ptr, dw.ptr, dy.ptr, rows, dim, 1e-5, 2) == -4
    assert nat.lib.m40llm_rms_norm_f32_async(nat.ctx, None, dy.ptr, rows, dim, 1e-5) == -1
    nat.free_all()


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("heads,hd,rows,past,base", [(2, 4, 1, 3, 1e4), (32, 64, 1, 2047, 1e4), (32, 128, 4, 8191, 5e5),
                                                    (16, 128, 2, 32767, 1e6)])
def test_rope(nat, O, layout, heads, hd, rows, past, base):
    rng = np.random.default_rng(heads + hd + past)
    q = rng.standard_normal((rows, heads * hd)).astype(np.float32)
    k = rng.standard_normal((rows, heads * hd)).astype(np.float32)
    dq, dk = nat.buf(q), nat.buf(k)
    assert nat.lib.m40llm_rope_f32_layout_async(nat.ctx, dq.ptr, dk.ptr, rows, heads, hd, past, base, 1.0, layout) == 0
    nat.sync(1)
    eq = O.rope(q, heads, hd, past, base, 1.0, layout).reshape(q.shape)
    ek = O.rope(k, heads, hd, past, base, 1.0, layout).reshape(k.shape)
    # positions up to 32767 put f32 sin/cos arguments at ~3e4 rad: device and host libm agree to ~1e-4 abs there
    np.testing.assert_allclose(dq.download(np.float32, q.shape), eq, atol=2e-4)
    np.testing.assert_allclose(dk.download(np.float32, k.shape), ek, atol=2e-4)
    dq.upload(q)
    assert nat.lib.m40llm_rope_f32_inplace_layout_async(nat.ctx, dq.ptr, rows, heads, hd, past, base, 1.0, layout) == 0
    nat.sync(1)
    np.testing.assert_allclose(dq.download(np.float32, q.shape), eq, atol=2e-4)
    dq.upload(q)
    dpos = nat.buf(np.array([past], dtype=np.uint32))
    assert nat.lib.m40llm_rope_f32_inplace_position_dev_layout_async(nat.ctx, dq.ptr, rows, heads, hd, dpos.ptr, base,
                                                                     1.0, layout) == 0
    nat.sync(1)
    np.testing.assert_allclose(dq.download(np.float32, q.shape), eq, atol=2e-4)
    # freq_scale 0 is the identity (the reference's attention tests rely on it)
    dq.upload(q)
    assert nat.lib.m40llm_rope_f32_inplace_layout_async(nat.ctx, dq.ptr, rows, heads, hd, past, base, 0.0, layout) == 0
    nat.sync(1)
    assert np.array_equal(dq.download(np.float32, q.shape), q)
    assert nat.lib.m40llm_rope_f32_inplace_layout_async(nat.ctx, dq.ptr, rows, heads, 5, past, base, 1.0, layout) == -2
    nat.free_all()


def test_residual_swiglu_casts(nat, O):
    rng = np.random.default_rng(3)
    for n in (1, 7, 4096, 14336 * 3 + 1):
        a = rng.standard_normal(n).astype(np.float32) * 3
        b = rng.standard_normal(n).astype(np.float32)
        da, db, do = nat.buf(a), nat.buf(b), nat.buf(a.nbytes)
        assert nat.lib.m40llm_residual_add_f32_async(nat.ctx, da.ptr, db.ptr, do.ptr, n) == 0
        nat.sync(1)
        assert np.array_equal(do.download(np.float32, n), a + b)
        assert nat.lib.m40llm_swiglu_f32(nat.ctx, da.ptr, db.ptr, do.ptr, n) == 0
        np.testing.assert_allclose(do.download(np.float32, n), O.swiglu(a, b), atol=1e-5, rtol=1e-5)
        h = a.astype(np.float16)
        dh = nat.buf(h)
        assert nat.lib.m40llm_f16_to_f32(nat.ctx, dh.ptr, do.ptr, n) == 0
        assert np.array_equal(do.download(np.float32, n), h.astype(np.float32))
        nat.free_all()
    assert nat.lib.m40llm_residual_add_f32_async(nat.ctx, None, None, None, 4) == -1


def test_q80_dequant(nat, O):
    """tests/embedding_dequant_cuda.rs: Q8_0 row dequant against the host form."""
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((3, 4096)) * 0.02).astype(np.float32)
    q = O.q80_quantize(w)
    dq, do = nat.buf(q), nat.buf(w.nbytes)
    assert nat.lib.m40llm_q80_to_f32(nat.ctx, dq.ptr, do.ptr, w.size) == 0
    assert np.array_equal(do.download(np.float32, w.size), O.q80_to_f32(q, w.size))
    nat.free_all()


def test_streams_events_graphs(nat):
    """tests/cuda_elementwise.rs: graph capture/replay of an elementwise op, stream waits, events."""
    n = 1 << 16
    a = np.arange(n, dtype=np.float32)
    b = np.ones(n, dtype=np.float32)
    da, db, do = nat.buf(a), nat.buf(b), nat.buf(a.nbytes)
    L, ctx = nat.lib, nat.ctx
    assert L.m40llm_cuda_graph_begin_capture(ctx, 1) == 0
    assert L.m40llm_residual_add_f32_async(ctx, da.ptr, db.ptr, do.ptr, n) == 0
    assert L.m40llm_residual_add_f32_async(ctx, do.ptr, db.ptr, do.ptr, n) == 0
    g = C.c_void_p()
    assert L.m40llm_cuda_graph_end_capture(ctx, 1, C.byref(g)) == 0 and g.value
    for rep in range(3):
        da.upload(a + rep)
        ms = C.c_float()
        assert L.m40llm_cuda_graph_launch_timed_sync(ctx, g, 1, C.byref(ms)) == 0
        assert ms.value >= 0
        assert np.array_equal(do.download(np.float32, n), a + rep + 2)
    assert L.m40llm_cuda_graph_launch(ctx, g, 1) == 0
    nat.sync(1)
    L.m40llm_cuda_graph_destroy(g)
    e0, e1 = C.c_void_p(), C.c_void_p()
    assert L.m40llm_cuda_event_create(ctx, C.byref(e0)) == 0 and L.m40llm_cuda_event_create(ctx, C.byref(e1)) == 0
    assert L.m40llm_cuda_event_record(ctx, e0, 1) == 0
    assert L.m40llm_residual_add_f32_async(ctx, da.ptr, db.ptr, do.ptr, n) == 0
    assert L.m40llm_stream_wait_for_stream(ctx, 0, 1) == 0
    assert L.m40llm_memcpy_d2d_async(ctx, da.ptr, do.ptr, a.nbytes, 0) == 0
    assert L.m40llm_stream_wait_for_stream(ctx, 1, 0) == 0
    assert L.m40llm_cuda_event_record(ctx, e1, 1) == 0
    ms = C.c_float()
    assert L.m40llm_cuda_event_elapsed_sync(ctx, e0, e1, C.byref(ms)) == 0 and ms.value >= 0
    assert np.array_equal(da.download(np.float32, n), do.download(np.float32, n))
    L.m40llm_cuda_event_destroy(e0)
    L.m40llm_cuda_event_destroy(e1)
    assert L.m40llm_stream_synchronize(ctx, 7) == -3
    assert L.m40llm_cuda_graph_begin_capture(ctx, 1) == 0
    assert L.m40llm_cuda_graph_cancel_capture(ctx, 1) == 0
    assert L.m40llm_validate_device_ptr(da.ptr) == 0 and L.m40llm_validate_device_ptr(None) == -1
    name = C.create_string_buffer(128)
    major, minor, dev = C.c_int(), C.c_int(), C.c_int()
    assert L.m40llm_current_device_props(name, 128, C.byref(major), C.byref(minor), C.byref(dev)) == 0
    assert major.value == 10, (name.value, major.value, minor.value)
    # out-of-scope entry points answer "unsupported", never a silent success
    assert L.m40llm_start_persistent_decode(ctx) == -100
    nat.free_all()


def test_stream_ordered_copies(nat):
    """The additive async host<->device copies are ordered with the kernels of their stream."""
    import ctypes as C
    x = np.arange(4096, dtype=np.float32)
    y = np.full(4096, 2.0, np.float32)
    out = np.zeros(4096, np.float32)
    dx, dy, do = nat.buf(x.nbytes), nat.buf(y.nbytes), nat.buf(out.nbytes)
    L = nat.lib
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    assert L.m40llm_memcpy_h2d_async(nat.ctx, dx.ptr, vp(x), x.nbytes, 1) == 0
    assert L.m40llm_memcpy_h2d_async(nat.ctx, dy.ptr, vp(y), y.nbytes, 1) == 0
    assert L.m40llm_residual_add_f32_async(nat.ctx, dx.ptr, dy.ptr, do.ptr, 4096) == 0
    assert L.m40llm_memcpy_d2h_async(nat.ctx, vp(out), do.ptr, out.nbytes, 1) == 0
    nat.sync(1)
    assert np.array_equal(out, x + 2.0)
    assert L.m40llm_memcpy_h2d_async(nat.ctx, None, vp(x), 4, 1) == -1
    assert L.m40llm_memcpy_d2h_async(nat.ctx, vp(out), do.ptr, 4, 7) == -4
    nat.free_all()
