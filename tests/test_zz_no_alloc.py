"""The allocation-free RMSNorm backward (luaTL_rmsnorm_bwd_noalloc) against the regular entry point.

Some callers cannot call cudaMalloc at the moment they need this gradient: all device memory is
already owned by their own arena, or they cannot take the device synchronisation an allocation
implies.  The variant keeps its dgamma partials in a
fixed array inside the library instead of a workspace grown on demand.  This file sorts last so
that a run stopping at the first failure has already run every other test."""
import numpy as np
import pytest

from lanternl_b200 import _lib, luatl_adapter as ad, synth

pytestmark = pytest.mark.gpu


def dev(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return ad.pin(a.ravel(), a.shape[0], a.shape[1])


def run(entry, x, g, dy, rows, cols, accumulate_into=None):
    X, G, DY = dev(x), dev(g), dev(dy)
    DX = ad.alloc(rows, cols)
    DG = accumulate_into if accumulate_into is not None else ad.alloc(1, cols)
    _lib.call(entry, X.t.data, G.t.data, DY.t.data, DX.t.data, DG.t.data, rows, cols, 1e-5, _lib.F32)
    return DX.toflat().reshape(rows, cols), DG


@pytest.mark.parametrize("rows,cols", [(777, 512), (64, 1024), (5, 30)])
def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row(rows, cols):
    n = rows * cols
    for call in range(2):                                   # the shared array keeps the last call's contents
        x = synth.normal(100 + call, 0, n).reshape(rows, cols).astype(np.float32)
        g = (1.0 + 0.1 * synth.normal(200 + call, 0, cols)).reshape(1, cols).astype(np.float32)
        dy = synth.normal(300 + call, 0, n).reshape(rows, cols).astype(np.float32)
        dx_ref, dg_ref = run("luaTL_rmsnorm_bwd", x, g, dy, rows, cols)
        dx_new, dg_new = run("luaTL_rmsnorm_bwd_noalloc", x, g, dy, rows, cols)
        tol = 1e-5 * max(1.0, float(np.abs(dx_ref).max()))   # the tolerance of the other RMSNorm tests
        assert np.abs(dx_new - dx_ref).max() <= tol
        a, b = dg_new.toflat(), dg_ref.toflat()
        assert np.abs(a - b).max() <= 1e-5 * max(1.0, float(np.abs(b).max()))
        # dgamma accumulates across calls exactly like the regular entry point
        run("luaTL_rmsnorm_bwd", x, g, dy, rows, cols, accumulate_into=dg_ref)
        run("luaTL_rmsnorm_bwd_noalloc", x, g, dy, rows, cols, accumulate_into=dg_new)
        assert np.abs(dg_new.toflat() - dg_ref.toflat()).max() <= 2e-5 * max(1.0, float(np.abs(b).max()))


@pytest.mark.parametrize("rows,cols", [(333, 256), (4, 1030)])
def test_noalloc_against_the_analytic_gradient_in_float64(rows, cols):
    """Independent of the regular entry point: dx and dgamma of y = x * rsqrt(mean x^2 + eps) * g in float64.  The
    second shape (a row width that is no whole number of 16-byte packets per lane) takes the kernel that needs no
    scratch, so it is accepted although it is wider than the static array's limit."""
    n = rows * cols
    x = synth.normal(11, 0, n).reshape(rows, cols).astype(np.float32)
    g = (1.0 + 0.1 * synth.normal(12, 0, cols)).reshape(1, cols).astype(np.float32)
    dy = synth.normal(13, 0, n).reshape(rows, cols).astype(np.float32)
    dx, dg = run("luaTL_rmsnorm_bwd_noalloc", x, g, dy, rows, cols)
    x64, g64, dy64 = x.astype(np.float64), g.astype(np.float64), dy.astype(np.float64)
    sc = 1.0 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + 1e-5)
    dot = (dy64 * g64 * x64).sum(1, keepdims=True)
    want_dx = sc * g64 * dy64 - sc ** 3 / cols * dot * x64
    want_dg = (dy64 * x64 * sc).sum(0)
    assert np.abs(dx - want_dx).max() <= 1e-5 * max(1.0, np.abs(want_dx).max())
    assert np.abs(dg.toflat() - want_dg).max() <= 2e-5 * max(1.0, np.abs(want_dg).max())


def test_noalloc_rejects_rows_wider_than_its_static_scratch():
    rows, cols = 4, 2048
    x = np.ones((rows, cols), np.float32)
    X, DX, DG = dev(x), ad.alloc(rows, cols), ad.alloc(1, cols)
    with pytest.raises(_lib.LuaTLError, match="CAPACITY"):
        _lib.call("luaTL_rmsnorm_bwd_noalloc", X.t.data, None, X.t.data, DX.t.data, DG.t.data, rows, cols, 1e-5, _lib.F32)
    # without dgamma no scratch is needed: any width is accepted
    _lib.call("luaTL_rmsnorm_bwd_noalloc", X.t.data, None, X.t.data, DX.t.data, None, rows, cols, 1e-5, _lib.F32)
