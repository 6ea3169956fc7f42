"""Parity of the HBM-bound row kernels with the reference's CPU outputs."""
import numpy as np
import pytest

import cases
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-6  # fp32 kernels: differences are rounding only


def test_against_reference_outputs(backend, golden):
    r = cases.rowops()
    f = backend.fnn
    assert O.rel_l2(f.layernorm(r["ln_x"], r["ln_g"], r["ln_b"], 1e-5), golden["ln_y"]) < TOL
    assert O.rel_l2(f.layernorm(r["ln_x"]), golden["ln_y_default"]) < TOL
    assert O.rel_l2(f.layernorm(r["ln_x"], r["ln_g"], r["ln_b"], 1e-12), golden["ln_y_eps12"]) < TOL
    assert O.rel_l2(f.rmsnorm(r["ln_x"], r["ln_g"], 1e-5), golden["rms_y"]) < TOL
    assert O.rel_l2(f.activation_softmax(r["sm_x"]), golden["sm_y"]) < TOL
    assert O.rel_l2(f.activation_gelu(r["act_x"]), golden["act_gelu"]) < TOL
    assert O.rel_l2(f.activation_silu(r["act_x"]), golden["act_silu"]) < TOL
    assert np.array_equal(f.activation_relu(r["act_x"]), golden["act_relu"])
    assert O.rel_l2(f.activation_swiglu(r["act_x"]), golden["act_swiglu"]) < TOL
    assert np.array_equal(f.residual(r["act_x"], r["act_x"][::-1].copy()), golden["residual"])
    assert np.array_equal(f.activation_softmax(r["sm_x"]).argmax(-1), golden["sm_y"].argmax(-1))


@pytest.mark.parametrize("rows,F", [(1, 4), (3, 7), (1000, 384), (77, 1024), (5, 2048), (9, 5000)])
def test_norm_shapes(backend, rows, F):
    rng = np.random.default_rng(F)
    x = (rng.standard_normal((rows, F)) * 3 + 2).astype(np.float32)
    g, b = rng.standard_normal(F).astype(np.float32), rng.standard_normal(F).astype(np.float32)
    assert O.rel_l2(backend.fnn.layernorm(x, g, b), O.layernorm(x, g, b)) < TOL
    assert O.rel_l2(backend.fnn.rmsnorm(x, g), O.rmsnorm(x, g)) < TOL
    res = rng.standard_normal((rows, F)).astype(np.float32)
    assert O.rel_l2(backend.fnn.residual_layernorm(x, res, g, b), O.layernorm(x + res, g, b)) < TOL


def test_softmax_other_axis_and_known_answers(backend):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((4, 9, 6)).astype(np.float32)
    assert O.rel_l2(backend.fnn.activation_softmax(x, axis=1), np.moveaxis(O.softmax(np.moveaxis(x, 1, -1)), -1, 1)) < TOL
    # the reference's assertions (tests/test_gpu_operations.py:100-130)
    v = np.array([-2.0, -0.5, 0.0, 0.5, 2.0], np.float32)
    assert np.array_equal(backend.fnn.activation_relu(v), np.maximum(v, 0))
    g = backend.fnn.activation_gelu(np.array([0.0, 1.0], np.float32))
    assert g[0] == 0.0 and g[1] > 0.0
    y = backend.fnn.layernorm(rng.standard_normal((8, 64)).astype(np.float32) * 5 + 3)
    assert np.abs(y.mean(-1)).max() < 1e-5 and np.abs(y.std(-1) - 1).max() < 1e-3


def test_embedding_lookup_and_pool(backend):
    rng = np.random.default_rng(2)
    table = rng.standard_normal((1000, 384)).astype(np.float32)
    ids = rng.integers(0, 1000, size=(4, 19))
    ids[0, 0], ids[1, 5] = 1000, -3  # out of range -> zero rows
    out = backend.learning.embedding_lookup(ids, table)
    assert np.array_equal(out, O.embedding_lookup(ids, table))
    assert np.array_equal(backend.embedding_lookup(ids[0], table), O.embedding_lookup(ids[0], table))
    x = rng.standard_normal((4, 19, 384)).astype(np.float32)
    mask = (rng.random((4, 19)) > 0.3).astype(np.float32)
    mask[2] = 0
    assert O.rel_l2(backend.pooling.mean_pool(x, mask), O.mean_pool(x, mask)) < TOL
    assert O.rel_l2(backend.pooling.mean_pool(x), O.mean_pool(x)) < TOL
    pn = backend.pooling.mean_pool_normalize(x, mask)
    assert O.rel_l2(pn, O.embedding_normalize(O.mean_pool(x, mask))) < TOL
    assert np.array_equal(pn[2], np.zeros(384, np.float32))
    # feature counts on the other pooling kernels: eight 16-byte pieces per lane (768) and the scalar form (770)
    for feat in (768, 770):
        xf = rng.standard_normal((3, 37, feat)).astype(np.float32)
        mf = (rng.random((3, 37)) > 0.4).astype(np.float32)
        assert O.rel_l2(backend.pooling.mean_pool(xf, mf), O.mean_pool(xf, mf)) < TOL
        assert O.rel_l2(backend.pooling.mean_pool_normalize(xf, mf), O.embedding_normalize(O.mean_pool(xf, mf))) < TOL


def test_device_resident_chain(backend):
    """DeviceTensor in -> DeviceTensor out: LayerNorm -> linear+GELU -> linear+residual stays on the GPU."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((256, 384)).astype(np.float32)
    w1 = (rng.standard_normal((1536, 384)) * 0.05).astype(np.float32)
    w2 = (rng.standard_normal((384, 1536)) * 0.05).astype(np.float32)
    xd = backend.to_device(x, mma_operand=False)
    h = backend.fnn.layernorm(xd)
    h = backend.fnn.fused_linear_gelu(h, w1)
    y = backend.fnn.linear(h, w2)
    from grilly_b200 import DeviceTensor

    assert isinstance(y, DeviceTensor)
    ref = O.linear(O.fused_linear_gelu(O.layernorm(x), w1), w2)
    assert O.rel_l2(y.numpy(), ref) < 2e-3


def test_bounded_wait_reports_timeout_and_context_survives(backend):
    """Failure detection without a GPU fault: a device-side wait on a flag nothing sets gives up after its budget,
    the host reads GRILLY_ERR_TIMEOUT, and the same context then computes correctly."""
    from grilly_b200 import _lib as L

    dev = backend.device
    dev.sync()
    dev.check(dev.lib.grilly_selftest_wait_timeout(dev.ctx, 50))
    with pytest.raises(L.GrillyError) as ei:
        dev.sync()
    assert ei.value.code == L.ERR_TIMEOUT
    dev.sync()  # the status word was cleared: no second report
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    assert np.array_equal(backend.fnn.activation_relu(x - 5), np.maximum(x - 5, 0))


def test_gcu_and_roswish(backend):
    """activation_gcu / activation_roswish and their fused-linear forms (backend/fnn.py:385-497, 2307-2463)."""
    rng = np.random.default_rng(60)
    x = (rng.standard_normal((7, 50)) * 3).astype(np.float32)
    assert O.rel_l2(backend.fnn.activation_gcu(x), O.gcu(x)) < 2e-6
    assert O.rel_l2(backend.fnn.activation_roswish(x, alpha=0.7, beta=1.3), O.roswish(x, 0.7, 1.3)) < 2e-6
    xs = rng.standard_normal((3, 40, 96)).astype(np.float32)
    w, b = (rng.standard_normal((64, 96)) / 10).astype(np.float32), rng.standard_normal(64).astype(np.float32)
    y = backend.fnn.fused_linear_gcu(xs, w, b)
    assert y.shape == (3, 40, 64) and O.rel_l2(y, O.gcu(O.linear(xs, w, b))) < 2e-3
    assert O.rel_l2(backend.fnn.fused_linear_roswish(xs, w, b, alpha=0.5, beta=2.0), O.roswish(O.linear(xs, w, b), 0.5, 2.0)) < 2e-3
