"""The training-side ops on the GPU (csrc/backward.cu) against the reference's CPU outputs and the oracle."""
from pathlib import Path

import numpy as np
import pytest

import cases
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL_F32 = 2e-5   # fp32 kernels: sums in a different order than NumPy's


@pytest.fixture(scope="module")
def ref():
    return dict(np.load(Path(__file__).resolve().parent / "golden" / "extras_golden.npz"))


def test_layernorm_backward(backend, ref):
    c = cases.backward_ops()
    gi, gg, gb = backend.fnn.layernorm_backward(c["ln_go"], c["ln_x"], c["ln_g"])
    assert gi.shape == c["ln_x"].shape and gg.shape == (96,) and gb.shape == (96,)
    assert O.rel_l2(gi, ref["lnb_grad_input"]) < TOL_F32
    assert O.rel_l2(gg, ref["lnb_grad_gamma"]) < TOL_F32
    assert O.rel_l2(gb, ref["lnb_grad_beta"]) < TOL_F32
    # statistics handed in from the forward pass, 2-D input, many rows (several slabs in the column reduction)
    rng = np.random.default_rng(40)
    x = (rng.standard_normal((5000, 384)) * 1.5 - 0.4).astype(np.float32)
    go = rng.standard_normal((5000, 384)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(384)).astype(np.float32)
    mean, var = x.mean(-1, keepdims=True), x.var(-1, keepdims=True)
    got = backend.fnn.layernorm_backward(go, x, g, mean, var, 1e-5)
    for a, b in zip(got, O.layernorm_backward(go, x, g, mean, var, 1e-5)):
        assert O.rel_l2(a, b) < TOL_F32
    again = backend.fnn.layernorm_backward(go, x, g, mean, var, 1e-5)
    assert all(np.array_equal(a, b) for a, b in zip(got, again))      # no atomics: bit-stable
    with pytest.raises(ValueError):
        backend.fnn.layernorm_backward(go[:10], x, g)


def test_softmax_backward(backend, ref):
    c = cases.backward_ops()
    gi = backend.fnn.softmax_backward(c["sm_go"], c["sm_y"])
    assert O.rel_l2(gi, ref["smb_grad_input"]) < TOL_F32
    # along another axis
    y0 = np.ascontiguousarray(np.moveaxis(c["sm_y"], -1, 0))
    g0 = np.ascontiguousarray(np.moveaxis(c["sm_go"], -1, 0))
    assert O.rel_l2(backend.fnn.softmax_backward(g0, y0, dim=0), O.softmax_backward(g0, y0, dim=0)) < TOL_F32


def test_attention_backward(backend, ref):
    c = cases.backward_ops()
    gq, gk, gv = backend.attention.attention_backward(c["go"], c["q"], c["k"], c["v"], c["aw"], c["scale"])
    assert O.rel_l2(gq, ref["atb_grad_q"]) < TOL_F32
    assert O.rel_l2(gk, ref["atb_grad_k"]) < TOL_F32
    assert O.rel_l2(gv, ref["atb_grad_v"]) < TOL_F32
    # ragged sizes that do not fill the 32 x 32 tiles, against the oracle
    rng = np.random.default_rng(41)
    q, k, v, go = (rng.standard_normal((3, 4, 77, 24)).astype(np.float32) for _ in range(4))
    sc = np.einsum("bhqd,bhkd->bhqk", q, k) * 0.2
    e = np.exp(sc - sc.max(-1, keepdims=True))
    aw = (e / e.sum(-1, keepdims=True)).astype(np.float32)
    for a, b in zip(backend.attention.attention_backward(go, q, k, v, aw, 0.2), O.attention_backward(go, q, k, v, aw, 0.2)):
        assert O.rel_l2(a, b) < TOL_F32
    # finite differences on one entry: the analytic grad_q matches d(sum(out * go))/dq
    out = lambda qq: np.einsum("bhqk,bhkd->bhqd", _softmax(np.einsum("bhqd,bhkd->bhqk", qq, k.astype(np.float64)) * 0.2), v.astype(np.float64))  # noqa: E731
    q64 = q.astype(np.float64)
    dq = np.zeros_like(q64)
    dq[1, 2, 5, 7] = 1e-4
    num = ((out(q64 + dq) - out(q64 - dq)) * go).sum() / 2e-4
    gq2 = backend.attention.attention_backward(go, q, k, v, aw, 0.2)[0]
    assert abs(num - gq2[1, 2, 5, 7]) < 1e-3 * max(1.0, abs(num))


def _softmax(s):
    e = np.exp(s - s.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def test_adam_update(backend, ref):
    c = cases.backward_ops()
    w, m1, m2 = backend.learning.adam_update(c["w"], c["g"], c["m1"], c["m2"], c["lr"], c["beta1"], c["beta2"], c["eps"],
                                             c["beta1_t"], c["beta2_t"])
    # the kernel forms 1 - beta in fp32 like adam-update.glsl does; 1 - 0.999f is 1.3e-5 off 0.001, which shows in m2
    assert O.rel_l2(w, ref["adam_w"]) < 2e-6 and O.rel_l2(m1, ref["adam_m1"]) < 2e-6 and O.rel_l2(m2, ref["adam_m2"]) < 2e-5
    # shape is kept; beta^t = 1 switches the bias correction off as in the reference's CPU branch
    w2 = c["w"].reshape(10, 100)
    out = backend.learning.adam_update(w2, c["g"].reshape(10, 100), c["m1"].reshape(10, 100), c["m2"].reshape(10, 100), 1e-3,
                                       beta1_t=1.0, beta2_t=1.0)
    want = O.adam_update(w2, c["g"].reshape(10, 100), c["m1"].reshape(10, 100), c["m2"].reshape(10, 100), 1e-3, beta1_t=1.0, beta2_t=1.0)
    assert out[0].shape == (10, 100)
    for a, b in zip(out, want):
        assert O.rel_l2(a, b) < 2e-5
    with pytest.raises(ValueError):
        backend.learning.adam_update(c["w"], c["g"][:5], c["m1"], c["m2"], 1e-3)
