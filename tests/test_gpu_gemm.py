"""Parity of the tcgen05 GEMM family with the reference's CPU implementation (oracle + golden vectors),
called through the C ABI. Tolerances: rel-L2 <= 2e-3 in tf32 mode, <= 1e-2 in bf16 mode; argmax identical."""
import numpy as np
import pytest

import cases
from conftest import TOL_BF16, TOL_TF32, index_mismatches
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_linear_config0_against_reference_outputs(backend, golden):
    c = cases.linear_cfg0()
    y = backend.fnn.linear(c["x"], c["w"], c["b"])
    assert y.dtype == np.float32 and y.shape == (32, 1536)
    assert O.rel_l2(y, golden["lin_y"]) < TOL_TF32
    assert index_mismatches(y, golden["lin_y"], 1, TOL_TF32)[1] == 0
    for name, fn in (("gelu", backend.fnn.fused_linear_gelu), ("silu", backend.fnn.fused_linear_silu),
                     ("relu", backend.fnn.fused_linear_relu)):
        out = fn(c["x"][:8], c["w"], c["b"])
        ref = golden[f"lin_{name}_y8"]
        assert O.rel_l2(out, ref) < TOL_TF32, name
        assert index_mismatches(out, ref, 1, TOL_TF32)[1] == 0, name
    # 3-D input, ragged sizes (K = 50 is padded to 52 at the boundary), with and without bias
    assert O.rel_l2(backend.fnn.linear(c["x3"], c["w3"], c["b3"]), golden["lin3_y"]) < TOL_TF32
    y3 = backend.fnn.linear(c["x3"], c["w3"])
    assert y3.shape == (3, 5, 21) and O.rel_l2(y3, golden["lin3_nobias_y"]) < TOL_TF32


def test_linear_config0_batch_4096(backend):
    c = cases.linear_cfg0()
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4096, 384)).astype(np.float32)
    y = backend.fnn.fused_linear_gelu(x, c["w"], c["b"])
    ref = O.fused_linear_gelu(x, c["w"], c["b"])
    assert O.rel_l2(y, ref) < TOL_TF32
    # default tf32 mode: argmax and top-5 may differ from the fp64 oracle only where the oracle's own values are
    # closer together than the tf32 tolerance (no tf32 implementation can order those); the count is reported
    for k in (1, 5):
        differ, real = index_mismatches(y, ref, k, TOL_TF32)
        print(f"tf32 linear+GELU 4096 rows: top-{k} differs in {differ} of 4096 rows, {real} of them not near-ties")
        assert real == 0
        assert differ < 4096 * 0.02


def test_exact_indices_in_tf32x3_mode(backend_x3, golden):
    """precision='tf32x3' (tf32 hi/lo split products, fp32-level results): argmax and top-5 indices of config 0 at
    32 and at 4096 rows are IDENTICAL to the reference's, and the values agree to fp32 accuracy."""
    c = cases.linear_cfg0()
    y = backend_x3.fnn.linear(c["x"], c["w"], c["b"])
    assert O.rel_l2(y, golden["lin_y"]) < 1e-5
    assert np.array_equal(y.argmax(-1), golden["lin_y"].argmax(-1))
    assert np.array_equal(np.argsort(-y, -1, kind="stable")[:, :5], np.argsort(-golden["lin_y"], -1, kind="stable")[:, :5])
    yg = backend_x3.fnn.fused_linear_gelu(c["x"], c["w"], c["b"])
    refg = O.fused_linear_gelu(c["x"], c["w"], c["b"])
    assert O.rel_l2(yg, refg) < 2e-4          # one tanh.approx in the epilogue: 5e-4 absolute in tanh at most
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4096, 384)).astype(np.float32)
    y = backend_x3.fnn.linear(x, c["w"], c["b"])
    ref = O.linear(x, c["w"], c["b"])
    assert O.rel_l2(y, ref) < 1e-5
    assert np.array_equal(y.argmax(-1), ref.argmax(-1))
    assert np.array_equal(np.argsort(-y, -1, kind="stable")[:, :5], np.argsort(-ref, -1, kind="stable")[:, :5])
    # a per-call override on a tf32 backend does the same, and gemm has the mode too
    a, b = rng.standard_normal((300, 200)).astype(np.float32), rng.standard_normal((200, 260)).astype(np.float32)
    cg = backend_x3.fnn.gemm(a, b)
    assert O.rel_l2(cg, O.gemm(a, b)) < 1e-5
    assert np.array_equal(np.argsort(-cg, -1, kind="stable")[:, :5], np.argsort(-O.gemm(a, b), -1, kind="stable")[:, :5])


def test_tf32x3_per_call_override(backend):
    rng = np.random.default_rng(31)
    x = rng.standard_normal((200, 100)).astype(np.float32)       # K = 100: not a multiple of 4 floats
    w = rng.standard_normal((70, 100)).astype(np.float32)
    b = rng.standard_normal(70).astype(np.float32)
    y = backend.fnn.linear(x, w, b, precision="tf32x3")
    assert O.rel_l2(y, O.linear(x, w, b)) < 1e-5
    assert O.rel_l2(backend.fnn.linear(x, w, b), O.linear(x, w, b)) > 1e-5   # the plain tf32 product is coarser
    a, bm = rng.standard_normal((130, 72)).astype(np.float32), rng.standard_normal((72, 258)).astype(np.float32)
    assert O.rel_l2(backend.fnn.gemm(a, bm, precision="tf32x3"), O.gemm(a, bm)) < 1e-5
    with pytest.raises(ValueError):
        backend.fnn.linear(x, w, b, precision="fp64")


@pytest.mark.parametrize("M,N,K", [(1, 8, 4), (7, 13, 20), (128, 64, 32), (129, 65, 36), (300, 200, 100), (1000, 1152, 384),
                                   (513, 384, 1536), (64, 2816, 1024)])
def test_linear_edge_shapes(backend, M, N, K):
    rng = np.random.default_rng(M * 7 + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    assert O.rel_l2(backend.fnn.linear(x, w, b), O.linear(x, w, b)) < TOL_TF32
    assert O.rel_l2(backend.fnn.fused_linear_silu(x, w), O.fused_linear_silu(x, w)) < TOL_TF32


@pytest.mark.parametrize("bn", [64, 128, 192, 256])
def test_every_n_tile(backend, bn):
    backend.device.set_tuning("gemm_bn", bn)
    try:
        rng = np.random.default_rng(bn)
        x = rng.standard_normal((700, 384)).astype(np.float32)
        w = (rng.standard_normal((1000, 384)) / 20).astype(np.float32)
        assert O.rel_l2(backend.fnn.fused_linear_relu(x, w), O.fused_linear_relu(x, w)) < TOL_TF32
    finally:
        backend.device.set_tuning("gemm_bn", 0)


@pytest.mark.parametrize("M,N,K", [(300, 520, 40), (1000, 384, 96), (2049, 1536, 384), (256, 256, 8)])
def test_cta_pair_kernel(backend, backend_bf16, M, N, K):
    """The cta_group::2 kernel (two CTAs share one MMA, 256 x 256 tiles) on ragged shapes it would not be picked
    for by default: partial token tiles, a feature count that leaves the second CTA of a pair without rows."""
    backend.device.set_tuning("gemm_pair", 1)
    backend_bf16.device.set_tuning("gemm_pair", 1)
    try:
        rng = np.random.default_rng(M + N + K)
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
        b = rng.standard_normal(N).astype(np.float32)
        assert O.rel_l2(backend.fnn.linear(x, w, b), O.linear(x, w, b)) < TOL_TF32
        assert O.rel_l2(backend.fnn.fused_linear_gelu(x, w, b), O.fused_linear_gelu(x, w, b)) < TOL_TF32
        assert O.rel_l2(backend_bf16.fnn.fused_linear_silu(x, w), O.fused_linear_silu(x, w)) < TOL_BF16
        # the same launch through the single-CTA kernel gives the same numbers bit for bit (same MMA order per output)
        y_pair = backend.fnn.linear(x, w, b)
        backend.device.set_tuning("gemm_pair", 0)
        assert np.array_equal(y_pair, backend.fnn.linear(x, w, b))
    finally:
        backend.device.set_tuning("gemm_pair", -1)
        backend_bf16.device.set_tuning("gemm_pair", -1)


def test_linear_is_deterministic_and_weight_cache_is_used(backend):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((256, 384)).astype(np.float32)
    w = rng.standard_normal((384, 384)).astype(np.float32)
    before = backend.fnn.buffer_pool.get_stats()["cached_weights"]
    a = backend.fnn.linear(x, w)
    b = backend.fnn.linear(x, w)
    assert np.array_equal(a, b)
    assert backend.fnn.buffer_pool.get_stats()["cached_weights"] == before + 1
    # an in-place change is picked up after invalidate()
    w *= 2
    backend.invalidate(w)
    assert O.rel_l2(backend.fnn.linear(x, w), 2 * a) < 1e-6


def test_non_contiguous_weight_view(backend):
    # utils/pytorch_ops.py:48 passes other.T, a strided view, as the weight
    rng = np.random.default_rng(6)
    x = rng.standard_normal((64, 128)).astype(np.float32)
    other = rng.standard_normal((128, 96)).astype(np.float32)
    assert O.rel_l2(backend.fnn.linear(x, other.T), O.linear(x, other.T)) < TOL_TF32


def test_shape_errors(backend):
    with pytest.raises(ValueError):
        backend.fnn.linear(np.zeros((4, 8), np.float32), np.zeros((3, 9), np.float32))
    with pytest.raises(AssertionError):
        backend.fnn.gemm(np.zeros((4, 8), np.float32), np.zeros((9, 3), np.float32))


def test_fused_qkv_projection(backend):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((2, 50, 384)).astype(np.float32)
    ws = [(rng.standard_normal((384, 384)) * 0.05).astype(np.float32) for _ in range(3)]
    bs = [rng.standard_normal(384).astype(np.float32) for _ in range(3)]
    out = backend.fnn.fused_qkv_projection(x, np.concatenate(ws, 0), np.concatenate(bs, 0), 12, 32)
    assert out.shape == (2, 50, 1152)
    assert O.rel_l2(out, O.fused_qkv_projection(x, *ws, *bs)) < TOL_TF32


@pytest.mark.parametrize("mode", ["layer", "rms"])
def test_fused_layernorm_linear(backend, mode):
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((300, 384)) * 2 + 0.7).astype(np.float32)
    g, bt = (1 + 0.1 * rng.standard_normal(384)).astype(np.float32), (0.1 * rng.standard_normal(384)).astype(np.float32)
    w, b = (rng.standard_normal((512, 384)) * 0.05).astype(np.float32), rng.standard_normal(512).astype(np.float32)
    out = backend.fnn.fused_layernorm_linear(x, g, bt, w, b, eps=1e-5, mode=mode)
    ref = O.fused_layernorm_linear(x, g, bt, w, b) if mode == "layer" else O.linear(O.rmsnorm(x, g), w, b)
    assert O.rel_l2(out, ref) < TOL_TF32
    out2 = backend.fnn.fused_layernorm_linear(x, g, bt, w, b, eps=1e-5, mode=mode)
    assert np.array_equal(out, out2)


@pytest.mark.parametrize("ratio", [0.0, 1.0, 4.0, 16.0])
def test_fused_layernorm_linear_accuracy_envelope(backend, backend_bf16, ratio):
    """Row means of `ratio` standard deviations (fused-layernorm-linear.glsl:102-126 normalises before the product,
    so the reference has no cancellation): small ratios take the folded form, large ones are normalised first; both
    stay inside the tolerance, in tf32 and in bf16."""
    rng = np.random.default_rng(80 + int(ratio))
    x = (rng.standard_normal((700, 384)) + ratio * (1 + 0.2 * rng.standard_normal((700, 1)))).astype(np.float32)
    g, bt = (1 + 0.1 * rng.standard_normal(384)).astype(np.float32), (0.1 * rng.standard_normal(384)).astype(np.float32)
    w, b = (rng.standard_normal((512, 384)) * 0.05).astype(np.float32), rng.standard_normal(512).astype(np.float32)
    ref = O.fused_layernorm_linear(x, g, bt, w, b)
    err = O.rel_l2(backend.fnn.fused_layernorm_linear(x, g, bt, w, b), ref)
    err16 = O.rel_l2(backend_bf16.fnn.fused_layernorm_linear(x, g, bt, w, b), ref)
    print(f"|mean|/std = {ratio}: rel-L2 {err:.2e} (tf32), {err16:.2e} (bf16)")
    assert err < TOL_TF32
    # bf16 mode stores x itself in bf16: a row mean of `ratio` standard deviations costs ratio * 2^-9 of accuracy
    # before any arithmetic, so the bf16 tolerance can only hold for moderate offsets
    if ratio <= 4.0:
        assert err16 < TOL_BF16
    # RMSNorm has no mean term: always folded, any offset
    ref_rms = O.linear(O.rmsnorm(x, g), w, b)
    assert O.rel_l2(backend.fnn.fused_layernorm_linear(x, g, None, w, b, mode="rms"), ref_rms) < TOL_TF32
    if ratio <= 4.0:
        assert O.rel_l2(backend_bf16.fnn.fused_layernorm_linear(x, g, None, w, b, mode="rms"), ref_rms) < TOL_BF16


def test_invalidate_refreshes_folded_weights(backend):
    rng = np.random.default_rng(81)
    x = rng.standard_normal((64, 128)).astype(np.float32)
    g, bt = np.ones(128, np.float32), np.zeros(128, np.float32)
    w = (rng.standard_normal((96, 128)) * 0.1).astype(np.float32)
    y1 = backend.fnn.fused_layernorm_linear(x, g, bt, w)
    w *= 3
    backend.invalidate(w)
    y2 = backend.fnn.fused_layernorm_linear(x, g, bt, w)
    assert O.rel_l2(y2, 3 * y1) < TOL_TF32       # the new weights are in use (tf32 rounding of 3w is not 3 x that of w)
    assert O.rel_l2(y2, y1) > 0.5


@pytest.mark.parametrize("M,N,K", [(1, 384, 384), (127, 384, 384), (129, 128, 64), (1000, 384, 1536), (300, 256, 100),
                                   (4133, 512, 200), (700, 96, 384), (260, 768, 128)])
def test_linear_residual_layernorm(backend, backend_bf16, M, N, K):
    """LayerNorm(x W^T + b + residual): one kernel for 128/256/384/512 features (whole rows in tensor memory, the
    statistics in the epilogue), GEMM + row kernel for the other widths; against linear -> add -> layernorm of the
    oracle (utils/vulkan_sentence_transformer.py:997-1011)."""
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    res = (rng.standard_normal((M, N)) * 1.5 + 0.3).astype(np.float32)
    g, bt = (1 + 0.2 * rng.standard_normal(N)).astype(np.float32), (0.3 * rng.standard_normal(N)).astype(np.float32)
    ref = O.layernorm(O.linear(x, w, b) + res, g, bt, 1e-5)
    out = backend.fnn.linear_residual_layernorm(x, w, b, res, g, bt, 1e-5)
    assert out.shape == (M, N) and np.isfinite(out).all()
    assert O.rel_l2(out, ref) < TOL_TF32
    assert O.rel_l2(backend_bf16.fnn.linear_residual_layernorm(x, w, b, res, g, bt, 1e-5), ref) < TOL_BF16
    # optional operands left out
    ref0 = O.layernorm(O.linear(x, w), None, None, 1e-5)
    assert O.rel_l2(backend.fnn.linear_residual_layernorm(x, w, None, None), ref0) < TOL_TF32
    # the two-launch form gives the same values up to the rounding of the statistics
    backend.device.set_tuning("fused_ln", 0)
    try:
        two = backend.fnn.linear_residual_layernorm(x, w, b, res, g, bt, 1e-5)
    finally:
        backend.device.set_tuning("fused_ln", 1)
    assert O.rel_l2(out, two) < 1e-5


@pytest.mark.parametrize("N,K", [(128, 256), (256, 384), (384, 384), (384, 1536), (512, 128)])
def test_linear_residual_layernorm_many_tiles_per_cta(backend, backend_bf16, N, K):
    """Enough rows that every CTA pair walks several 256-row tiles (both accumulators where two fit tensor memory, the
    staging buffers reused for the next tile's residual boxes, a ragged last tile): the one-kernel form against the
    two-launch form on all rows, and against the oracle on a spread of them."""
    M = 74 * 256 * 5 + 77
    rng = np.random.default_rng(N + K)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N), dtype=np.float32) + 0.3
    g, bt = (1 + 0.2 * rng.standard_normal(N)).astype(np.float32), (0.3 * rng.standard_normal(N)).astype(np.float32)
    rows = np.r_[0:300, M // 2:M // 2 + 300, M - 400:M]
    ref = O.layernorm(O.linear(x[rows], w, b) + res[rows], g, bt, 1e-5)
    for be, tol, tol2 in ((backend, TOL_TF32, 1e-5), (backend_bf16, TOL_BF16, 1e-5)):
        out = be.fnn.linear_residual_layernorm(x, w, b, res, g, bt, 1e-5)
        be.device.set_tuning("fused_ln", 0)
        try:
            two = be.fnn.linear_residual_layernorm(x, w, b, res, g, bt, 1e-5)
        finally:
            be.device.set_tuning("fused_ln", 1)
        assert np.isfinite(out).all()
        assert O.rel_l2(out, two) < tol2
        assert float(np.abs(out - two).max()) < 1e-3      # no single row is off
        assert O.rel_l2(out[rows], ref) < tol


def test_linear_residual_layernorm_3d_and_large_mean(backend):
    rng = np.random.default_rng(77)
    x = rng.standard_normal((3, 50, 384)).astype(np.float32)
    w = (rng.standard_normal((384, 384)) * 0.05).astype(np.float32)
    res = (rng.standard_normal((3, 50, 384)) + 25.0).astype(np.float32)     # row mean 25 standard deviations from zero
    out = backend.fnn.linear_residual_layernorm(x, w, None, res)
    assert out.shape == (3, 50, 384)
    assert O.rel_l2(out, O.layernorm(O.linear(x, w) + res, None, None, 1e-5)) < TOL_TF32
    with pytest.raises(ValueError):
        backend.fnn.linear_residual_layernorm(x, w, None, res[:, :10])


def test_fused_swiglu(backend):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((200, 256)).astype(np.float32)
    wg, wu = ((rng.standard_normal((352, 256)) / 16).astype(np.float32) for _ in range(2))
    out = backend.fnn.fused_swiglu(x, wg, wu)
    assert out.shape == (200, 352)
    assert O.rel_l2(out, O.fused_swiglu(x, wg, wu)) < TOL_TF32
    bg, bu = rng.standard_normal(352).astype(np.float32), rng.standard_normal(352).astype(np.float32)
    assert O.rel_l2(backend.fnn.fused_swiglu(x, wg, wu, bg, bu), O.fused_swiglu(x, wg, wu, bg, bu)) < TOL_TF32


@pytest.mark.parametrize("rows", [200, 2048])
def test_fused_geglu(backend, backend_bf16, rows):
    """gate * gelu(up) through the same pair epilogue (fused-geglu.glsl:53-84, backend/_glu_append.py:224-262);
    2048 rows take the CTA-pair kernel, 200 the single-CTA one."""
    rng = np.random.default_rng(19)
    x = rng.standard_normal((rows, 256)).astype(np.float32)
    wg, wu = ((rng.standard_normal((384, 256)) / 16).astype(np.float32) for _ in range(2))
    bg, bu = rng.standard_normal(384).astype(np.float32), rng.standard_normal(384).astype(np.float32)
    out = backend.fnn.fused_geglu(x, wg, wu)
    assert out.shape == (rows, 384)
    assert O.rel_l2(out, O.fused_geglu(x, wg, wu)) < TOL_TF32
    assert O.rel_l2(backend.fnn.fused_geglu(x, wg, wu, bg, bu), O.fused_geglu(x, wg, wu, bg, bu)) < TOL_TF32
    assert O.rel_l2(backend_bf16.fnn.fused_geglu(x, wg, wu, bg, bu), O.fused_geglu(x, wg, wu, bg, bu)) < TOL_BF16
    # the SiLU gate is a different function: the two entry points must not be mixed up
    assert O.rel_l2(out, O.fused_swiglu(x, wg, wu)) > 0.05


def test_gemm_mnk_multi_destinations(backend, lib):
    """One product stored to three matrices of a wider pitch at a column offset (the layout of a column-split
    product: on several GPUs the destinations are peer-mapped, here they are local)."""
    import ctypes as C
    rng = np.random.default_rng(21)
    M, K, N, ld, off = 300, 96, 128, 512, 256
    A, B = rng.standard_normal((M, K)).astype(np.float32), rng.standard_normal((K, N)).astype(np.float32)
    dev = backend.device
    ad, bd = backend.to_device(A), backend.to_device(B)
    outs = [dev.upload(np.full((M, ld), 7.0, np.float32)) for _ in range(3)]
    ptrs = (C.c_void_p * 3)(*[o.ptr + off * 4 for o in outs])
    dev.check(lib.grilly_gemm_mnk_multi(dev.ctx, C.c_void_p(ad.ptr), C.c_void_p(bd.ptr), ptrs, 3, M, K, N, C.c_longlong(ld), 0))
    want = backend.fnn.gemm(A, B)
    for o in outs:
        got = o.numpy()
        assert np.array_equal(got[:, off:off + N], want)                       # same kernel, same bits
        assert np.all(got[:, :off] == 7.0) and np.all(got[:, off + N:] == 7.0)   # nothing else is touched
    # a following plain gemm writes one destination only (the list is cleared after the launch)
    again = backend.fnn.gemm(A, B)
    assert np.array_equal(again, want) and np.all(outs[1].numpy()[:, :off] == 7.0)
    assert lib.grilly_gemm_mnk_multi(dev.ctx, C.c_void_p(ad.ptr), C.c_void_p(bd.ptr), ptrs, 3, M, K, 100, C.c_longlong(ld), 0) != 0


def test_linear_backward(backend):
    """The three products of the backward pass (backend/fnn.py:1501-1573) against the reference's CPU outputs."""
    from pathlib import Path
    ref = dict(np.load(Path(__file__).resolve().parent / "golden" / "extras_golden.npz"))
    c = cases.linear_backward()
    gi, gw, gb = backend.fnn.linear_backward(c["grad_out"], c["x"], c["w"], c["bias"])
    assert gi.shape == (3, 40, 96) and gw.shape == (160, 96) and gb.shape == (160,)
    assert O.rel_l2(gi, ref["lb_grad_input"]) < TOL_TF32
    assert O.rel_l2(gw, ref["lb_grad_weight"]) < TOL_TF32
    assert O.rel_l2(gb, ref["lb_grad_bias"]) < TOL_TF32
    assert backend.fnn.linear_backward(c["grad_out"], c["x"], c["w"])[2] is None
    # a training-sized case (4096 tokens, 384 -> 1536) against the oracle
    rng = np.random.default_rng(12)
    go, x = rng.standard_normal((4096, 1536)).astype(np.float32), rng.standard_normal((4096, 384)).astype(np.float32)
    w = (rng.standard_normal((1536, 384)) / 20).astype(np.float32)
    got, want = backend.fnn.linear_backward(go, x, w, np.zeros(1536, np.float32)), O.linear_backward(go, x, w, np.zeros(1536))
    for a, b in zip(got, want):
        assert O.rel_l2(a, b) < TOL_TF32
    with pytest.raises(ValueError):
        backend.fnn.linear_backward(go, x[:-1], w)


def test_gemm_mnk_golden_and_sweep(backend, golden):
    r = cases.rowops()
    assert O.rel_l2(backend.fnn.gemm(r["gemm_a"], r["gemm_b"]), golden["gemm_c"]) < TOL_TF32
    for n in (1024, 2048):
        rng = np.random.default_rng(4 + int(np.log2(n)))
        a, b = rng.standard_normal((n, n)).astype(np.float32), rng.standard_normal((n, n)).astype(np.float32)
        assert O.rel_l2(backend.fnn.gemm(a, b), O.gemm(a, b)) < TOL_TF32
    for m, k, n in ((5, 7, 9), (130, 70, 258), (64, 33, 100)):
        rng = np.random.default_rng(m)
        a, b = rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32)
        c = backend.fnn.gemm(a, b)
        assert c.shape == (m, n) and O.rel_l2(c, O.gemm(a, b)) < TOL_TF32


@pytest.mark.parametrize("n", [4096, 8192, 16384])
def test_gemm_mnk_full_size_property(backend, backend_bf16, n):
    """At the sweep's large sizes the O(N^3) oracle is too slow: check C v = A (B v) and u C = (u A) B for random
    u, v (checksums that any wrong tile, k-block or swizzle would break, and that localise an error to a tile), in
    both modes of the sweep. The checks use float32 matrix-vector products (error ~1e-5, far below the tolerances),
    which keeps them to seconds at 16384 (1 GiB per matrix)."""
    rng = np.random.default_rng(4 + int(np.log2(n)))
    a = rng.standard_normal((n, n), dtype=np.float32)
    b = rng.standard_normal((n, n), dtype=np.float32)
    v = rng.standard_normal((n, 3)).astype(np.float32)
    u = rng.standard_normal((3, n)).astype(np.float32)
    want_v, want_u = a @ (b @ v), (u @ a) @ b
    for be, tol in ((backend, TOL_TF32), (backend_bf16, TOL_BF16)):
        c = be.fnn.gemm(a, b)
        assert c.shape == (n, n) and c.dtype == np.float32
        assert O.rel_l2(c @ v, want_v) < tol
        assert O.rel_l2(u @ c, want_u) < tol
        # the checksums would pass for a C that is right on average: a sample of entries against float64 dot products
        rows, cols = rng.integers(0, n, size=64), rng.integers(0, n, size=64)
        exact = np.einsum("ik,ki->i", a[rows].astype(np.float64), b[:, cols].astype(np.float64))
        assert O.rel_l2(c[rows, cols], exact) < 3 * tol
        del c


def test_bf16_mode(backend_bf16):
    c = cases.linear_cfg0()
    y = backend_bf16.fnn.fused_linear_gelu(c["x"], c["w"], c["b"])
    assert O.rel_l2(y, O.fused_linear_gelu(c["x"], c["w"], c["b"])) < TOL_BF16
    rng = np.random.default_rng(3)
    a, b = rng.standard_normal((1024, 1024)).astype(np.float32), rng.standard_normal((1024, 1024)).astype(np.float32)
    assert O.rel_l2(backend_bf16.fnn.gemm(a, b), O.gemm(a, b)) < TOL_BF16
    x = rng.standard_normal((300, 1024)).astype(np.float32)
    wg, wu = ((rng.standard_normal((2816, 1024)) * 0.02).astype(np.float32) for _ in range(2))
    assert O.rel_l2(backend_bf16.fnn.fused_swiglu(x, wg, wu), O.fused_swiglu(x, wg, wu)) < TOL_BF16
