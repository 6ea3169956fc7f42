"""BASELINE config 3: a GPT-style decoder block in bf16 mode assembled from the hot-path ops -- pre-RMSNorm, fused QKV,
flash_attention2_rope (causal, interleaved RoPE, base 10000), out-projection + residual, pre-RMSNorm, fused SwiGLU FFN
1024 -> 2816 -> 1024 + residual -- against the same block computed by the CPU oracle. Tolerance: rel-L2 <= 1e-2.
The CPU oracle materialises (H, S, S) scores, so parity runs at batch 1, seq 1024; the full shape (batch 8, seq 4096)
is checked for finiteness and for the causal property (outputs at position < p do not depend on inputs at >= p)."""
import numpy as np
import pytest

from conftest import TOL_BF16
from oracle import oracle as O

pytestmark = pytest.mark.gpu
HID, HEADS, D, FFN = 1024, 16, 64, 2816


def make_weights(rng):
    n = lambda *s: (rng.standard_normal(s) * 0.02).astype(np.float32)  # noqa: E731
    return dict(g1=np.ones(HID, np.float32), wqkv=n(3 * HID, HID), wo=n(HID, HID), g2=np.ones(HID, np.float32),
                wg=n(FFN, HID), wu=n(FFN, HID), wd=n(HID, FFN))


def block_gpu(b, x, w):
    B, S, _ = x.shape
    h = b.fnn.rmsnorm(x, w["g1"], 1e-5)
    qkv = b.fnn.fused_qkv_projection(h, w["wqkv"], None, HEADS, D).reshape(B, S, 3, HEADS, D)
    a = b.attention.flash_attention2_rope(np.ascontiguousarray(qkv[:, :, 0]), np.ascontiguousarray(qkv[:, :, 1]),
                                          np.ascontiguousarray(qkv[:, :, 2]), causal=True, rope_base=10000.0)
    x = x + b.fnn.linear(a.reshape(B, S, HID), w["wo"])
    h = b.fnn.rmsnorm(x, w["g2"], 1e-5)
    return x + b.fnn.linear(b.fnn.fused_swiglu(h, w["wg"], w["wu"]), w["wd"])


def block_oracle(x, w):
    B, S, _ = x.shape
    h = O.rmsnorm(x, w["g1"], 1e-5)
    qkv = O.linear(h, w["wqkv"]).reshape(B, S, 3, HEADS, D)
    a = O.flash_attention2_rope(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=True)
    x = x + O.linear(a.reshape(B, S, HID), w["wo"])
    h = O.rmsnorm(x, w["g2"], 1e-5)
    return x + O.linear(O.fused_swiglu(h, w["wg"], w["wu"]), w["wd"])


def test_decoder_block_parity_bf16(backend_bf16):
    rng = np.random.default_rng(3)
    w = make_weights(rng)
    x = rng.standard_normal((1, 1024, HID)).astype(np.float32)
    y = block_gpu(backend_bf16, x, w)
    ref = block_oracle(x, w)
    assert O.rel_l2(y, ref) < TOL_BF16
    # the block's own contribution (without the residual stream that dominates the norm)
    assert O.rel_l2(y - x, ref - x) < 3 * TOL_BF16


def test_decoder_block_full_shape_is_causal(backend_bf16):
    rng = np.random.default_rng(3)
    w = make_weights(rng)
    x = rng.standard_normal((2, 4096, HID)).astype(np.float32)
    y = block_gpu(backend_bf16, x, w)
    assert np.isfinite(y).all()
    x2 = x.copy()
    x2[:, 3000:] = rng.standard_normal((2, 1096, HID)).astype(np.float32)
    y2 = block_gpu(backend_bf16, x2, w)
    assert np.array_equal(y[:, :3000], y2[:, :3000])       # positions before the change are untouched, bit for bit
    assert not np.array_equal(y[:, 3000:], y2[:, 3000:])
