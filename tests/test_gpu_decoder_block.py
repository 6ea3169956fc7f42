"""BASELINE config 3: a GPT-style decoder block in bf16 mode assembled from the hot-path ops -- pre-RMSNorm, fused QKV,
flash_attention2_rope (causal, interleaved RoPE, base 10000), out-projection + residual, pre-RMSNorm, fused SwiGLU FFN
1024 -> 2816 -> 1024 + residual -- against the same block computed by the CPU oracle. Tolerance: rel-L2 <= 1e-2.
Numeric parity at the configuration's own sizes: the attention at (batch 8, seq 4096, 16 heads, dim 64) against the
oracle on a set of (batch, head) slices (the oracle materialises an S x S score matrix per slice), and the whole block
at batch 1 x seq 4096 with the oracle's attention taken head by head. The full shape is also checked for the causal
property (outputs at position < p do not depend on inputs at >= p), bit for bit."""
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


def block_gpu(b, x, w, fold_norm=False):
    B, S, _ = x.shape
    if fold_norm:
        # RMSNorm folded into the QKV product (one statistics kernel + one GEMM, the normalised rows never stored)
        qkv = b.fnn.fused_layernorm_linear(x, w["g1"], None, w["wqkv"], None, 1e-5, mode="rms").reshape(B, S, 3, HEADS, D)
    else:
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
    # head by head: one (S, S) score matrix at a time
    a = np.concatenate([O.flash_attention2_rope(qkv[:, :, 0, hd:hd + 1], qkv[:, :, 1, hd:hd + 1], qkv[:, :, 2, hd:hd + 1], causal=True)
                        for hd in range(HEADS)], axis=2)
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
    # the same block with the first RMSNorm folded into the QKV projection
    yf = block_gpu(backend_bf16, x, w, fold_norm=True)
    assert O.rel_l2(yf, ref) < TOL_BF16 and O.rel_l2(yf - x, ref - x) < 3 * TOL_BF16


def test_attention_at_the_configurations_own_shape(backend_bf16):
    """flash_attention2_rope, causal, interleaved RoPE base 10000, bf16, q/k/v (8, 4096, 16, 64) ~ N(0,1), seed 3:
    the long-sequence path (K rotated by the pre-pass, 32 key tiles per query tile, causal tile skipping) against the
    oracle on ten (batch, head) slices, with the first and the last query tile looked at on their own."""
    rng = np.random.default_rng(3)
    B, S = 8, 4096
    q, k, v = (rng.standard_normal((B, S, HEADS, D), dtype=np.float32) for _ in range(3))
    o = backend_bf16.attention.flash_attention2_rope(q, k, v, causal=True, rope_base=10000.0)
    assert o.shape == (B, S, HEADS, D) and np.isfinite(o).all()
    slices = [(0, 0), (0, 15), (1, 3), (2, 7), (3, 8), (4, 12), (5, 1), (6, 5), (7, 0), (7, 15)]
    worst = 0.0
    for b, hd in slices:
        ref = O.flash_attention2_rope(q[b:b + 1, :, hd:hd + 1], k[b:b + 1, :, hd:hd + 1], v[b:b + 1, :, hd:hd + 1], causal=True)[0, :, 0]
        got = o[b, :, hd]
        errs = (O.rel_l2(got, ref), O.rel_l2(got[:128], ref[:128]), O.rel_l2(got[-128:], ref[-128:]),
                O.rel_l2(got[2048 - 64:2048 + 64], ref[2048 - 64:2048 + 64]))
        worst = max(worst, *errs)
        assert max(errs) < TOL_BF16, (b, hd, errs)
        assert np.allclose(got[0], v[b, 0, hd], atol=2e-2)     # the first query sees only the first key
    print(f"attention (8, 4096, 16, 64) bf16 causal RoPE: worst rel-L2 over {len(slices)} slices and their edge tiles {worst:.2e}")


def test_decoder_block_parity_at_seq_4096(backend_bf16):
    rng = np.random.default_rng(3)
    w = make_weights(rng)
    x = rng.standard_normal((1, 4096, HID)).astype(np.float32)
    y = block_gpu(backend_bf16, x, w)
    ref = block_oracle(x, w)
    assert O.rel_l2(y, ref) < TOL_BF16
    assert O.rel_l2(y - x, ref - x) < 3 * TOL_BF16
    # the last positions attend over all 32 key tiles
    assert O.rel_l2((y - x)[:, -128:], (ref - x)[:, -128:]) < 3 * TOL_BF16


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
