"""Parity of the tcgen05 flash-attention kernel (and its RoPE variant) with the reference's CPU attention."""
import numpy as np
import pytest

import cases
from conftest import TOL_BF16, TOL_TF32, index_mismatches
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_config1_against_reference_outputs(backend, golden):
    a = cases.attention_cfg1()
    o = backend.attention.flash_attention2(a["q"], a["k"], a["v"], 8, 64)
    assert o.dtype == np.float32 and o.shape == a["q"].shape
    assert O.rel_l2(o, golden["att_o"]) < TOL_TF32
    om = backend.attention.flash_attention2(a["q"], a["k"], a["v"], 8, 64, mask=a["mask"])
    assert O.rel_l2(om, golden["att_o_masked"]) < TOL_TF32
    o32 = backend.attention.flash_attention2(a["q32"], a["k32"], a["v32"])
    assert O.rel_l2(o32, golden["att32_o"]) < TOL_TF32
    # 3-D (B, S, H*D) form and the explicit scale argument
    B, S, H, D = a["q"].shape
    o3 = backend.attention.flash_attention2(a["q"].reshape(B, S, H * D), a["k"].reshape(B, S, H * D),
                                            a["v"].reshape(B, S, H * D), H, D, scale=0.125)
    assert np.array_equal(o3, o)


def test_config1_full_batch(backend):
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((32, 64, 8, 64)).astype(np.float32) for _ in range(3))
    o = backend.attention.flash_attention2(q, k, v, 8, 64)
    ref = O.flash_attention2(q, k, v)
    assert O.rel_l2(o, ref) < TOL_TF32
    # indices derived from the output (argmax and top-5 over the head dim per (b, s, h)): in tf32 mode they may
    # differ from the oracle's only where the oracle's own values are closer than the tolerance; count reported
    for kk in (1, 5):
        differ, real = index_mismatches(o, ref, kk, TOL_TF32)
        print(f"tf32 attention cfg 1: top-{kk} differs in {differ} of {o.size // 64} rows, {real} of them not near-ties")
        assert real == 0
        assert differ < 0.02 * o.size / 64


def test_config1_exact_indices_in_tf32x3_mode(backend_x3):
    """A 'tf32x3' backend computes attention with fp32 products and sums: values agree with the oracle to fp32
    accuracy and the argmax / top-5 indices over the head dim are identical at the full batch of 32."""
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((32, 64, 8, 64)).astype(np.float32) for _ in range(3))
    o = backend_x3.attention.flash_attention2(q, k, v, 8, 64)
    ref = O.flash_attention2(q, k, v)
    assert O.rel_l2(o, ref) < 1e-5
    assert np.array_equal(o.argmax(-1), ref.argmax(-1))
    assert index_mismatches(o, ref, 5, 1e-5) == (0, 0)
    # masks, the causal rule and RoPE go through the same fp32 path
    lens = rng.integers(1, 65, size=32)
    mask = (np.arange(64)[None, :] < lens[:, None]).astype(np.float32)
    om = backend_x3.attention.flash_attention2(q, k, v, mask=mask, causal=True)
    assert O.rel_l2(om, O.flash_attention2(q, k, v, mask=mask, causal=True)) < 1e-5
    orp = backend_x3.attention.flash_attention2_rope(q[:2], k[:2], v[:2], causal=True)
    assert O.rel_l2(orp, O.flash_attention2_rope(q[:2], k[:2], v[:2], causal=True)) < 1e-5


@pytest.mark.parametrize("B,S,H,D", [(1, 1, 1, 32), (2, 17, 3, 32), (2, 128, 12, 32), (1, 129, 2, 64), (2, 300, 4, 64),
                                     (1, 513, 2, 32)])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_lengths_masks_causal(backend, B, S, H, D, causal):
    rng = np.random.default_rng(S * 3 + D)
    q, k, v = (rng.standard_normal((B, S, H, D)).astype(np.float32) for _ in range(3))
    lens = rng.integers(1, S + 1, size=B)
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.float32)
    o = backend.attention.flash_attention2(q, k, v, mask=mask, causal=causal)
    assert np.isfinite(o).all()
    assert O.rel_l2(o, O.flash_attention2(q, k, v, mask=mask, causal=causal)) < TOL_TF32


def test_mask_with_holes_and_fully_masked_row(backend):
    rng = np.random.default_rng(11)
    q, k, v = (rng.standard_normal((3, 40, 2, 32)).astype(np.float32) for _ in range(3))
    mask = (rng.random((3, 40)) > 0.4).astype(np.float32)
    mask[1] = 0  # every key masked: the reference's scores all become -1e9 -> uniform weights
    o = backend.attention.flash_attention2(q, k, v, mask=mask)
    assert O.rel_l2(o, O.flash_attention2(q, k, v, mask=mask)) < TOL_TF32


@pytest.mark.parametrize("style", ["interleaved", "rotate_half"])
@pytest.mark.parametrize("D", [32, 64])
def test_rope_variant(backend, style, D):
    rng = np.random.default_rng(D)
    q, k, v = (rng.standard_normal((2, 200, 4, D)).astype(np.float32) for _ in range(3))
    o = backend.attention.flash_attention2_rope(q, k, v, causal=True, rope_base=10000.0, rope_style=style)
    ref = O.flash_attention2_rope(q, k, v, causal=True, rope_style=style)
    assert O.rel_l2(o, ref) < TOL_TF32
    o2 = backend.attention.flash_attention2(q, k, v, use_rope=True, rope_scaling=2.0, rope_base=500.0, rope_style=style)
    assert O.rel_l2(o2, O.flash_attention2_rope(q, k, v, rope_scaling=2.0, rope_base=500.0, rope_style=style)) < TOL_TF32


@pytest.mark.parametrize("style", ["interleaved", "rotate_half"])
def test_rope_long_sequences_use_the_prepass(backend, style):
    """Beyond 256 positions Q and K are rotated once into scratch instead of on every tile load: same result."""
    rng = np.random.default_rng(77)
    q, k, v = (rng.standard_normal((1, 600, 3, 64)).astype(np.float32) for _ in range(3))
    o = backend.attention.flash_attention2_rope(q, k, v, causal=True, rope_style=style)
    assert O.rel_l2(o, O.flash_attention2_rope(q, k, v, causal=True, rope_style=style)) < TOL_TF32
    lens = np.array([311])
    mask = (np.arange(600)[None, :] < lens[:, None]).astype(np.float32)
    o = backend.attention.flash_attention2_rope(q, k, v, mask=mask, rope_style=style, rope_scaling=4.0)
    assert O.rel_l2(o, O.flash_attention2_rope(q, k, v, mask=mask, rope_style=style, rope_scaling=4.0)) < TOL_TF32


def test_apply_rope_against_reference_outputs(backend, golden):
    a = cases.attention_cfg1()
    q1 = a["q"][:1]
    assert O.rel_l2(backend.attention.apply_rope(q1), golden["rope_half"]) < 1e-5
    out = backend.attention.apply_rope(q1, a["pid"][:1], 10000.0, 2.0)
    assert O.rel_l2(out, golden["rope_half_pid"]) < 1e-4


def test_bf16_decoder_shapes(backend_bf16):
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((1, 700, 4, 64)).astype(np.float32) for _ in range(3))
    o = backend_bf16.attention.flash_attention2_rope(q, k, v, causal=True)
    assert O.rel_l2(o, O.flash_attention2_rope(q, k, v, causal=True)) < TOL_BF16
    q, k, v = (rng.standard_normal((1, 256, 2, 128)).astype(np.float32) for _ in range(3))
    assert O.rel_l2(backend_bf16.attention.flash_attention2(q, k, v), O.flash_attention2(q, k, v)) < TOL_BF16


def test_bf16_head_dim_32_short_sequences(backend_bf16):
    """head_dim 32 in bf16 is 64 bytes per head: two neighbouring heads share one 128-byte swizzled row."""
    rng = np.random.default_rng(9)
    for B, S, H in ((2, 128, 12), (3, 77, 5), (1, 16, 1)):
        q, k, v = (rng.standard_normal((B, S, H, 32)).astype(np.float32) for _ in range(3))
        lens = rng.integers(1, S + 1, size=B)
        mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.float32)
        o = backend_bf16.attention.flash_attention2(q, k, v, mask=mask)
        assert O.rel_l2(o, O.flash_attention2(q, k, v, mask=mask)) < TOL_BF16


def test_errors(backend):
    z = np.zeros((1, 4, 2, 160), np.float32)
    with pytest.raises(Exception):
        backend.attention.flash_attention2(z, z, z)  # head_dim above 128 is not supported: raises, never falls back
    with pytest.raises(ValueError):
        backend.attention.flash_attention2(np.zeros((1, 4, 64), np.float32), np.zeros((1, 4, 64), np.float32),
                                           np.zeros((1, 4, 64), np.float32))


def test_unfused_pipeline_matches_flash_and_oracle(backend):
    """The four calls the reference's encoder makes today (utils/vulkan_sentence_transformer.py:1037-1067):
    attention_scores -> attention_mask(custom) -> activation_softmax -> attention_output."""
    rng = np.random.default_rng(5)
    B, S, H, D = 3, 50, 12, 32
    q, k, v = (rng.standard_normal((B, S, H, D)).astype(np.float32) for _ in range(3))
    lens = np.array([50, 7, 31])
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.float32)
    a = backend.attention
    scores = a.attention_scores(q, k, H, D)
    assert scores.shape == (B, H, S, S)
    ref_scores = np.einsum("bqhd,bkhd->bhqk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(D)
    assert O.rel_l2(scores, ref_scores) < 1e-6
    masked = a.attention_mask(scores, use_causal=False, mask_value=-1e9, custom_mask=mask)
    assert np.all(masked[1, :, :, 7:] == np.float32(-1e9)) and np.array_equal(masked[0], scores[0])
    w = backend.fnn.activation_softmax(masked.reshape(-1, S), axis=-1).reshape(masked.shape)
    out = a.attention_output(w, v, H, D)
    assert out.shape == (B, S, H, D)
    ref = O.attention(q, k, v, key_mask=mask)
    assert O.rel_l2(out, ref) < 1e-5                                     # fp32 path
    assert O.rel_l2(a.flash_attention2(q, k, v, mask=mask), out) < TOL_TF32
    assert a.attention_concat_heads(out).shape == (B, S, H * D)
    # causal variant and the 3-D input form
    cm = a.attention_mask(a.attention_scores(q.reshape(B, S, H * D), k.reshape(B, S, H * D), H, D), use_causal=True)
    assert np.all(cm[:, :, 3, 4:] == np.float32(-1e9)) and np.all(cm[:, :, 3, :4] == scores[:, :, 3, :4])
    assert np.array_equal(a.attention_mask(scores, use_causal=False), scores)


def test_attention_output_architecture_forms(backend):
    """attention_output as the reference's registry selects it (backend/shader_registry.py:154-156): the causal sum of
    attention-output-gpt.glsl and the decoder-over-encoder form of attention-output-t5.glsl."""
    rng = np.random.default_rng(77)
    B, H, S, D, Sk = 2, 3, 37, 16, 53
    w = rng.random((B, H, S, S)).astype(np.float32)
    v = rng.standard_normal((B, S, H, D)).astype(np.float32)
    try:
        backend.set_architecture("gpt")
        got = backend.attention.attention_output(w, v, H, D)
        ref = np.einsum("bhqk,bkhd->bqhd", np.tril(w).astype(np.float64), v.astype(np.float64))
        assert got.shape == (B, S, H, D) and O.rel_l2(got, ref) < 2e-6
        backend.set_architecture("t5")
        wx = rng.random((B, H, S, Sk)).astype(np.float32)
        ve = rng.standard_normal((B, Sk, H, D)).astype(np.float32)
        got = backend.attention.attention_output(wx, ve, H, D)
        ref = np.einsum("bhqk,bkhd->bqhd", wx.astype(np.float64), ve.astype(np.float64))
        assert got.shape == (B, S, H, D) and O.rel_l2(got, ref) < 2e-6
        backend.set_architecture("bert")
        with pytest.raises(ValueError):
            backend.attention.attention_output(wx, ve, H, D)
        got = backend.attention.attention_output(w, v, H, D)
        assert O.rel_l2(got, np.einsum("bhqk,bkhd->bqhd", w.astype(np.float64), v.astype(np.float64))) < 2e-6
    finally:
        backend.set_architecture(None)


@pytest.mark.parametrize("D,S,causal", [(96, 200, False), (128, 300, True), (128, 100, False), (80, 150, True), (48, 64, False), (16, 40, False)])
def test_more_head_dims_tf32(backend, D, S, causal):
    """Head dims 96 and 128 have their own tf32 instances of the long-sequence kernel; anything else up to 128 runs
    zero-padded to the next instantiated size."""
    rng = np.random.default_rng(D * 1000 + S)
    B, H = 2, 3
    q, k, v = (rng.standard_normal((B, S, H, D)).astype(np.float32) for _ in range(3))
    got = backend.attention.flash_attention2(q, k, v, causal=causal)
    ref = O.flash_attention2(q, k, v, causal=causal)
    assert got.shape == (B, S, H, D) and O.rel_l2(got, ref) < TOL_TF32


@pytest.mark.parametrize("D,S,causal", [(32, 300, True), (96, 200, False), (80, 64, False), (32, 64, False)])
def test_more_head_dims_bf16(backend_bf16, D, S, causal):
    rng = np.random.default_rng(D * 1000 + S + 1)
    B, H = 2, 4
    q, k, v = (rng.standard_normal((B, S, H, D)).astype(np.float32) for _ in range(3))
    got = backend_bf16.attention.flash_attention2(q, k, v, causal=causal)
    ref = O.flash_attention2(q, k, v, causal=causal)
    assert got.shape == (B, S, H, D) and O.rel_l2(got, ref) < TOL_BF16


def test_rope_with_a_padded_head_dim_is_refused(backend):
    q = np.zeros((1, 8, 2, 48), np.float32)
    with pytest.raises(ValueError):
        backend.attention.flash_attention2_rope(q, q, q, causal=True)
