"""The pre-norm ModernBERT architecture (utils/vulkan_sentence_transformer.py:799-970: q/k/v from x, rotate-half RoPE,
x += attn, LayerNorm, GeGLU MLP, x += mlp; final LayerNorm and CLS pooling in encode, :1145-1183): the layer composed
from Compute() ops against the reference's own output, and the resident encoder against the oracle."""
from pathlib import Path

import numpy as np
import pytest

import cases
from conftest import TOL_TF32
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def layer_over_compute(b, x, lw, mask, num_heads):
    """The reference's layer written against the backend namespaces, with the fused ops where the reference has
    separate calls: one QKV GEMM, flash attention with RoPE on the load, the GeGLU as one GEMM."""
    B, S, hid = x.shape
    d = hid // num_heads
    wqkv = np.concatenate([lw["attn_q_weight"], lw["attn_k_weight"], lw["attn_v_weight"]], 0)
    bqkv = np.concatenate([lw["attn_q_bias"], lw["attn_k_bias"], lw["attn_v_bias"]], 0)
    qkv = b.fnn.fused_qkv_projection(x, wqkv, bqkv, num_heads, d).reshape(B, S, 3, num_heads, d)
    a = b.attention.flash_attention2(np.ascontiguousarray(qkv[:, :, 0]), np.ascontiguousarray(qkv[:, :, 1]),
                                     np.ascontiguousarray(qkv[:, :, 2]), mask=mask, use_rope=True, rope_base=10000.0,
                                     rope_style="rotate_half")
    x = x + b.fnn.linear(a.reshape(B, S, hid), lw["attn_out_weight"], lw["attn_out_bias"])
    n = b.fnn.layernorm(x, lw["ffn_ln_gamma"], lw["ffn_ln_beta"], 1e-5)
    # fused_geglu computes first * gelu(second): the reference applies GELU to the gate projection and multiplies by up
    h = b.fnn.fused_geglu(n, lw["ffn_up_weight"], lw["ffn_gate_weight"], lw["ffn_up_bias"], lw["ffn_gate_bias"])
    return x + b.fnn.linear(h, lw["ffn_w2"], lw["ffn_b2"])


def test_layer_against_reference_output(backend):
    ref = dict(np.load(Path(__file__).resolve().parent / "golden" / "extras_golden.npz"))
    m = cases.modernbert_layer()
    y = layer_over_compute(backend, m["x"], m["lw"], m["mask"], m["num_heads"])
    assert O.rel_l2(y, ref["mb_y"]) < TOL_TF32
    assert O.rel_l2(y - m["x"], ref["mb_y"] - m["x"]) < 3 * TOL_TF32     # the layer's own contribution


def test_resident_modernbert_encoder(backend):
    import grilly_b200

    rng = np.random.default_rng(50)
    w = grilly_b200.EncoderWeights.random_modernbert(rng, num_layers=3, hidden=384, ffn=576, vocab=3000)
    enc = grilly_b200.SentenceEncoder(w, num_heads=12, device=backend.device, arch="modernbert", rope_base=10000.0)
    try:
        ids = rng.integers(0, 3000, size=(9, 70))
        lens = np.array([70, 1, 33, 64, 65, 17, 70, 2, 40])
        mask = (np.arange(70)[None, :] < lens[:, None]).astype(np.float32)
        enc.keep_hidden(True)
        out = enc.encode_ids(ids, mask)
        want, hidden = O.modernbert_forward(ids, mask, w.as_dict(), 12, return_hidden=True)
        assert out.shape == (9, 384)
        assert O.rel_l2(out, want) < TOL_TF32
        np.testing.assert_allclose(np.linalg.norm(out, axis=-1), 1.0, atol=1e-5)
        packed = np.concatenate([hidden[i, : lens[i]] for i in range(9)], 0)
        assert O.rel_l2(enc.last_hidden(), packed) < TOL_TF32
        # the one-layer resident model equals the layer composed from the ops above
        # padding never matters, and a longer sequence than 128 tokens takes more than one key tile
        ids2 = ids.copy()
        ids2[mask < 0.5] = 5
        assert np.array_equal(enc.encode_ids(ids2, mask), out)
        ids_long = rng.integers(0, 3000, size=(2, 300))
        mlong = (np.arange(300)[None, :] < np.array([300, 131])[:, None]).astype(np.float32)
        assert O.rel_l2(enc.encode_ids(ids_long, mlong), O.modernbert_forward(ids_long, mlong, w.as_dict(), 12)) < TOL_TF32
    finally:
        enc.close()
    with pytest.raises(Exception):
        grilly_b200.SentenceEncoder(w, num_heads=12, device=backend.device, arch="modernbert", precision="bf16")
