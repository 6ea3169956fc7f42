"""The device-resident encoder against the reference's CPU encoder maths (oracle), end to end through the C ABI."""
import numpy as np
import pytest

import cases
from conftest import TOL_TF32, index_mismatches
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def make_batch(rng, B, S, lo=1):
    ids = rng.integers(1000, 30000, size=(B, S))
    lens = rng.integers(lo, S + 1, size=B)
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.float32)
    return ids, lens, mask


@pytest.fixture(scope="module")
def small_model():
    import grilly_b200

    rng = np.random.default_rng(2)
    w = grilly_b200.EncoderWeights.random(rng, num_layers=2, hidden=384, ffn=1536, vocab=30522, max_pos=512)
    # non-trivial LayerNorm parameters and biases so every epilogue term is exercised
    for lw in w.layers:
        for key in lw:
            if key.endswith("bias") or key in ("ffn_b1", "ffn_b2") or key.endswith("beta"):
                lw[key] = (rng.standard_normal(lw[key].shape) * 0.02).astype(np.float32)
            if key.endswith("gamma"):
                lw[key] = (1 + rng.standard_normal(lw[key].shape) * 0.05).astype(np.float32)
    enc = grilly_b200.SentenceEncoder(w, num_heads=12)
    yield w, enc
    enc.close()


def test_one_layer_against_reference_outputs(golden):
    """One post-LN BERT layer + pooling, compared with what the reference's _forward_layer produced."""
    import grilly_b200

    e = cases.encoder_layer_cfg2()
    b = grilly_b200.Compute()
    try:
        x, lw, mask = e["x"], e["lw"], e["mask"]
        B, S, hid = x.shape
        wqkv = np.concatenate([lw["attn_q_weight"], lw["attn_k_weight"], lw["attn_v_weight"]], 0)
        bqkv = np.concatenate([lw["attn_q_bias"], lw["attn_k_bias"], lw["attn_v_bias"]], 0)
        qkv = b.fnn.fused_qkv_projection(x, wqkv, bqkv, 12, 32).reshape(B, S, 3, 12, 32)
        att = b.attention.flash_attention2(np.ascontiguousarray(qkv[:, :, 0]), np.ascontiguousarray(qkv[:, :, 1]),
                                           np.ascontiguousarray(qkv[:, :, 2]), mask=mask).reshape(B, S, hid)
        a = b.fnn.linear(att, lw["attn_out_weight"], lw["attn_out_bias"])
        h = b.fnn.residual_layernorm(a, x, lw["attn_ln_gamma"], lw["attn_ln_beta"], 1e-5)
        f = b.fnn.linear(b.fnn.fused_linear_gelu(h, lw["ffn_w1"], lw["ffn_b1"]), lw["ffn_w2"], lw["ffn_b2"])
        y = b.fnn.residual_layernorm(f, h, lw["ffn_ln_gamma"], lw["ffn_ln_beta"], 1e-5)
        valid = mask > 0.5
        assert O.rel_l2(y[valid], golden["enc_y"][valid]) < TOL_TF32
        pooled = b.pooling.mean_pool_normalize(y, mask)
        assert O.rel_l2(pooled, golden["enc_pooled"]) < TOL_TF32
    finally:
        b.cleanup()


def test_encoder_forward_parity(small_model):
    w, enc = small_model
    rng = np.random.default_rng(20)
    ids, lens, mask = make_batch(rng, 48, 128, lo=16)
    enc.keep_hidden(True)
    out = enc.encode_ids(ids, mask)
    assert out.shape == (48, 384) and out.dtype == np.float32
    ref, hidden = O.encoder_forward(ids, mask, w.as_dict(), 12, return_hidden=True)
    assert O.rel_l2(out, ref) < TOL_TF32
    np.testing.assert_allclose(np.linalg.norm(out, axis=-1), 1.0, atol=1e-5)
    packed_ref = np.concatenate([hidden[i, : lens[i]] for i in range(48)], 0)
    assert O.rel_l2(enc.last_hidden(), packed_ref) < TOL_TF32
    enc.keep_hidden(False)
    # top-k identity of the cosine-similarity ranking derived from the embeddings
    sim_g, sim_r = out @ out.T, ref @ ref.T
    np.fill_diagonal(sim_g, -2), np.fill_diagonal(sim_r, -2)
    # (similarities are O(1) and carry twice the embeddings' tolerance: rankings closer than that cannot be kept)
    for k in (1, 5):
        differ, real = index_mismatches(sim_g, sim_r, k, 2 * TOL_TF32)
        print(f"encoder cosine ranking: top-{k} differs in {differ} of 48 rows, {real} of them not near-ties")
        assert real == 0


def test_chunking_padding_and_batch_invariance(small_model):
    import grilly_b200

    w, enc = small_model
    rng = np.random.default_rng(21)
    ids, lens, mask = make_batch(rng, 40, 64)
    lens[3] = 0
    mask[3] = 0  # an empty sentence pools to the zero vector
    full = enc.encode_ids(ids, mask)
    assert np.array_equal(full[3], np.zeros(384, np.float32))
    # token ids under the padding never matter
    ids2 = ids.copy()
    ids2[mask < 0.5] = 7
    assert np.array_equal(enc.encode_ids(ids2, mask), full)
    # chunked execution (activations reused per chunk) and per-sentence execution give the same bits
    enc_c = grilly_b200.SentenceEncoder(w, num_heads=12, device=enc.dev, chunk_tokens=300)
    try:
        assert np.array_equal(enc_c.encode_ids(ids, mask), full)
    finally:
        enc_c.close()
    for i in (0, 7, 39):
        one = enc.encode_ids(ids[i: i + 1], mask[i: i + 1])
        assert np.array_equal(one[0], full[i])
    # no mask = every position valid
    assert O.rel_l2(enc.encode_ids(ids[:4]), O.encoder_forward(ids[:4], None, w.as_dict(), 12)) < TOL_TF32


def test_page_locked_io_buffers_give_the_same_embeddings(small_model):
    """Ids written into the encoder's own staging buffer and embeddings read from it: same bits as the pageable path."""
    w, enc = small_model
    rng = np.random.default_rng(33)
    ids, lens, mask = make_batch(rng, 24, 48)
    want = enc.encode_ids(ids, mask)
    pin_ids, pin_out = enc.io_buffers(24, 48)
    assert pin_ids.shape == (24, 48) and pin_ids.dtype == np.int32 and pin_out.shape == (24, 384)
    pin_ids[...] = ids
    got = enc.encode_ids(pin_ids, mask, out=pin_out)
    assert got is pin_out and np.array_equal(got, want)
    # a smaller batch afterwards reuses the same buffers; a plain call in between does not disturb them
    assert np.array_equal(enc.encode_ids(ids[:5], mask[:5]), want[:5])


@pytest.mark.parametrize("heads", [4, 3])
def test_encoder_with_wide_heads(heads):
    """hidden 384 split into 4 heads of 96 or 3 heads of 128: the long-sequence attention kernel's tf32 instances."""
    import grilly_b200

    rng = np.random.default_rng(50 + heads)
    w = grilly_b200.EncoderWeights.random(rng, num_layers=2, hidden=384, ffn=768, vocab=3000, max_pos=256)
    enc = grilly_b200.SentenceEncoder(w, num_heads=heads)
    try:
        ids, lens, mask = make_batch(rng, 9, 150)
        assert O.rel_l2(enc.encode_ids(ids, mask), O.encoder_forward(ids, mask, w.as_dict(), heads)) < TOL_TF32
    finally:
        enc.close()


def test_masks_with_holes_run_on_the_padded_layout(small_model):
    """A mask that is not a prefix of ones cannot be packed; the encoder then runs padded with the mask as key mask
    and pooling mask, like the reference (positions keep their own position embeddings)."""
    w, enc = small_model
    rng = np.random.default_rng(33)
    ids = rng.integers(1000, 30000, size=(6, 40))
    mask = (rng.random((6, 40)) > 0.35).astype(np.float32)
    mask[:, 0] = 1
    mask[2, 5:] = 0  # one ordinary prefix row in the same batch
    out = enc.encode_ids(ids, mask)
    ref = O.encoder_forward(ids, mask, w.as_dict(), 12)
    assert O.rel_l2(out, ref) < TOL_TF32
    # a prefix mask gives the same embedding on the packed and on the padded path (to tolerance, different kernels)
    pm = np.zeros((6, 40), np.float32)
    pm[:, :17] = 1
    packed = enc.encode_ids(ids, pm)
    pm_holes = pm.copy()
    pm_holes[5, 30] = 1  # forces the padded path for the whole batch; rows 0-4 are unchanged
    padded = enc.encode_ids(ids, pm_holes)
    assert O.rel_l2(padded[:5], packed[:5]) < 1e-3


def test_encoder_bf16_mode(small_model):
    import grilly_b200
    from conftest import TOL_BF16

    w, enc = small_model
    rng = np.random.default_rng(44)
    ids, lens, mask = make_batch(rng, 40, 128, lo=8)
    e16 = grilly_b200.SentenceEncoder(w, num_heads=12, device=enc.dev, precision="bf16")
    try:
        e16.keep_hidden(True)
        out = e16.encode_ids(ids, mask)
        ref, hidden = O.encoder_forward(ids, mask, w.as_dict(), 12, return_hidden=True)
        assert O.rel_l2(out, ref) < TOL_BF16
        packed_ref = np.concatenate([hidden[i, : lens[i]] for i in range(40)], 0)
        assert O.rel_l2(e16.last_hidden(), packed_ref) < TOL_BF16
        assert O.rel_l2(out, enc.encode_ids(ids, mask)) < TOL_BF16
    finally:
        e16.close()


def test_encoder_rejects_bad_input(small_model):
    _, enc = small_model
    with pytest.raises(ValueError):
        enc.encode_ids(np.zeros((2, 600), np.int64))  # longer than the position table
