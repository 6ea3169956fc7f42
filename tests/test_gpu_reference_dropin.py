"""The reference's own encoder code, unchanged, on top of ``grilly_b200.Compute()``.

``VulkanSentenceTransformer._forward_layer`` (utils/vulkan_sentence_transformer.py:972-1033) is taken from the copy of
the reference package under oracle/_ref (made by oracle/make_ref.py) and run twice: with its own CPU branches, and
with ``grilly.Compute`` pointed at this library, so that ``functional.linear`` / ``functional.layer_norm`` /
``functional.gelu`` (functional/linear.py:28-29, normalization.py:40, activations.py:30-31) and ``_attention_gpu``
(:1037-1067: attention_scores, attention_mask, activation_softmax, attention_output) all land in the CUDA library."""
import numpy as np
import pytest

import cases
from conftest import TOL_TF32
from oracle import oracle as O
from oracle import ref_encoder as R

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason="oracle/_ref (copy of the reference package) is not present")]


def test_forward_layer_unchanged_over_compute(backend, golden):
    e = cases.encoder_layer_cfg2()
    before = backend.device.launch_count()
    st = R.make_transformer(384, e["num_heads"], backend=backend)
    y = R.forward_layers(st, e["x"], [e["lw"]], e["mask"])
    launched = backend.device.launch_count() - before
    # 6 linears, 2 layernorms, 1 gelu, scores + mask + softmax + output (+ the tf32 rounding of uploaded operands)
    assert launched >= 13, f"only {launched} kernels launched: the reference's code fell back to its CPU branches"
    assert np.asarray(y).shape == e["x"].shape
    assert O.rel_l2(y, golden["enc_y"]) < TOL_TF32
    # the same method on its CPU branches is the reference output itself
    st_cpu = R.make_transformer(384, e["num_heads"], backend=None)
    import logging
    logging.disable(logging.CRITICAL)
    try:
        y_cpu = R.forward_layers(st_cpu, e["x"], [e["lw"]], e["mask"])
    finally:
        logging.disable(logging.NOTSET)
    assert O.rel_l2(y_cpu, golden["enc_y"]) < 1e-6


def test_reference_encoder_over_compute_matches_resident_encoder(backend):
    """Six layers of the reference's layer code over Compute() against the resident SentenceEncoder and the oracle."""
    import grilly_b200

    rng = np.random.default_rng(33)
    w = grilly_b200.EncoderWeights.random(rng, num_layers=3, vocab=2000, max_pos=64)
    ids = rng.integers(0, 2000, size=(6, 48))
    lens = np.array([48, 7, 30, 48, 1, 19])
    mask = (np.arange(48)[None, :] < lens[:, None]).astype(np.float32)
    out_ref_code = R.encoder_forward(ids, mask, w.as_dict(), 12, backend=backend)
    want = O.encoder_forward(ids, mask, w.as_dict(), 12)
    assert O.rel_l2(out_ref_code, want) < TOL_TF32
    enc = grilly_b200.SentenceEncoder(w, num_heads=12, device=backend.device)
    try:
        assert O.rel_l2(enc.encode_ids(ids, mask), out_ref_code) < TOL_TF32
    finally:
        enc.close()
    R.make_transformer(384, 12, backend=None)   # put the reference's stock Compute back
