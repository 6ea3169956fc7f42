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


def test_reference_encode_unchanged_over_compute(backend):
    """The reference's whole ``encode`` (utils/vulkan_sentence_transformer.py:1109-1219: tokenize, embedding lookup,
    position / type embeddings, embedding LayerNorm, the layers, masked mean pooling, normalisation), unmodified, with
    ``grilly.Compute`` pointed at this library; against the same method on its CPU branches and against the resident
    encoder on the same token ids. Texts are seeded pseudo-words."""
    import grilly_b200

    rng = np.random.default_rng(44)
    w = grilly_b200.EncoderWeights.random(rng, num_layers=2, vocab=5000, max_pos=64)
    words = ["".join(chr(97 + int(c)) for c in rng.integers(0, 26, size=int(n))) for n in rng.integers(2, 9, size=300)]
    texts = [" ".join(words[int(i)] for i in rng.integers(0, 300, size=int(n))) for n in rng.integers(1, 40, size=21)]
    before = backend.device.launch_count()
    got = R.encode_texts(texts, w.as_dict(), 12, backend=backend, batch_size=8)
    assert backend.device.launch_count() - before >= 3 * (2 * 13 + 3), "the reference's encode fell back to its CPU branches"
    want = R.encode_texts(texts, w.as_dict(), 12, backend=None, batch_size=8)
    assert got.shape == want.shape == (21, 384) and got.dtype == np.float32
    assert O.rel_l2(got, want) < TOL_TF32
    # the resident encoder on what the tokenizer produced (whole list at once: padding to the longest text)
    enc = grilly_b200.SentenceEncoder(w, num_heads=12, device=backend.device)
    try:
        tok = R.WhitespaceTokenizer(5000)(texts, max_length=128)
        res = enc.encode_ids(tok["input_ids"], tok["attention_mask"].astype(np.float32))
    finally:
        enc.close()
    assert O.rel_l2(res, want) < TOL_TF32
    R.make_transformer(384, 12, backend=None)   # put the reference's stock Compute back


def test_modernbert_layer_branch_unchanged_over_compute(backend):
    """The pre-norm branch of the reference's ``_forward_layer`` (utils/vulkan_sentence_transformer.py:799-970),
    unmodified, over this backend: its linears, LayerNorm and GELU run through ``functional.*`` on the CUDA library, its
    RoPE through ``backend.attention.apply_rope`` (the branch asks for ``_rope_cpu`` first, which this backend does not
    have); the attention of that branch is the reference's own ``_attention_cpu`` by its author's choice. Against the
    golden output of the same branch on the reference's NumPy paths."""
    import types

    from pathlib import Path

    gold = np.load(Path(__file__).resolve().parent / "golden" / "extras_golden.npz")
    m = cases.modernbert_layer()
    st = R.make_transformer(384, m["num_heads"], backend=backend, model_type="modernbert")
    st.config = types.SimpleNamespace(hidden_size=384, num_attention_heads=m["num_heads"], local_rope_theta=10000.0, rope_scaling=None)
    before = backend.device.launch_count()
    import logging
    logging.disable(logging.CRITICAL)
    try:
        y = R.forward_layers(st, m["x"], [m["lw"]], m["mask"])
    finally:
        logging.disable(logging.NOTSET)
    # 7 linears, 1 layernorm, 1 gelu, 2 rope (+ uploads' rounding kernels)
    assert backend.device.launch_count() - before >= 11
    assert O.rel_l2(y, gold["mb_y"]) < TOL_TF32
    R.make_transformer(384, 12, backend=None)   # put the reference's stock Compute back


def test_reference_nn_modules_over_compute(backend):
    """``grilly.nn.Linear`` and ``grilly.nn.LayerNorm`` of the reference (nn/modules.py:123-181, 340-367), unmodified,
    with this backend behind them: ``Linear.forward`` reads ``backend.core.shaders`` and takes its ``fnn.gemm`` path for
    large products (on a transposed VIEW of the weight) and ``fnn.linear`` for small ones."""
    M = R.reference_nn()
    R.make_transformer(384, 12, backend=backend)     # points grilly.Compute at this backend (the modules build one)
    rng = np.random.default_rng(46)
    lin = M.Linear(96, 160)
    assert lin._get_backend() is backend
    W, b = M._get_param_array(lin.weight), M._get_param_array(lin.bias)
    b[...] = rng.standard_normal(160).astype(np.float32)
    for shape in ((3, 40, 96), (4, 96)):          # 120 x 160 >= 4096 -> gemm path; 4 x 160 -> linear path
        x = rng.standard_normal(shape).astype(np.float32)
        before = backend.device.launch_count()
        y = lin.forward(x)
        assert backend.device.launch_count() > before, "nn.Linear fell back to NumPy"
        assert y.shape == shape[:-1] + (160,) and O.rel_l2(y, O.linear(x, W, b)) < TOL_TF32
    ln = M.LayerNorm(96)
    x = (rng.standard_normal((5, 7, 96)) * 2 + 1).astype(np.float32)
    assert O.rel_l2(ln.forward(x), O.layernorm(x, np.ones(96, np.float32), np.zeros(96, np.float32), 1e-5)) < 2e-6
    R.make_transformer(384, 12, backend=None)   # put the reference's stock Compute back
