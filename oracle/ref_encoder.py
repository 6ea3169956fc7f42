"""Runs the REFERENCE's own encoder code (from the copy under ``oracle/_ref``, see make_ref.py) on this repository's
weight containers. TEST INFRASTRUCTURE ONLY: used by bench.py's reference arm (as the timed CPU implementation) and
by tests/ (as the checker and as the unchanged caller of ``grilly_b200.Compute()``); the product never imports it.

What is the reference's and what is restated here:
  * every transformer layer is ``VulkanSentenceTransformer._forward_layer`` (utils/vulkan_sentence_transformer.py:
    972-1033), called unmodified on a bare instance. With ``backend=None`` every GPU call in it raises and its own
    ``except`` branches run the NumPy maths (the reference's CPU path); with a backend given, ``grilly.Compute`` is
    pointed at it and the same code drives that backend instead.
  * embedding sum + embedding LayerNorm, masked mean pooling and L2 normalisation are the few NumPy lines of
    ``encode`` (:620-705, :726-744, :1185-1201), which need torch modules only as weight containers; they are
    restated below in float32, as the reference computes them (``encoder_forward``).
  * ``encode_texts`` runs the reference's whole ``encode`` (:1109-1219) unmodified instead: the torch modules it reads
    weights from are replaced by plain containers of tensors, and the HuggingFace tokenizer (not available offline) by
    a whitespace tokenizer with the same call signature.
"""
from __future__ import annotations

import inspect
import logging
import os
import sys
import tempfile
import types
from pathlib import Path

import numpy as np

REF_ROOT = Path(__file__).resolve().parent / "_ref"


def available() -> bool:
    return (REF_ROOT / "grilly" / "utils" / "vulkan_sentence_transformer.py").exists()


_VST = None


def _load():
    """Imports the reference package from oracle/_ref (about 20 s cold: it pulls in numba and torch)."""
    global _VST
    if _VST is not None:
        return _VST
    if not available():
        raise RuntimeError("oracle/_ref/grilly is missing: run `python oracle/make_ref.py <grilly source tree>`")
    os.environ.setdefault("NUMBA_CACHE_DIR", os.path.join(tempfile.gettempdir(), "grilly_ref_numba_cache"))
    if str(REF_ROOT) not in sys.path:
        sys.path.insert(0, str(REF_ROOT))
    logging.getLogger("grilly").setLevel(logging.CRITICAL)
    from grilly.utils.vulkan_sentence_transformer import VulkanSentenceTransformer  # noqa: E402

    _VST = VulkanSentenceTransformer
    return _VST


def make_transformer(hidden: int, num_heads: int, backend=None, model_type: str = "bert"):
    """A bare ``VulkanSentenceTransformer`` (no model download, no Vulkan) whose ``_forward_layer`` can be called.
    ``backend``: None for the reference's CPU path, or an object with the ``grilly.Compute()`` namespaces; the
    reference's ``functional.*`` wrappers build ``grilly.Compute()`` per call (functional/linear.py:9-12), so that
    name is pointed at the given backend."""
    VST = _load()
    import grilly

    st = object.__new__(VST)
    st.model_type = model_type
    st.config = types.SimpleNamespace(hidden_size=hidden, num_attention_heads=num_heads)
    if backend is None:
        st.backend = types.SimpleNamespace()          # no attention namespace: _attention_gpu raises, CPU branch runs
        if not hasattr(grilly, "_stock_Compute"):
            grilly._stock_Compute = grilly.Compute
        grilly.Compute = grilly._stock_Compute
    else:
        st.backend = backend
        if not hasattr(grilly, "_stock_Compute"):
            grilly._stock_Compute = grilly.Compute
        grilly.Compute = lambda *a, **k: backend
    return st


def forward_layers(st, x, layers, mask):
    """x (B, S, hidden) through every layer with the reference's ``_forward_layer``."""
    has_idx = "layer_idx" in inspect.signature(st._forward_layer).parameters
    for i, lw in enumerate(layers):
        x = st._forward_layer(x, lw, mask, **({"layer_idx": i} if has_idx else {}))
    return x


def embed(ids, w, eps=1e-12):
    """word + token-type row 0 + position, then LayerNorm: utils/vulkan_sentence_transformer.py:620-705, 726-744."""
    ids = np.asarray(ids)
    x = w["word"][ids]
    if w.get("type") is not None:
        x = x + w["type"][0][None, None, :]
    x = x + w["pos"][: ids.shape[1]][None, :, :]
    mean = x.mean(axis=-1, keepdims=True)
    var = x.var(axis=-1, keepdims=True)
    return ((x - mean) / np.sqrt(var + eps) * w["emb_ln_g"] + w["emb_ln_b"]).astype(np.float32)


def pool_normalize(x, mask):
    """masked mean (:1185-1191) and x / (||x|| + 1e-8) (:1196-1201)."""
    m = np.asarray(mask, dtype=np.float32)[:, :, None]
    pooled = (x * m).sum(axis=1) / (m.sum(axis=1) + 1e-8)
    return pooled / (np.linalg.norm(pooled, axis=-1, keepdims=True) + 1e-8)


def encoder_forward(ids, mask, w, num_heads, backend=None, return_hidden=False):
    """The whole sentence encoder with the reference's layer code; w as ``EncoderWeights.as_dict()`` gives it."""
    st = make_transformer(int(w["word"].shape[1]), num_heads, backend)
    logging.disable(logging.CRITICAL)   # the reference logs every failed GPU call
    try:
        x = forward_layers(st, embed(ids, w), w["layers"], np.asarray(mask, dtype=np.float32))
    finally:
        logging.disable(logging.NOTSET)
    out = np.asarray(pool_normalize(np.asarray(x), mask), dtype=np.float32)
    return (out, np.asarray(x)) if return_hidden else out


class WhitespaceTokenizer:
    """Stands in for the HuggingFace tokenizer ``encode`` calls (:550-556): ids from a checksum of each whitespace-
    separated word, [CLS] = 1 in front, [SEP] = 2 behind, padding 0; returns NumPy arrays like ``return_tensors='np'``."""

    def __init__(self, vocab: int):
        self.vocab = int(vocab)

    def __call__(self, texts, padding=True, truncation=True, max_length=128, return_tensors="np"):
        import zlib

        rows = []
        for t in texts:
            ids = [1] + [3 + zlib.crc32(wd.encode()) % (self.vocab - 3) for wd in t.split()][: max_length - 2] + [2]
            rows.append(ids)
        width = max(len(r) for r in rows)
        input_ids = np.zeros((len(rows), width), dtype=np.int64)
        mask = np.zeros((len(rows), width), dtype=np.int64)
        for i, r in enumerate(rows):
            input_ids[i, : len(r)] = r
            mask[i, : len(r)] = 1
        return {"input_ids": input_ids, "attention_mask": mask}


def make_full_transformer(w, num_heads, backend=None, max_seq_length=128, embed_ln_eps=1e-12):
    """A ``VulkanSentenceTransformer`` on which the reference's own ``encode`` runs: weights of ``EncoderWeights.as_dict()``
    in the containers the method reads them from (``transformer_model.embeddings.*.weight``, ``self.layers``)."""
    import torch

    st = make_transformer(int(w["word"].shape[1]), num_heads, backend)
    t = lambda a: types.SimpleNamespace(weight=torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)))  # noqa: E731
    emb = types.SimpleNamespace(word_embeddings=t(w["word"]), position_embeddings=t(w["pos"]))
    if w.get("type") is not None:
        emb.token_type_embeddings = t(w["type"])
    emb.LayerNorm = types.SimpleNamespace(weight=torch.from_numpy(np.asarray(w["emb_ln_g"], np.float32)),
                                          bias=torch.from_numpy(np.asarray(w["emb_ln_b"], np.float32)), eps=embed_ln_eps)
    st.transformer_model = types.SimpleNamespace(embeddings=emb)
    st.tokenizer = WhitespaceTokenizer(int(w["word"].shape[0]))
    st.max_seq_length = max_seq_length
    st.layers = list(w["layers"])
    st.final_norm_weight = None
    return st


def encode_texts(texts, w, num_heads, backend=None, batch_size=32):
    """``VulkanSentenceTransformer.encode(texts)`` of the reference, unchanged (:1109-1219)."""
    st = make_full_transformer(w, num_heads, backend)
    logging.disable(logging.CRITICAL)
    try:
        return np.asarray(st.encode(list(texts), batch_size=batch_size))
    finally:
        logging.disable(logging.NOTSET)


def reference_nn():
    """The reference's ``grilly.nn.modules`` (nn/modules.py), for tests that drive its ``Linear`` / ``LayerNorm`` modules."""
    _load()
    import grilly.nn.modules as M

    return M
