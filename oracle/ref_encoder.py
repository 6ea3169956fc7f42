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
    restated below in float32, as the reference computes them.
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
