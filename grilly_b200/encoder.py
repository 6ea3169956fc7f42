"""Device-resident sentence encoder: the counterpart of ``VulkanSentenceTransformer.encode``
(utils/vulkan_sentence_transformer.py:1109-1219, BERT branch of ``_forward_layer`` :972-1033).

Weights are uploaded once; ``encode_ids`` uploads token ids, runs the packed (padding-free) forward in the
CUDA library and returns mean-pooled, L2-normalised float32 embeddings.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib as L
from .device import Device


@dataclass
class EncoderWeights:
    """Host-side weights in the reference's layout (every matrix is (out, in), as ``_extract_weights`` stores them,
    utils/vulkan_sentence_transformer.py:114-542)."""

    word: np.ndarray                 # (vocab, hidden)
    pos: np.ndarray                  # (max_pos, hidden)
    type: np.ndarray | None          # (2, hidden) or None (DistilBERT)
    emb_ln_g: np.ndarray
    emb_ln_b: np.ndarray
    layers: list = field(default_factory=list)  # dicts with the reference's per-layer keys
    final_norm_weight: np.ndarray | None = None  # pre-norm (ModernBERT) models: the LayerNorm after the last layer
    final_norm_bias: np.ndarray | None = None

    @staticmethod
    def random(rng, num_layers=6, hidden=384, ffn=1536, vocab=30522, max_pos=512, std=0.02):
        """Random-init MiniLM-L6-shaped weights: N(0, std^2) matrices and tables, zero biases, LayerNorm gamma=1, beta=0."""
        f32 = np.float32
        n = lambda *s: (rng.standard_normal(s) * std).astype(f32)  # noqa: E731
        layers = []
        for _ in range(num_layers):
            layers.append({
                "attn_q_weight": n(hidden, hidden), "attn_q_bias": np.zeros(hidden, f32),
                "attn_k_weight": n(hidden, hidden), "attn_k_bias": np.zeros(hidden, f32),
                "attn_v_weight": n(hidden, hidden), "attn_v_bias": np.zeros(hidden, f32),
                "attn_out_weight": n(hidden, hidden), "attn_out_bias": np.zeros(hidden, f32),
                "attn_ln_gamma": np.ones(hidden, f32), "attn_ln_beta": np.zeros(hidden, f32),
                "ffn_w1": n(ffn, hidden), "ffn_b1": np.zeros(ffn, f32),
                "ffn_w2": n(hidden, ffn), "ffn_b2": np.zeros(hidden, f32),
                "ffn_ln_gamma": np.ones(hidden, f32), "ffn_ln_beta": np.zeros(hidden, f32),
            })
        return EncoderWeights(word=n(vocab, hidden), pos=n(max_pos, hidden), type=n(2, hidden),
                              emb_ln_g=np.ones(hidden, f32), emb_ln_b=np.zeros(hidden, f32), layers=layers)

    @staticmethod
    def random_modernbert(rng, num_layers=2, hidden=384, ffn=576, vocab=30522, std=0.02):
        """Random-init weights of the pre-norm architecture with the per-layer keys the reference's ModernBERT
        branch reads (utils/vulkan_sentence_transformer.py:799-970): no position table, ``ffn_gate_weight`` (goes
        through GELU) and ``ffn_up_weight`` (multiplies), one LayerNorm per layer (before the MLP), a final norm."""
        f32 = np.float32
        n = lambda *s: (rng.standard_normal(s) * std).astype(f32)  # noqa: E731
        g = lambda: (1 + 0.1 * rng.standard_normal(hidden)).astype(f32)  # noqa: E731
        layers = []
        for _ in range(num_layers):
            layers.append({
                "attn_q_weight": n(hidden, hidden), "attn_q_bias": n(hidden), "attn_k_weight": n(hidden, hidden), "attn_k_bias": n(hidden),
                "attn_v_weight": n(hidden, hidden), "attn_v_bias": n(hidden), "attn_out_weight": n(hidden, hidden), "attn_out_bias": n(hidden),
                "ffn_ln_gamma": g(), "ffn_ln_beta": n(hidden),
                "ffn_gate_weight": n(ffn, hidden), "ffn_gate_bias": n(ffn), "ffn_up_weight": n(ffn, hidden), "ffn_up_bias": n(ffn),
                "ffn_w2": n(hidden, ffn), "ffn_b2": n(hidden),
            })
        return EncoderWeights(word=n(vocab, hidden), pos=np.zeros((1, hidden), f32), type=None, emb_ln_g=g(), emb_ln_b=n(hidden),
                              layers=layers, final_norm_weight=g(), final_norm_bias=n(hidden))

    def as_dict(self) -> dict:
        return {"word": self.word, "pos": self.pos, "type": self.type, "emb_ln_g": self.emb_ln_g,
                "emb_ln_b": self.emb_ln_b, "layers": self.layers, "final_norm_weight": self.final_norm_weight,
                "final_norm_bias": self.final_norm_bias}


class SentenceEncoder:
    """Sentence encoder resident on one GPU: the post-LN BERT/MiniLM architecture with mean pooling (arch 'bert'), or
    the pre-norm ModernBERT one with RoPE, a GeGLU MLP, a final LayerNorm and CLS pooling (arch 'modernbert', tf32 mode);
    L2-normalised embeddings either way.

    precision 'tf32': fp32 activations, tf32 tensor-core products (parity tolerance 2e-3).
    precision 'bf16': bf16 weights and activations between the GEMMs, fp32 accumulation, fp32 LayerNorm inputs and
    pooling (tolerance 1e-2); with head_dim 32 it handles sequences up to 128 tokens."""

    def __init__(self, weights: EncoderWeights, num_heads: int = 12, embed_ln_eps: float = 1e-12,
                 layer_ln_eps: float = 1e-5, device: Device | int = 0, chunk_tokens: int = 0, precision: str = "tf32",
                 arch: str = "bert", rope_base: float = 10000.0, final_ln_eps: float = 1e-5):
        if precision not in ("tf32", "bf16"):
            raise ValueError("precision must be 'tf32' or 'bf16'")
        if arch not in ("bert", "modernbert"):
            raise ValueError("arch must be 'bert' or 'modernbert'")
        self.arch = arch
        self.precision = precision
        self.dev = device if isinstance(device, Device) else Device(device)
        self._own_dev = not isinstance(device, Device)
        self.lib = self.dev.lib
        self.hidden = int(weights.word.shape[1])
        self.num_heads = num_heads
        ffn_key = "ffn_w1" if arch == "bert" else "ffn_gate_weight"
        cfg = L.EncoderConfig(
            num_layers=len(weights.layers), hidden=self.hidden, num_heads=num_heads,
            ffn=int(weights.layers[0][ffn_key].shape[0]), vocab=int(weights.word.shape[0]),
            max_pos=int(weights.pos.shape[0]), embed_ln_eps=embed_ln_eps, layer_ln_eps=layer_ln_eps,
            has_token_type=int(weights.type is not None), precision=L.PREC_BF16 if precision == "bf16" else L.PREC_TF32,
            chunk_tokens=int(chunk_tokens), arch=L.ARCH_MODERNBERT if arch == "modernbert" else L.ARCH_POST_LN,
            rope_base=float(rope_base), final_ln_eps=float(final_ln_eps))
        h = C.c_void_p()
        self.dev.check(self.lib.grilly_encoder_create(self.dev.ctx, C.byref(cfg), C.byref(h)))
        self.handle = h
        self._upload(weights)

    def _set(self, name: str, layer: int, arr) -> None:
        a = np.ascontiguousarray(arr, dtype=np.float32)
        self.dev.check(self.lib.grilly_encoder_set_weight(self.handle, name.encode(), layer, a.ctypes.data, a.size))

    def _upload(self, w: EncoderWeights) -> None:
        if self.arch == "modernbert":
            return self._upload_modernbert(w)
        self._set("word", -1, w.word)
        self._set("pos", -1, w.pos)
        if w.type is not None:
            self._set("type", -1, w.type[:2])
        self._set("emb_ln_g", -1, w.emb_ln_g)
        self._set("emb_ln_b", -1, w.emb_ln_b)
        for i, lw in enumerate(w.layers):
            # stacked [Wq; Wk; Wv] so Q, K, V come out of one GEMM (fused-qkv-projection.glsl:48-74)
            self._set("wqkv", i, np.concatenate([lw["attn_q_weight"], lw["attn_k_weight"], lw["attn_v_weight"]], 0))
            self._set("bqkv", i, np.concatenate([lw["attn_q_bias"], lw["attn_k_bias"], lw["attn_v_bias"]], 0))
            self._set("wo", i, lw["attn_out_weight"]); self._set("bo", i, lw["attn_out_bias"])
            self._set("ln1_g", i, lw["attn_ln_gamma"]); self._set("ln1_b", i, lw["attn_ln_beta"])
            self._set("w1", i, lw["ffn_w1"]); self._set("b1", i, lw["ffn_b1"])
            self._set("w2", i, lw["ffn_w2"]); self._set("b2", i, lw["ffn_b2"])
            self._set("ln2_g", i, lw["ffn_ln_gamma"]); self._set("ln2_b", i, lw["ffn_ln_beta"])

    def _upload_modernbert(self, w: EncoderWeights) -> None:
        self._set("word", -1, w.word)
        self._set("pos", -1, np.zeros((1, self.hidden), np.float32) if w.pos is None else w.pos)   # unused: positions are RoPE
        self._set("emb_ln_g", -1, w.emb_ln_g)
        self._set("emb_ln_b", -1, w.emb_ln_b)
        self._set("final_g", -1, w.final_norm_weight)
        self._set("final_b", -1, w.final_norm_bias)
        for i, lw in enumerate(w.layers):
            self._set("wqkv", i, np.concatenate([lw["attn_q_weight"], lw["attn_k_weight"], lw["attn_v_weight"]], 0))
            self._set("bqkv", i, np.concatenate([lw["attn_q_bias"], lw["attn_k_bias"], lw["attn_v_bias"]], 0))
            self._set("wo", i, lw["attn_out_weight"]); self._set("bo", i, lw["attn_out_bias"])
            self._set("ln2_g", i, lw["ffn_ln_gamma"]); self._set("ln2_b", i, lw["ffn_ln_beta"])
            # rows (up_j, gate_j): the pair epilogue computes first * gelu(second)  (:893-918: gelu(gate) * up)
            ffn = lw["ffn_gate_weight"].shape[0]
            wgu = np.empty((2 * ffn, self.hidden), np.float32)
            wgu[0::2], wgu[1::2] = lw["ffn_up_weight"], lw["ffn_gate_weight"]
            bgu = np.empty(2 * ffn, np.float32)
            bgu[0::2], bgu[1::2] = lw["ffn_up_bias"], lw["ffn_gate_bias"]
            self._set("wgu", i, wgu); self._set("bgu", i, bgu)
            self._set("w2", i, lw["ffn_w2"]); self._set("b2", i, lw["ffn_b2"])

    def encode_ids(self, input_ids, attention_mask=None, out: np.ndarray | None = None) -> np.ndarray:
        """input_ids (B, S) ints, attention_mask (B, S) 1 = token / 0 = padding (prefix masks run packed, masks with holes run padded).
        Returns float32 (B, hidden). Host buffers in, host buffer out: both copies are part of the call."""
        ids = np.ascontiguousarray(input_ids, dtype=np.int32)
        if ids.ndim != 2:
            raise ValueError("input_ids must be (batch, seq_len)")
        B, S = ids.shape
        mask = None
        if attention_mask is not None:
            mask = np.ascontiguousarray(attention_mask, dtype=np.float32)
            if mask.shape != (B, S):
                raise ValueError(f"attention_mask must have shape {(B, S)}")
        if out is None:
            out = np.empty((B, self.hidden), dtype=np.float32)
        self.dev.check(self.lib.grilly_encoder_forward(self.handle, ids.ctypes.data,
                                                       mask.ctypes.data if mask is not None else None, B, S, out.ctypes.data))
        return out

    def io_buffers(self, B: int, S: int):
        """(ids, out): int32 (B, S) and float32 (B, hidden) NumPy views of the encoder's page-locked staging buffers.
        Ids written there and passed to ``encode_ids(ids, mask, out=out)`` are copied to the device straight from
        page-locked memory, and the embeddings arrive in ``out`` without a second host copy. The views stay valid until
        a larger batch or sequence length is encoded, or the encoder is closed."""
        ip, op = C.c_void_p(), C.c_void_p()
        self.dev.check(self.lib.grilly_encoder_io_buffers(self.handle, int(B), int(S), C.byref(ip), C.byref(op)))
        ids = np.ctypeslib.as_array(C.cast(ip, C.POINTER(C.c_int32)), shape=(int(B), int(S)))
        out = np.ctypeslib.as_array(C.cast(op, C.POINTER(C.c_float)), shape=(int(B), self.hidden))
        return ids, out

    def forward_device(self, ids_dev_ptr: int, lengths, B: int, S: int, out_dev_ptr: int) -> None:
        """Device buffers in and out, no copies, asynchronous (for timing the kernels alone)."""
        ln = np.ascontiguousarray(lengths, dtype=np.int32)
        self.dev.check(self.lib.grilly_encoder_forward_device(self.handle, C.c_void_p(ids_dev_ptr), ln.ctypes.data, B, S,
                                                              C.c_void_p(out_dev_ptr)))

    def keep_hidden(self, on: bool = True) -> None:
        self.dev.check(self.lib.grilly_encoder_keep_hidden(self.handle, int(on)))

    def last_hidden(self) -> np.ndarray:
        """Final hidden states of the last forward as packed rows (total valid tokens, hidden)."""
        rows = C.c_longlong(0)
        self.dev.check(self.lib.grilly_encoder_last_hidden(self.handle, None, 0, C.byref(rows)))
        out = np.empty((rows.value, self.hidden), dtype=np.float32)
        self.dev.check(self.lib.grilly_encoder_last_hidden(self.handle, out.ctypes.data, rows.value, C.byref(rows)))
        return out

    def close(self) -> None:
        if self.handle is not None:
            self.lib.grilly_encoder_destroy(self.handle)
            self.handle = None
            if self._own_dev:
                self.dev.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
