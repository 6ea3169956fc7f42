"""Generates tests/golden/hotpath_golden.npz and extras_golden.npz by running the REFERENCE's own CPU code paths.

Run where the reference source tree is available:

    python tests/golden/make_golden.py /path/to/grilly-source            # both files
    python tests/golden/make_golden.py /path/to/grilly-source --extras-only

The reference is imported as the package ``grilly`` through a temporary symlink (its tree is not copied),
Vulkan is absent so every op takes its numba/NumPy branch. Inputs come from the seeded generators in
cases.py; only the reference's outputs are stored, as small float32 arrays. tests/test_oracle_golden.py pins oracle/oracle.py against this file.
"""
from __future__ import annotations

import os
import sys
import tempfile
import types
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent))
import cases  # noqa: E402

OUT = Path(__file__).resolve().parent / "hotpath_golden.npz"
OUT_EXTRAS = Path(__file__).resolve().parent / "extras_golden.npz"


def import_reference(src: str):
    tmp = tempfile.mkdtemp(prefix="grilly_ref_")
    os.symlink(src, os.path.join(tmp, "grilly"))
    os.environ.setdefault("NUMBA_CACHE_DIR", os.path.join(tmp, "numba_cache"))
    sys.path.insert(0, tmp)
    import grilly  # noqa: F401
    from grilly.backend.fnn import VulkanFNN
    from grilly.backend.attention import VulkanAttention
    from grilly.nn.modules import FlashAttention2
    from grilly.utils.vulkan_sentence_transformer import VulkanSentenceTransformer
    from grilly.backend.capsule_transformer import VulkanCapsuleTransformer
    return VulkanFNN, VulkanAttention, FlashAttention2, VulkanSentenceTransformer, VulkanCapsuleTransformer


def main(src: str) -> None:
    VulkanFNN, VulkanAttention, FlashAttention2, VST, Capsule = import_reference(src)
    g: dict[str, np.ndarray] = {}
    f32 = np.float32
    fnn = VulkanFNN(None, None, {})  # empty shader table: every method takes its CPU branch

    # ---- config 0: linear / fused linear
    c = cases.linear_cfg0()
    x, w, b = c["x"], c["w"], c["b"]
    g["lin_y"] = np.asarray(fnn.linear(x, w, b), f32)
    g["lin_gelu_y8"] = np.asarray(fnn.fused_linear_gelu(x[:8], w, b), f32)
    g["lin_silu_y8"] = np.asarray(fnn.fused_linear_silu(x[:8], w, b), f32)
    g["lin_relu_y8"] = np.asarray(fnn.fused_linear_relu(x[:8], w, b), f32)
    g["lin3_y"] = np.asarray(fnn.linear(c["x3"], c["w3"], c["b3"]), f32)
    g["lin3_nobias_y"] = np.asarray(fnn.linear(c["x3"], c["w3"]), f32)

    # ---- gemm, layernorm, softmax, activations
    r = cases.rowops()
    g["gemm_c"] = np.asarray(fnn.gemm(r["gemm_a"], r["gemm_b"]), f32)
    xl, gam, bet = r["ln_x"], r["ln_g"], r["ln_b"]
    g["ln_y"] = np.asarray(fnn.layernorm(xl, gam, bet, eps=1e-5), f32)
    g["ln_y_default"] = np.asarray(fnn.layernorm(xl), f32)
    g["ln_y_eps12"] = np.asarray(fnn.layernorm(xl, gam, bet, eps=1e-12), f32)
    g["sm_y"] = np.asarray(fnn.activation_softmax(r["sm_x"]), f32)
    xa = r["act_x"]
    g["act_gelu"] = np.asarray(fnn.activation_gelu(xa), f32)
    g["act_silu"] = np.asarray(fnn.activation_silu(xa), f32)
    g["act_relu"] = np.asarray(fnn.activation_relu(xa), f32)
    g["act_swiglu"] = np.asarray(fnn.activation_swiglu(xa), f32)
    g["residual"] = np.asarray(fnn.residual(xa, xa[::-1].copy()), f32)
    # RMSNorm as nn/snn.py:374-375 states it
    rms = np.sqrt(np.mean(xl ** 2, axis=-1, keepdims=True) + 1e-5)
    g["rms_y"] = (xl / rms * gam).astype(f32)

    # ---- config 1 (batch 2): attention on the (B,S,H,D) layout
    a = cases.attention_cfg1()
    q, k, v, mask = a["q"], a["k"], a["v"], a["mask"]
    fa = FlashAttention2(512, 8)
    fa._backend = types.SimpleNamespace()  # no flash_attention2 attribute -> NumPy branch (nn/modules.py:1421-1456)
    g["att_o"] = np.asarray(fa.forward(q, k, v), f32)
    # key-padding mask through the encoder's CPU attention (utils/vulkan_sentence_transformer.py:1069-1107)
    st = object.__new__(VST)
    g["att_o_masked"] = np.asarray(st._attention_cpu(q, k, v, mask), f32)
    g["att32_o"] = np.asarray(st._attention_cpu(a["q32"], a["k32"], a["v32"], None), f32)

    # ---- RoPE: interleaved (capsule transformer) and rotate-half (attention._rope_cpu), on q[:1]
    cap = object.__new__(Capsule)
    cap.config = types.SimpleNamespace(head_dim=64, rope_base=10000.0, max_seq_len=64, rope_scaling=1.0)
    cap._precompute_rope_cache()
    g["rope_interleaved"] = np.asarray(cap._apply_rope(q[:1], 64), f32)
    att = VulkanAttention(None, None, {})
    g["rope_half"] = np.asarray(att._rope_cpu(q[:1], None, 10000.0, 1.0), f32)
    g["rope_half_pid"] = np.asarray(att._rope_cpu(q[:1], a["pid"][:1], 10000.0, 2.0), f32)

    # ---- config 2 (reduced): one post-LN BERT layer + pooling
    e = cases.encoder_layer_cfg2()
    lw, xe, emask = e["lw"], e["x"], e["mask"]
    st.model_type = "bert"
    st.config = types.SimpleNamespace(hidden_size=384, num_attention_heads=e["num_heads"])
    st.backend = types.SimpleNamespace()
    import inspect
    import logging
    logging.disable(logging.CRITICAL)
    kwargs = {"layer_idx": 0} if "layer_idx" in inspect.signature(st._forward_layer).parameters else {}
    y = st._forward_layer(xe, lw, emask, **kwargs)
    g["enc_y"] = np.asarray(y, f32)
    # pooling + normalise as the encoder's CPU branches state them (:1189-1201)
    me = emask[:, :, None]
    pooled = (np.asarray(y) * me).sum(axis=1) / (me.sum(axis=1) + 1e-8)
    pooled = pooled / (np.linalg.norm(pooled, axis=-1, keepdims=True) + 1e-8)
    g["enc_pooled"] = pooled.astype(f32)

    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KiB, {len(g)} arrays)")


def main_extras(src: str) -> None:
    """Top-k through the reference's own CPU selection (backend/faiss.py:106-118; ``topk`` takes it when there is no
    Vulkan device). ``compute_distances`` has no CPU branch in the reference, so no distance matrix is stored."""
    import_reference(src)
    from grilly.backend.faiss import VulkanFAISS
    c = cases.faiss_search()
    idx, val = VulkanFAISS(None, None).topk(c["dist"], c["k"])
    g = {"topk_idx": np.asarray(idx, np.uint32), "topk_val": np.asarray(val, np.float32)}
    # linear_backward through the reference's CPU branch (backend/fnn.py:1575-1587; no shaders registered)
    from grilly.backend.fnn import VulkanFNN
    b = cases.linear_backward()
    gi, gw, gb = VulkanFNN(None, None, {}).linear_backward(b["grad_out"], b["x"], b["w"], b["bias"])
    g.update(lb_grad_input=np.asarray(gi, np.float32), lb_grad_weight=np.asarray(gw, np.float32), lb_grad_bias=np.asarray(gb, np.float32))
    # backward ops through the reference's CPU branches (no shaders registered): backend/fnn.py:1733-1751 and
    # :1869-1872, backend/autograd_core.py:609-646, backend/learning.py:1003-1010
    from grilly.backend.autograd_core import VulkanBackwardOps
    from grilly.backend.learning import VulkanLearning
    c = cases.backward_ops()
    fnn = VulkanFNN(None, None, {})
    gi, gg, gbeta = fnn.layernorm_backward(c["ln_go"], c["ln_x"], c["ln_g"])
    g.update(lnb_grad_input=np.asarray(gi, np.float32), lnb_grad_gamma=np.asarray(gg, np.float32), lnb_grad_beta=np.asarray(gbeta, np.float32))
    g["smb_grad_input"] = np.asarray(fnn.softmax_backward(c["sm_go"], c["sm_y"]), np.float32)
    ops = VulkanBackwardOps(backend=types.SimpleNamespace())
    gq, gk, gv = ops.attention_backward(c["go"], c["q"], c["k"], c["v"], c["aw"], c["scale"])
    g.update(atb_grad_q=np.asarray(gq, np.float32), atb_grad_k=np.asarray(gk, np.float32), atb_grad_v=np.asarray(gv, np.float32))
    learn = object.__new__(VulkanLearning)
    learn.shaders = {}
    wn, m1n, m2n = learn.adam_update(c["w"], c["g"], c["m1"], c["m2"], c["lr"], c["beta1"], c["beta2"], c["eps"], c["beta1_t"], c["beta2_t"])
    g.update(adam_w=np.asarray(wn, np.float32), adam_m1=np.asarray(m1n, np.float32), adam_m2=np.asarray(m2n, np.float32))
    # one ModernBERT (pre-norm, RoPE, GeGLU) layer through the reference's NumPy branches
    # (utils/vulkan_sentence_transformer.py:799-970; RoPE by VulkanAttention._rope_cpu, attention by _attention_cpu)
    import inspect
    import logging
    from grilly.backend.attention import VulkanAttention
    from grilly.utils.vulkan_sentence_transformer import VulkanSentenceTransformer
    m = cases.modernbert_layer()
    st = object.__new__(VulkanSentenceTransformer)
    st.model_type = "modernbert"
    st.config = types.SimpleNamespace(hidden_size=384, num_attention_heads=m["num_heads"], local_rope_theta=10000.0, rope_scaling=None)
    st.backend = types.SimpleNamespace(attention=VulkanAttention(None, None, {}))
    logging.disable(logging.CRITICAL)
    kwargs = {"layer_idx": 0} if "layer_idx" in inspect.signature(st._forward_layer).parameters else {}
    g["mb_y"] = np.asarray(st._forward_layer(m["x"], m["lw"], m["mask"], **kwargs), np.float32)
    logging.disable(logging.NOTSET)
    np.savez_compressed(OUT_EXTRAS, **g)
    print(f"wrote {OUT_EXTRAS} ({OUT_EXTRAS.stat().st_size / 1024:.0f} KiB, {len(g)} arrays)")


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    if not args:
        sys.exit("usage: python make_golden.py <path to the grilly source tree> [--extras-only]")
    src = args[0]
    if "--extras-only" in sys.argv:
        main_extras(src)
    else:
        main(src)
        main_extras(src)
