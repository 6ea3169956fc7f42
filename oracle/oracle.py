"""CPU oracle: a NumPy restatement of grilly's CPU code paths for the dense transformer hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this module; it is used by
tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline leg as the checker / reported
baseline, never as a compute path of the product.

Parity pin: every function below is checked against outputs of the reference's own Python code
(imported from its source tree) stored in tests/golden/*.npz by tests/golden/make_golden.py, and
against the known-answer assertions of the reference's test-suite (tests/test_gpu_operations.py:100-205,
tests/test_gemm_backward.py:68-76) in tests/test_oracle_golden.py.

Citations are file:line in the reference (grilly 0.1.0), relative to its project root.
All functions take and return float32 unless stated; accumulation is done in float64 and cast, so
the oracle is a tighter statement of the maths than the reference's fastmath numba kernels.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
SQRT_2_OVER_PI = 0.7978845608028654


# --------------------------------------------------------------------------- GEMM family
def linear(x, weights, bias=None):
    """y = x @ W.T + b with W (out, in): backend/fnn.py:1394-1416, utils/numba_ops.py:203-281,
    shader fnn-linear.glsl:43-57."""
    x = np.asarray(x, dtype=F32)
    w = np.asarray(weights, dtype=F32)
    y = x.astype(np.float64) @ w.astype(np.float64).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return y.astype(F32)


def gelu(x):
    """tanh-approximation GELU: utils/numba_ops.py:300-306, backend/fnn.py:292-294,
    fused-linear-gelu.glsl:42-62 (the shader's +-50 clamp never changes a float32 result)."""
    x = np.asarray(x, dtype=np.float64)
    return (0.5 * x * (1.0 + np.tanh(SQRT_2_OVER_PI * (x + 0.044715 * x ** 3)))).astype(F32)


def silu(x):
    """x * sigmoid(x): utils/numba_ops.py:346-349, fused-linear-silu.glsl:43-48."""
    x = np.asarray(x, dtype=np.float64)
    return (x / (1.0 + np.exp(-x))).astype(F32)


def relu(x):
    """max(0, x): fused-linear-relu.glsl:63."""
    return np.maximum(np.asarray(x, dtype=F32), F32(0))


def gcu(x):
    """x * cos(x): backend/fnn.py:399-400, utils/numba_ops.py (numba_gcu)."""
    x = np.asarray(x, dtype=np.float64)
    return (x * np.cos(x)).astype(F32)


def roswish(x, alpha=1.0, beta=1.0):
    """(x + alpha) * sigmoid(beta x) - alpha / 2: backend/fnn.py:456-457."""
    x = np.asarray(x, dtype=np.float64)
    return ((x + alpha) / (1.0 + np.exp(-beta * x)) - 0.5 * alpha).astype(F32)


def fused_linear_gelu(x, w, b=None):
    """backend/fnn.py:2022-2123 (falls back to linear then activation_gelu, :2043-2046)."""
    return gelu(linear(x, w, b))


def fused_linear_silu(x, w, b=None):
    """backend/fnn.py:2214-2303."""
    return silu(linear(x, w, b))


def fused_linear_relu(x, w, b=None):
    """backend/fnn.py:2125-2212."""
    return relu(linear(x, w, b))


def gemm(a, b):
    """C = A @ B, all row-major: backend/fnn.py:104-112 (always the NumPy branch), gemm_mnk.glsl:48-87."""
    return (np.asarray(a, dtype=np.float64) @ np.asarray(b, dtype=np.float64)).astype(F32)


def fused_qkv_projection(x, wq, wk, wv, bq=None, bk=None, bv=None):
    """Stacked projection, output columns [Q | K | V]: fused-qkv-projection.glsl:52-73; equals three
    linear calls (utils/vulkan_sentence_transformer.py:976-978)."""
    return np.concatenate([linear(x, wq, bq), linear(x, wk, bk), linear(x, wv, bv)], axis=-1)


def layernorm(x, gamma=None, beta=None, eps=1e-5):
    """gamma * (x - mean) / sqrt(var + eps) + beta, biased variance over the last dim:
    backend/fnn.py:1285-1313, utils/numba_ops.py:70-87, fnn-layernorm.glsl:55-101."""
    x = np.asarray(x, dtype=np.float64)
    mean = x.mean(axis=-1, keepdims=True)
    var = x.var(axis=-1, keepdims=True)
    y = (x - mean) / np.sqrt(var + eps)
    if gamma is not None:
        y = y * np.asarray(gamma, dtype=np.float64)
    if beta is not None:
        y = y + np.asarray(beta, dtype=np.float64)
    return y.astype(F32)


def rmsnorm(x, gamma=None, eps=1e-5):
    """x / sqrt(mean(x^2) + eps) * gamma: snn-rmsnorm.glsl:45-73, nn/snn.py:374-375."""
    x = np.asarray(x, dtype=np.float64)
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    if gamma is not None:
        y = y * np.asarray(gamma, dtype=np.float64)
    return y.astype(F32)


def fused_layernorm_linear(x, gamma, beta, w, b=None, eps=1e-5):
    """Linear(LayerNorm(x)): fused-layernorm-linear.glsl:102-126."""
    return linear(layernorm(x, gamma, beta, eps), w, b)


def softmax(x):
    """Row softmax with max subtraction: activation-softmax.glsl:45-82, utils/numba_ops.py:148-164."""
    x = np.asarray(x, dtype=np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return (e / e.sum(axis=-1, keepdims=True)).astype(F32)


def swiglu(x):
    """Activation form: halves [x1, x2] of the last dim, x1 * silu(x2): activation-swiglu.glsl:32-51,
    utils/numba_ops.py:527-540."""
    x = np.asarray(x, dtype=np.float64)
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return (x1 * (x2 / (1.0 + np.exp(-x2)))).astype(F32)


def fused_swiglu(x, w_gate, w_up, b_gate=None, b_up=None):
    """(x Wg^T + bg) * silu(x Wu^T + bu): backend/_glu_append.py:47-60, fused-swiglu.glsl:54-78. Parity unpinned as a
    fused op (the file is a fragment no class includes); its parts, linear and SiLU, are pinned by the golden file."""
    g = linear(x, w_gate, b_gate if (b_gate is not None and b_up is not None) else None).astype(np.float64)
    u = linear(x, w_up, b_up if (b_gate is not None and b_up is not None) else None).astype(np.float64)
    return (g * (u / (1.0 + np.exp(-u)))).astype(F32)


def fused_geglu(x, w_gate, w_up, b_gate=None, b_up=None):
    """(x Wg^T + bg) * gelu_tanh(x Wu^T + bu): backend/_glu_append.py:224-262 (CPU branch :256-267). Parity unpinned:
    that file is a fragment no class of the reference includes, so it cannot be run to generate outputs. The same gated
    product inside the ModernBERT layer (utils/vulkan_sentence_transformer.py:939-947) is pinned by the layer golden."""
    g = linear(x, w_gate, b_gate).astype(np.float64)
    u = linear(x, w_up, b_up).astype(np.float64)
    return (g * (0.5 * u * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (u + 0.044715 * u ** 3))))).astype(F32)


def linear_backward(grad_output, x, weights, bias=None):
    """(grad_input, grad_weight, grad_bias) of y = x W^T + b: backend/fnn.py:1501-1587 (grad_output @ W,
    grad_output^T @ x, column sums; grad_bias is None without a bias)."""
    go = np.asarray(grad_output, np.float64)
    go2, x2 = go.reshape(-1, go.shape[-1]), np.asarray(x, np.float64).reshape(-1, np.shape(x)[-1])
    gi = (go2 @ np.asarray(weights, np.float64)).reshape(go.shape[:-1] + (np.shape(weights)[1],))
    return gi.astype(F32), (go2.T @ x2).astype(F32), (go2.sum(0).astype(F32) if bias is not None else None)


def residual(a, b):
    """a + b: fnn-residual.glsl:25-34."""
    return (np.asarray(a, dtype=F32) + np.asarray(b, dtype=F32)).astype(F32)


# --------------------------------------------------------------------------- RoPE
def rope_tables(seq_len, head_dim, base=10000.0, scaling=1.0):
    """theta[pos, i] = (pos / scaling) * base^(-2 i / D): backend/capsule_transformer.py:756-768,
    flash-attention2-rope.glsl:74-88."""
    i = np.arange(head_dim // 2, dtype=np.float64)
    freqs = np.power(float(base), -2.0 * i / head_dim)
    theta = np.outer(np.arange(seq_len, dtype=np.float64) / scaling, freqs)
    return np.cos(theta), np.sin(theta)


def rope_interleaved(x, base=10000.0, scaling=1.0):
    """Pairs (2i, 2i+1) on (B, S, H, D): backend/capsule_transformer.py:775-788,
    flash-attention2-rope.glsl:101-141."""
    x = np.asarray(x, dtype=np.float64)
    _, s, _, d = x.shape
    cos, sin = rope_tables(s, d, base, scaling)
    cos, sin = cos[None, :, None, :], sin[None, :, None, :]
    out = np.empty_like(x)
    xe, xo = x[..., 0::2], x[..., 1::2]
    out[..., 0::2] = xe * cos - xo * sin
    out[..., 1::2] = xe * sin + xo * cos
    return out.astype(F32)


def rope_rotate_half(x, position_ids=None, base=10000.0, scaling=1.0):
    """Pairs (i, i + D/2) on (B, S, H, D): backend/attention.py:795-835, rope.glsl:76-125,
    utils/numba_ops.py:726-749."""
    x = np.asarray(x, dtype=np.float64)
    b, s, _, d = x.shape
    half = d // 2
    if position_ids is None:
        position_ids = np.tile(np.arange(s), (b, 1))
    inv_freq = 1.0 / (float(base) ** (np.arange(0, d, 2, dtype=np.float64) / d))
    theta = (np.asarray(position_ids, dtype=np.float64) / scaling)[..., None] * inv_freq  # (B, S, D/2)
    cos, sin = np.cos(theta)[:, :, None, :], np.sin(theta)[:, :, None, :]
    out = np.empty_like(x)
    a, c = x[..., :half], x[..., half:]
    out[..., :half] = a * cos - c * sin
    out[..., half:] = c * cos + a * sin
    return out.astype(F32)


# --------------------------------------------------------------------------- attention
def attention(q, k, v, scale=None, key_mask=None, causal=False):
    """softmax(scale * Q K^T + mask) V on the (B, S, H, D) layout.

    Unmasked: nn/modules.py:1421-1456 (FlashAttention2 NumPy branch). Key-padding mask (B, S), 1 = keep,
    added as (1 - m) * -1e9 on the key axis: utils/vulkan_sentence_transformer.py:1069-1107,
    flash-attention2.glsl:151-154. Causal: key position > query position is replaced by -1e9
    (attention-mask.glsl:42-46). The score arithmetic is float32 where the reference's is, so that a fully
    masked row degenerates the same way (all scores equal -1e9 -> uniform weights)."""
    q = np.asarray(q, dtype=F32)
    k = np.asarray(k, dtype=F32)
    v = np.asarray(v, dtype=F32)
    b, s, h, d = q.shape
    if scale is None:
        scale = 1.0 / np.sqrt(d)
    qt, kt, vt = (t.transpose(0, 2, 1, 3).astype(np.float64) for t in (q, k, v))
    scores = (np.einsum("bhqd,bhkd->bhqk", qt, kt) * scale).astype(F32)
    if key_mask is not None:
        m = np.asarray(key_mask, dtype=F32)
        scores = scores + ((F32(1.0) - m) * F32(-1e9))[:, None, None, :]
    if causal:
        sk = k.shape[1]
        future = np.arange(sk)[None, :] > np.arange(s)[:, None]
        scores = np.where(future[None, None], F32(-1e9), scores)
    scores = scores.astype(np.float64)
    e = np.exp(scores - scores.max(axis=-1, keepdims=True))
    p = e / (e.sum(axis=-1, keepdims=True) + 1e-8)
    out = np.einsum("bhqk,bhkd->bhqd", p, vt)
    return out.transpose(0, 2, 1, 3).astype(F32)


def flash_attention2(q, k, v, scale=None, mask=None, causal=False):
    """Intended semantics of VulkanAttention.flash_attention2 (backend/attention.py:361-597)."""
    return attention(q, k, v, scale=scale, key_mask=mask, causal=causal)


def flash_attention2_rope(q, k, v, scale=None, mask=None, causal=False, rope_base=10000.0, rope_scaling=1.0,
                          rope_style="interleaved"):
    """Scores on RoPE(q), RoPE(k); V is not rotated: flash-attention2-rope.glsl:101-149."""
    if rope_style == "interleaved":
        q, k = rope_interleaved(q, rope_base, rope_scaling), rope_interleaved(k, rope_base, rope_scaling)
    else:
        q = rope_rotate_half(q, None, rope_base, rope_scaling)
        k = rope_rotate_half(k, None, rope_base, rope_scaling)
    return attention(q, k, v, scale=scale, key_mask=mask, causal=causal)


# --------------------------------------------------------------------------- encoder glue
def embedding_lookup(ids, table):
    """Row gather, ids outside [0, vocab) give zero rows: embedding-lookup.glsl:36-54,
    utils/vulkan_sentence_transformer.py:628-637."""
    ids = np.asarray(ids)
    table = np.asarray(table, dtype=F32)
    ok = (ids >= 0) & (ids < table.shape[0])
    out = table[np.where(ok, ids, 0)]
    out[~ok] = 0
    return out.astype(F32)


def mean_pool(x, mask=None):
    """Masked mean over the sequence axis: embedding-pool.glsl:61-81 (m > 0.5, 0 when nothing counts),
    backend/pooling.py:93-96; the NumPy fallback (utils/vulkan_sentence_transformer.py:1189-1191) divides by
    (sum(m) + 1e-8), which differs by 1e-8 relative."""
    x = np.asarray(x, dtype=np.float64)
    if mask is None:
        return x.mean(axis=1).astype(F32)
    keep = (np.asarray(mask) > 0.5).astype(np.float64)[:, :, None]
    cnt = keep.sum(axis=1)
    return np.where(cnt > 0, (x * keep).sum(axis=1) / np.maximum(cnt, 1.0), 0.0).astype(F32)


def embedding_normalize(x):
    """x / (||x||_2 + 1e-8): functional/embedding.py:67-68."""
    x = np.asarray(x, dtype=np.float64)
    return (x / (np.linalg.norm(x, axis=-1, keepdims=True) + 1e-8)).astype(F32)


def encoder_layer(x, lw, mask, num_heads, eps=1e-5):
    """Post-LN BERT layer: utils/vulkan_sentence_transformer.py:972-1033 (NumPy branches).
    lw holds attn_{q,k,v,out}_{weight,bias}, attn_ln_{gamma,beta}, ffn_w1/b1/w2/b2, ffn_ln_{gamma,beta}."""
    b, s, hid = x.shape
    d = hid // num_heads
    q = linear(x, lw["attn_q_weight"], lw["attn_q_bias"]).reshape(b, s, num_heads, d)
    k = linear(x, lw["attn_k_weight"], lw["attn_k_bias"]).reshape(b, s, num_heads, d)
    v = linear(x, lw["attn_v_weight"], lw["attn_v_bias"]).reshape(b, s, num_heads, d)
    a = attention(q, k, v, key_mask=mask).reshape(b, s, hid)
    a = linear(a, lw["attn_out_weight"], lw["attn_out_bias"])
    x = layernorm(a + x, lw["attn_ln_gamma"], lw["attn_ln_beta"], eps)
    f = linear(gelu(linear(x, lw["ffn_w1"], lw["ffn_b1"])), lw["ffn_w2"], lw["ffn_b2"])
    return layernorm(f + x, lw["ffn_ln_gamma"], lw["ffn_ln_beta"], eps)


def modernbert_layer(x, lw, mask, num_heads, rope_base=10000.0, eps=1e-5):
    """Pre-norm ModernBERT layer: utils/vulkan_sentence_transformer.py:799-970 (NumPy branches). The attention norm is
    the identity; q and k get rotate-half RoPE (positions 0..S-1); x += attn; LayerNorm; GeGLU MLP
    (gelu(n Wgate^T + bgate) * (n Wup^T + bup)) W2^T + b2; x += mlp. The reference's clips (+-50 on the GELU input,
    +-1e6 elsewhere) do not act on finite activations of this size and are left out."""
    b, s, hid = x.shape
    d = hid // num_heads
    q = linear(x, lw["attn_q_weight"], lw["attn_q_bias"]).reshape(b, s, num_heads, d)
    k = linear(x, lw["attn_k_weight"], lw["attn_k_bias"]).reshape(b, s, num_heads, d)
    v = linear(x, lw["attn_v_weight"], lw["attn_v_bias"]).reshape(b, s, num_heads, d)
    q, k = rope_rotate_half(q, None, rope_base, 1.0), rope_rotate_half(k, None, rope_base, 1.0)
    a = attention(q, k, v, key_mask=mask).reshape(b, s, hid)
    x = (np.asarray(x, np.float64) + linear(a, lw["attn_out_weight"], lw["attn_out_bias"])).astype(F32)
    n = layernorm(x, lw["ffn_ln_gamma"], lw["ffn_ln_beta"], eps)
    h = (gelu(linear(n, lw["ffn_gate_weight"], lw["ffn_gate_bias"])).astype(np.float64)
         * linear(n, lw["ffn_up_weight"], lw["ffn_up_bias"])).astype(F32)
    return (np.asarray(x, np.float64) + linear(h, lw["ffn_w2"], lw["ffn_b2"])).astype(F32)


def modernbert_forward(ids, mask, w, num_heads, rope_base=10000.0, embed_eps=1e-12, layer_eps=1e-5, final_eps=1e-5,
                       return_hidden=False):
    """ModernBERT sentence encoder as ``encode`` runs it (utils/vulkan_sentence_transformer.py:1145-1201): token
    embeddings, embedding LayerNorm (no positions), the layers, the final LayerNorm, CLS pooling, L2 normalise."""
    ids = np.asarray(ids)
    b, s = ids.shape
    x = layernorm(embedding_lookup(ids, w["word"]), w["emb_ln_g"], w["emb_ln_b"], embed_eps)
    mask = np.ones((b, s), dtype=F32) if mask is None else np.asarray(mask, dtype=F32)
    for lw in w["layers"]:
        x = modernbert_layer(x, lw, mask, num_heads, rope_base, layer_eps)
    x = layernorm(x, w["final_norm_weight"], w["final_norm_bias"], final_eps)
    out = embedding_normalize(x[:, 0, :])
    return (out, x) if return_hidden else out


def encoder_forward(ids, mask, w, num_heads, embed_eps=1e-12, layer_eps=1e-5, return_hidden=False):
    """MiniLM/BERT sentence encoder: embeddings (utils/vulkan_sentence_transformer.py:620-705), embedding
    LayerNorm (:726-744), the layers (:972-1033), masked mean pool (:1185-1191), L2 normalise (:1196-1201).
    w: word, pos, type (or None), emb_ln_g, emb_ln_b, layers (list of per-layer dicts)."""
    ids = np.asarray(ids)
    b, s = ids.shape
    x = embedding_lookup(ids, w["word"])
    if w.get("type") is not None:
        x = x + w["type"][0][None, None, :]
    x = x + w["pos"][:s][None, :, :]
    x = layernorm(x, w["emb_ln_g"], w["emb_ln_b"], embed_eps)
    mask = np.ones((b, s), dtype=F32) if mask is None else np.asarray(mask, dtype=F32)
    for lw in w["layers"]:
        x = encoder_layer(x, lw, mask, num_heads, layer_eps)
    out = embedding_normalize(mean_pool(x, mask))
    return (out, x) if return_hidden else out


# --------------------------------------------------------------------------- backward pass and optimiser
def layernorm_backward(grad_output, x, gamma, mean=None, var=None, eps=1e-5):
    """(grad_input, grad_gamma, grad_beta) of LayerNorm: the CPU branch of backend/fnn.py:1733-1751 (the same maths as
    backend/autograd_core.py:566-606), in float64."""
    go, x = np.asarray(grad_output, np.float64), np.asarray(x, np.float64)
    mean = x.mean(axis=-1, keepdims=True) if mean is None else np.asarray(mean, np.float64).reshape(x.shape[:-1] + (1,))
    var = x.var(axis=-1, keepdims=True) if var is None else np.asarray(var, np.float64).reshape(x.shape[:-1] + (1,))
    std = np.sqrt(var + eps)
    x_norm = (x - mean) / std
    lead = tuple(range(x.ndim - 1))
    grad_gamma, grad_beta = np.sum(go * x_norm, axis=lead), np.sum(go, axis=lead)
    n = x.shape[-1]
    dxn = go * (1.0 if gamma is None else np.asarray(gamma, np.float64))
    dvar = np.sum(dxn * (x - mean) * (-0.5) * (var + eps) ** (-1.5), axis=-1, keepdims=True)
    dmean = np.sum(dxn * (-1.0 / std), axis=-1, keepdims=True) + dvar * np.mean(-2.0 * (x - mean), axis=-1, keepdims=True)
    grad_input = dxn / std + dvar * 2.0 * (x - mean) / n + dmean / n
    return grad_input.astype(F32), grad_gamma.astype(F32), grad_beta.astype(F32)


def softmax_backward(grad_output, softmax_output, dim=-1):
    """s * (g - sum(g * s)): backend/fnn.py:1869-1872, backend/autograd_core.py:550-564."""
    g, s = np.asarray(grad_output, np.float64), np.asarray(softmax_output, np.float64)
    return (s * (g - np.sum(g * s, axis=dim, keepdims=True))).astype(F32)


def attention_backward(grad_output, q, k, v, attn_weights, scale):
    """(grad_q, grad_k, grad_v) on the (B, H, S, D) layout: backend/autograd_core.py:609-646,
    shaders/attention-backward.glsl (grad_V = A^T dO; grad_scores = softmax_backward(dO V^T, A) * scale;
    grad_Q = grad_scores K; grad_K = grad_scores^T Q)."""
    go, q, k, v, a = (np.asarray(t, np.float64) for t in (grad_output, q, k, v, attn_weights))
    grad_v = np.matmul(a.swapaxes(-2, -1), go)
    grad_attn = np.matmul(go, v.swapaxes(-2, -1))
    gs = a * (grad_attn - np.sum(grad_attn * a, axis=-1, keepdims=True)) * scale
    return np.matmul(gs, k).astype(F32), np.matmul(gs.swapaxes(-2, -1), q).astype(F32), grad_v.astype(F32)


def adam_update(w, g, m1, m2, lr, beta1=0.9, beta2=0.999, eps=1e-8, beta1_t=0.0, beta2_t=0.0):
    """One Adam step (new weights, moment1, moment2): CPU branch of backend/learning.py:1003-1010, adam-update.glsl."""
    w, g, m1, m2 = (np.asarray(t, np.float64) for t in (w, g, m1, m2))
    m1n = beta1 * m1 + (1.0 - beta1) * g
    m2n = beta2 * m2 + (1.0 - beta2) * g * g
    mh = m1n / (1.0 - beta1_t) if beta1_t < 1.0 else m1n
    vh = m2n / (1.0 - beta2_t) if beta2_t < 1.0 else m2n
    return (w - lr * mh / (np.sqrt(vh) + eps)).astype(F32), m1n.astype(F32), m2n.astype(F32)


# --------------------------------------------------------------------------- vector search
def faiss_distances(queries, database, distance_type="cosine"):
    """Pairwise distances as the shader states them (shaders/faiss-distance.glsl:29-83; the reference has no CPU
    branch for this op): 'l2' sqrt(sum (q-d)^2), 'cosine' 1 - q.d / (sqrt(q.q) sqrt(d.d) + 1e-8), 'dot' -(q.d);
    any other name is treated as cosine (backend/faiss.py:44-45). Parity unpinned: there is no reference CPU code to
    generate outputs from; checked against the closed forms of the reference's tests (tests/test_gpu_operations.py:219-241)."""
    q = np.asarray(queries, np.float64)
    if q.ndim == 1:
        q = q.reshape(1, -1)
    d = np.asarray(database, np.float64)
    if distance_type == "l2":
        out = np.sqrt(((q[:, None, :] - d[None, :, :]) ** 2).sum(-1))
    elif distance_type == "dot":
        out = -(q @ d.T)
    else:
        out = 1.0 - (q @ d.T) / (np.sqrt((q * q).sum(-1))[:, None] * np.sqrt((d * d).sum(-1))[None, :] + 1e-8)
    return out.astype(np.float32)


def faiss_topk(distances, k):
    """k smallest entries per row, ascending (backend/faiss.py:106-118). The reference leaves the order of equal
    values to argpartition/argsort; here equal values come by ascending index, which is one of the orders it allows."""
    dist = np.asarray(distances, np.float32)
    if dist.ndim == 1:
        dist = dist.reshape(1, -1)
    k = min(int(k), dist.shape[1])
    idx = np.argsort(dist, axis=1, kind="stable")[:, :k]
    return idx.astype(np.uint32), np.take_along_axis(dist, idx, axis=1).astype(np.float32)


# --------------------------------------------------------------------------- checkers
def rel_l2(a, b):
    """||a - b||_2 / ||b||_2 in float64."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def xavier_uniform(rng, out_features, in_features):
    """U(-l, l), l = sqrt(6 / (in + out)), array shape (out, in): nn/modules.py:38-43."""
    lim = np.sqrt(6.0 / (in_features + out_features))
    return rng.uniform(-lim, lim, size=(out_features, in_features)).astype(F32)
