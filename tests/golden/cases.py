"""Seeded inputs of the golden cases, shared by make_golden.py (which runs the reference on them) and by the
tests (which run the oracle and the CUDA path on them). Only outputs are stored in hotpath_golden.npz."""
from __future__ import annotations

import numpy as np

f32 = np.float32


def linear_cfg0():
    """BASELINE config 0: x (32,384) ~ N(0,1); W Xavier-uniform in the reference layout (1536,384); zero bias; seed 0."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((32, 384)).astype(f32)
    lim = np.sqrt(6.0 / (384 + 1536))
    w = rng.uniform(-lim, lim, size=(1536, 384)).astype(f32)
    b = np.zeros(1536, f32)
    x3 = rng.standard_normal((3, 5, 50)).astype(f32)
    w3 = rng.standard_normal((21, 50)).astype(f32)
    b3 = rng.standard_normal(21).astype(f32)
    return dict(x=x, w=w, b=b, x3=x3, w3=w3, b3=b3)


def rowops():
    rng = np.random.default_rng(10)
    return dict(
        gemm_a=rng.standard_normal((40, 24)).astype(f32), gemm_b=rng.standard_normal((24, 36)).astype(f32),
        ln_x=(rng.standard_normal((7, 11, 96)) * 3 + 1.5).astype(f32),
        ln_g=rng.standard_normal(96).astype(f32), ln_b=rng.standard_normal(96).astype(f32),
        sm_x=rng.standard_normal((13, 37)).astype(f32) * 4,
        act_x=rng.standard_normal((9, 64)).astype(f32) * 3,
    )


def attention_cfg1(batch=2):
    """BASELINE config 1 at a reduced batch: q, k, v (batch, 64, 8, 64) in the reference's (B,S,H,D) layout, seed 1."""
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((batch, 64, 8, 64)).astype(f32) for _ in range(3))
    lens = np.array([64, 17, 1, 40])[:batch]
    mask = (np.arange(64)[None, :] < lens[:, None]).astype(f32)
    qs, ks, vs = (rng.standard_normal((2, 50, 12, 32)).astype(f32) for _ in range(3))
    pid = rng.integers(0, 200, size=(batch, 64)).astype(np.int32)
    return dict(q=q, k=k, v=v, mask=mask, q32=qs, k32=ks, v32=vs, pid=pid)


def encoder_layer_cfg2():
    """One post-LN BERT layer of the MiniLM shape (hidden 384, 12 heads, ffn 1536), std 0.02, seed 2."""
    rng = np.random.default_rng(2)
    hid, ffn, B, S = 384, 1536, 3, 24
    n = lambda *s: (rng.standard_normal(s) * 0.02).astype(f32)  # noqa: E731
    lw = {
        "attn_q_weight": n(hid, hid), "attn_q_bias": n(hid), "attn_k_weight": n(hid, hid), "attn_k_bias": n(hid),
        "attn_v_weight": n(hid, hid), "attn_v_bias": n(hid), "attn_out_weight": n(hid, hid), "attn_out_bias": n(hid),
        "attn_ln_gamma": (1 + n(hid)).astype(f32), "attn_ln_beta": n(hid),
        "ffn_w1": n(ffn, hid), "ffn_b1": n(ffn), "ffn_w2": n(hid, ffn), "ffn_b2": n(hid),
        "ffn_ln_gamma": (1 + n(hid)).astype(f32), "ffn_ln_beta": n(hid),
    }
    x = rng.standard_normal((B, S, hid)).astype(f32)
    lens = np.array([24, 9, 16])
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(f32)
    return dict(lw=lw, x=x, mask=mask, num_heads=12)


def faiss_search():
    """Vector search: 10 queries and 1000 database vectors of dimension 256 ~ N(0,1) (the sizes of the reference's
    end-to-end test), a distance matrix for top-k with exact ties in it, seed 42."""
    rng = np.random.default_rng(42)
    queries = rng.standard_normal((10, 256)).astype(f32)
    database = rng.standard_normal((1000, 256)).astype(f32)
    dist = rng.standard_normal((10, 1000)).astype(f32)
    dist[3, 100:140] = dist[3].min() - 1.0      # forty equal smallest values: more ties than k
    dist[5, ::7] = np.round(dist[5, ::7], 1)    # scattered exact ties
    return dict(queries=queries, database=database, dist=dist, k=20)


def linear_backward():
    """Gradients of a (3, 40, 96) -> 160 linear layer, seed 11 (3-D input as the encoder passes it)."""
    rng = np.random.default_rng(11)
    return dict(grad_out=rng.standard_normal((3, 40, 160)).astype(f32), x=rng.standard_normal((3, 40, 96)).astype(f32),
                w=(rng.standard_normal((160, 96)) / 10).astype(f32), bias=np.zeros(160, f32))


def backward_ops():
    """Training-side ops: LayerNorm backward on (4, 33, 96) with an offset input, softmax backward on (6, 5, 37),
    attention backward on (B 2, H 3, S 20, D 16) with its forward softmax weights, one Adam step on 1000 values; seed 12."""
    rng = np.random.default_rng(12)
    ln_x = (rng.standard_normal((4, 33, 96)) * 2 + 0.7).astype(f32)
    ln_go = rng.standard_normal((4, 33, 96)).astype(f32)
    ln_g = (1 + 0.2 * rng.standard_normal(96)).astype(f32)
    sm_logits = rng.standard_normal((6, 5, 37)) * 2
    e = np.exp(sm_logits - sm_logits.max(-1, keepdims=True))
    sm_y = (e / e.sum(-1, keepdims=True)).astype(f32)
    sm_go = rng.standard_normal((6, 5, 37)).astype(f32)
    q, k, v, go = (rng.standard_normal((2, 3, 20, 16)).astype(f32) for _ in range(4))
    scale = 0.25
    sc = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) * scale
    ew = np.exp(sc - sc.max(-1, keepdims=True))
    aw = (ew / ew.sum(-1, keepdims=True)).astype(f32)
    w, g = rng.standard_normal(1000).astype(f32), rng.standard_normal(1000).astype(f32)
    m1, m2 = (0.1 * rng.standard_normal(1000)).astype(f32), (0.01 * rng.random(1000)).astype(f32)
    return dict(ln_x=ln_x, ln_go=ln_go, ln_g=ln_g, sm_y=sm_y, sm_go=sm_go, q=q, k=k, v=v, go=go, aw=aw, scale=scale,
                w=w, g=g, m1=m1, m2=m2, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, beta1_t=0.9 ** 3, beta2_t=0.999 ** 3)


def modernbert_layer():
    """One pre-norm ModernBERT layer (hidden 384, 12 heads, GeGLU width 576), std 0.02, seed 13."""
    rng = np.random.default_rng(13)
    hid, ffn, B, S = 384, 576, 3, 40
    n = lambda *s: (rng.standard_normal(s) * 0.02).astype(f32)  # noqa: E731
    lw = {
        "attn_q_weight": n(hid, hid), "attn_q_bias": n(hid), "attn_k_weight": n(hid, hid), "attn_k_bias": n(hid),
        "attn_v_weight": n(hid, hid), "attn_v_bias": n(hid), "attn_out_weight": n(hid, hid), "attn_out_bias": n(hid),
        "ffn_ln_gamma": (1 + n(hid)).astype(f32), "ffn_ln_beta": n(hid),
        "ffn_gate_weight": n(ffn, hid), "ffn_gate_bias": n(ffn), "ffn_up_weight": n(ffn, hid), "ffn_up_bias": n(ffn),
        "ffn_w2": n(hid, ffn), "ffn_b2": n(hid),
    }
    x = rng.standard_normal((B, S, hid)).astype(f32)
    lens = np.array([40, 13, 27])
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(f32)
    return dict(lw=lw, x=x, mask=mask, num_heads=12)
