"""``Compute()``: the reference's op namespaces (backend/compute.py:23-128) on top of the CUDA library.

NumPy arrays in, new float32 NumPy arrays out, same method names and positional orders as
``grilly.Compute()`` for the dense transformer path: ``.fnn`` (backend/fnn.py), ``.attention``
(backend/attention.py), ``.pooling`` (backend/pooling.py), ``.learning.embedding_lookup``
(backend/learning.py:811-877). Any argument may also be a :class:`~grilly_b200.device.DeviceTensor`
(from ``backend.to_device``); then the result stays on the device as well.

There is no CPU fallback: an unsupported shape or a missing GPU raises.
"""
from __future__ import annotations

import ctypes as C
import math
from collections import OrderedDict

import numpy as np

from . import _lib as L
from .device import Device, DeviceTensor

_PREC = {"tf32": L.PREC_TF32, "bf16": L.PREC_BF16, "tf32x3": L.PREC_TF32X3}
_ACT = {None: L.ACT_NONE, "none": L.ACT_NONE, "gelu": L.ACT_GELU, "silu": L.ACT_SILU, "relu": L.ACT_RELU}


def _p(t):
    return None if t is None else C.c_void_p(t.ptr)


class _Namespace:
    def __init__(self, backend: "Compute"):
        self._b = backend
        self.dev = backend.device
        self.lib = backend.device.lib
        self.ctx = backend.device.ctx

    # operand staging -------------------------------------------------------------------------
    @property
    def _bf16(self) -> bool:
        return self._b.precision == "bf16"

    def _mode(self, precision=None) -> str:
        """Precision of one GEMM-family call: the per-call override, else the backend's. 'tf32x3' exists for
        linear / fused_linear_* / fused_qkv_projection / gemm only; everything else then runs in tf32."""
        mode = precision if precision is not None else self._b.precision
        if mode not in ("tf32", "bf16", "tf32x3"):
            raise ValueError("precision must be 'tf32', 'bf16' or 'tf32x3'")
        return mode

    def _act_in(self, x, mma_operand: bool = True, mode: str | None = None):
        """Activation operand -> (DeviceTensor, was_host). GEMM/attention operands are staged in the
        precision the tensor core consumes (bf16, or fp32 rounded to the nearest tf32 value; raw fp32 for the
        split products of 'tf32x3')."""
        if isinstance(x, DeviceTensor):
            return x, False
        bf16 = self._bf16 if mode is None else mode == "bf16"
        if mma_operand and bf16:
            return self.dev.upload(x, "bf16"), True
        return self.dev.upload(x, "f32", round_tf32=mma_operand and mode != "tf32x3"), True

    def _vec(self, v):
        """Small fp32 parameter vector (bias, gamma, beta): cached like a weight, never rounded."""
        if v is None:
            return None
        return self.dev.weight(v, "f32", round_tf32=False, tag="vec")

    def _out(self, t: DeviceTensor, to_host: bool, shape=None):
        if shape is not None:
            t = t.reshape(shape)
        return t.numpy() if to_host else t


class FNN(_Namespace):
    """backend/fnn.py ``VulkanFNN``: the GEMM family, normalisation and activations."""

    def __init__(self, backend):
        super().__init__(backend)
        self.buffer_pool = _PoolView(backend.device)

    # ---- GEMM family ------------------------------------------------------------------------
    def _linear(self, x, weights, bias, act, residual=None, flags=0, w_tag="", w_transform=None, n_out=None,
                precision=None, post=None):
        mode = self._mode(precision)
        bf16, x3 = mode == "bf16", mode == "tf32x3"
        w_shape = weights.shape
        if len(w_shape) != 2:
            raise ValueError("weights must be 2-D (out_features, in_features)")
        N, K = (int(s) for s in w_shape)
        x_shape = tuple(x.shape)
        if x_shape[-1] != K:
            raise ValueError(f"input feature size {x_shape[-1]} does not match weights {tuple(w_shape)}")
        elt = 2 if bf16 else 4
        kpad = 0 if x3 else (-K) % (16 // elt)   # the split kernels of tf32x3 pad K themselves
        dt = "bf16" if bf16 else "f32"
        if kpad and not isinstance(x, DeviceTensor):
            # TMA needs 16-byte row pitches: pad K with zeros on both operands
            x = np.pad(np.asarray(x, dtype=np.float32).reshape(-1, K), ((0, 0), (0, kpad)))
            base_tf = w_transform
            w_transform = (lambda a, f=base_tf: np.pad(np.asarray(f(a) if f else a, dtype=np.float32), ((0, 0), (0, kpad))))
            w_tag += f"|kpad{kpad}"
        elif kpad:
            raise ValueError("device-resident operands need in_features * element size to be a multiple of 16 bytes")
        xd, host = self._act_in(x, mode=mode)
        wd = self.dev.weight(weights, dt, round_tf32=not x3, transform=w_transform, tag="w" + w_tag)
        n_rows_w = wd.shape[0]
        bd = self._vec(bias) if not isinstance(bias, DeviceTensor) else bias
        rd = None
        if residual is not None:
            rd, _ = self._act_in(residual, mma_operand=False)
        M = xd.size // (K + kpad)
        n_cols = n_out if n_out is not None else n_rows_w
        y = self.dev.empty((M, n_cols), "f32")
        self.dev.check(self.lib.grilly_linear(self.ctx, _p(xd), _p(wd), _p(bd), _p(rd), _p(y), M, n_rows_w, K + kpad,
                                              act, _PREC[mode], flags))
        if post is not None:                      # (op, p0, p1): an activation the GEMM epilogue does not carry
            self.dev.check(self.lib.grilly_activation_params(self.ctx, post[0], _p(y), _p(y), y.size, float(post[1]), float(post[2])))
        return self._out(y, host, x_shape[:-1] + (n_cols,))

    def linear(self, x, weights, bias=None, precision=None):
        """y = x @ W.T + b, W (out, in): backend/fnn.py:1394-1496. ``precision='tf32x3'`` (here or on the backend)
        gives fp32-level products, for callers that take argmax / top-k indices from the result."""
        return self._linear(x, weights, bias, L.ACT_NONE, precision=precision)

    def fused_linear_gelu(self, x, weights, bias=None, precision=None):
        """gelu_tanh(x @ W.T + b): backend/fnn.py:2022-2123."""
        return self._linear(x, weights, bias, L.ACT_GELU, precision=precision)

    def fused_linear_relu(self, x, weights, bias=None, precision=None):
        """relu(x @ W.T + b): backend/fnn.py:2125-2212."""
        return self._linear(x, weights, bias, L.ACT_RELU, precision=precision)

    def fused_linear_silu(self, x, weights, bias=None, precision=None):
        """silu(x @ W.T + b): backend/fnn.py:2214-2303."""
        return self._linear(x, weights, bias, L.ACT_SILU, precision=precision)

    def linear_residual_layernorm(self, x, weights, bias, residual, gamma=None, beta=None, eps=1e-5):
        """LayerNorm(x @ W.T + b + residual) * gamma + beta: the post-LN step of a BERT layer, which the reference
        spells ``layer_norm(linear(attn_out) + x)`` (utils/vulkan_sentence_transformer.py:997-1011, 1018-1033). For
        128, 256, 384 or 512 output features it is one kernel (the statistics are taken in the GEMM's epilogue and
        the pre-norm sum never reaches memory); other widths run the GEMM and the LayerNorm kernel."""
        bf16 = self._bf16
        N, K = (int(s) for s in weights.shape)
        x_shape = tuple(x.shape)
        if x_shape[-1] != K:
            raise ValueError(f"input feature size {x_shape[-1]} does not match weights {tuple(weights.shape)}")
        if residual is not None and tuple(residual.shape) != x_shape[:-1] + (N,):
            raise ValueError(f"residual must have shape {x_shape[:-1] + (N,)}")
        for name, v in (("bias", bias), ("gamma", gamma), ("beta", beta)):
            if v is not None and int(np.prod(v.shape)) != N:
                raise ValueError(f"{name} has {int(np.prod(v.shape))} entries, expected {N}")
        elt = 2 if bf16 else 4
        kpad = (-K) % (16 // elt)
        w_transform, w_tag = None, ""
        if kpad:
            if isinstance(x, DeviceTensor):
                raise ValueError("device-resident operands need in_features * element size to be a multiple of 16 bytes")
            x = np.pad(np.asarray(x, dtype=np.float32).reshape(-1, K), ((0, 0), (0, kpad)))
            w_transform = lambda a: np.pad(np.asarray(a, dtype=np.float32), ((0, 0), (0, kpad)))  # noqa: E731
            w_tag = f"|kpad{kpad}"
        xd, host = self._act_in(x)
        wd = self.dev.weight(weights, "bf16" if bf16 else "f32", round_tf32=True, transform=w_transform, tag="w" + w_tag)
        rd = None
        if residual is not None:
            rd = residual if isinstance(residual, DeviceTensor) else self.dev.upload(residual, "bf16" if bf16 else "f32")
        M = xd.size // (K + kpad)
        y = self.dev.empty((M, N))
        scratch = self.dev.empty((M, N))
        self.dev.check(self.lib.grilly_linear_layernorm(self.ctx, _p(xd), _p(wd), _p(self._vec(bias)), _p(rd), _p(self._vec(gamma)),
                                                        _p(self._vec(beta)), _p(y), _p(scratch), M, N, K + kpad, float(eps),
                                                        L.PREC_BF16 if bf16 else L.PREC_TF32, 0))
        out = self._out(y, host, x_shape[:-1] + (N,))
        scratch.free()
        return out

    def _act_params(self, op, x, p0=0.0, p1=0.0):
        xd, host = self._act_in(x, mma_operand=False)
        y = self.dev.empty(tuple(x.shape))
        self.dev.check(self.lib.grilly_activation_params(self.ctx, op, _p(xd), _p(y), xd.size, float(p0), float(p1)))
        return self._out(y, host)

    def activation_gcu(self, input_data):
        """Growing cosine unit x * cos(x): backend/fnn.py:385-440."""
        return self._act_params(L.ELT_GCU, input_data)

    def activation_roswish(self, input_data, alpha=1.0, beta=1.0):
        """RoSwish (x + alpha) * sigmoid(beta * x) - alpha / 2: backend/fnn.py:442-497."""
        return self._act_params(L.ELT_ROSWISH, input_data, alpha, beta)

    def fused_linear_gcu(self, x, weights, bias=None, precision=None):
        """gcu(x @ W.T + b): backend/fnn.py:2307-2385 (fused-linear-gcu.glsl). The GEMM and the activation run back to
        back on the device (the GEMM's epilogue carries GELU, SiLU and ReLU; x cos x is applied to its result in place)."""
        return self._linear(x, weights, bias, L.ACT_NONE, precision=precision, post=(L.ELT_GCU, 0.0, 0.0))

    def fused_linear_roswish(self, x, weights, bias=None, alpha=1.0, beta=1.0, precision=None):
        """roswish(x @ W.T + b): backend/fnn.py:2387-2463 (fused-linear-roswish.glsl); GEMM then the activation in place."""
        return self._linear(x, weights, bias, L.ACT_NONE, precision=precision, post=(L.ELT_ROSWISH, alpha, beta))

    def fused_qkv_projection(self, x, w_qkv, b_qkv=None, num_heads=None, head_dim=None, precision=None):
        """x @ [Wq;Wk;Wv].T + [bq;bk;bv] -> (..., 3*H*D), column blocks Q, K, V: fused-qkv-projection.glsl:48-74."""
        if num_heads is not None and head_dim is not None and w_qkv.shape[0] != 3 * num_heads * head_dim:
            raise ValueError("stacked QKV weight must have 3 * num_heads * head_dim rows")
        return self._linear(x, w_qkv, b_qkv, L.ACT_NONE, precision=precision)

    def fused_swiglu(self, x, w_gate, w_up, b_gate=None, b_up=None):
        """(x Wg^T + bg) * silu(x Wu^T + bu) as ONE GEMM over row-interleaved [g0,u0,g1,u1,...] weights with a
        pairwise epilogue: backend/_glu_append.py:47-60, fused-swiglu.glsl:48-79."""
        return self._fused_glu(x, w_gate, w_up, b_gate, b_up, L.ACT_NONE, "swiglu")

    def fused_geglu(self, x, w_gate, w_up, b_gate=None, b_up=None):
        """(x Wg^T + bg) * gelu(x Wu^T + bu), tanh GELU, same single GEMM: backend/_glu_append.py:224-262,
        fused-geglu.glsl:53-84."""
        return self._fused_glu(x, w_gate, w_up, b_gate, b_up, L.ACT_GELU, "geglu")

    def _fused_glu(self, x, w_gate, w_up, b_gate, b_up, act, name):
        if tuple(w_gate.shape) != tuple(w_up.shape):
            raise ValueError("gate and up weights must have the same shape")
        n = int(w_gate.shape[0])
        up_host = np.asarray(w_up, dtype=np.float32)

        def interleave(g):
            out = np.empty((2 * n, g.shape[1]), dtype=np.float32)
            out[0::2] = np.asarray(g, dtype=np.float32)
            out[1::2] = up_host
            return out

        bias = None
        if b_gate is not None and b_up is not None:
            bias = np.empty(2 * n, dtype=np.float32)
            bias[0::2], bias[1::2] = np.asarray(b_gate, np.float32), np.asarray(b_up, np.float32)
        tag = f"|{name}{np.asarray(w_up).__array_interface__['data'][0]}"
        return self._linear(x, w_gate, bias, act, flags=L.FLAG_SWIGLU_PAIRS, w_tag=tag, w_transform=interleave,
                            n_out=n)

    def fused_layernorm_linear(self, x, gamma, beta, weights, bias=None, eps=1e-5, mode="layer"):
        """Linear(LayerNorm(x)) (or RMSNorm with mode='rms'): fused-layernorm-linear.glsl:67-128. One row-statistics
        kernel plus the GEMM on the raw rows with the normalisation finished in its epilogue; gamma/beta are folded
        into the weights once and cached (``invalidate(weights)`` after an in-place change). Rows whose mean is far
        from zero against their spread (|mean| > 1.5 std) are normalised first instead, so the result keeps the
        precision's tolerance for any input. Runs in the backend's precision (tf32 or bf16)."""
        bf16 = self._bf16
        N, K = (int(s) for s in weights.shape)
        x_shape = tuple(x.shape)
        if x_shape[-1] != K:
            raise ValueError(f"input feature size {x_shape[-1]} does not match weights {tuple(weights.shape)}")
        if K % (8 if bf16 else 4):
            raise ValueError("fused_layernorm_linear needs in_features * element size to be a multiple of 16 bytes")
        prec = L.PREC_BF16 if bf16 else L.PREC_TF32
        key = ("lnfold", id(weights), id(gamma), id(beta), id(bias), mode, prec)
        fold = self._b._folds.get(key)
        if fold is not None:
            self._b._folds.move_to_end(key)
        else:
            wd = self.dev.upload(np.asarray(weights, np.float32))
            gd = self.dev.upload(np.asarray(gamma, np.float32)) if gamma is not None else None
            bd = self.dev.upload(np.asarray(beta, np.float32)) if (beta is not None and mode == "layer") else None
            cd = self.dev.upload(np.asarray(bias, np.float32)) if bias is not None else None
            wf, cs, bf = self.dev.empty((N, K), "bf16" if bf16 else "f32"), self.dev.empty((N,)), self.dev.empty((N,))
            self.dev.check(self.lib.grilly_fold_layernorm_weights(self.ctx, _p(wd), _p(gd), _p(bd), _p(cd), _p(wf), _p(cs),
                                                                  _p(bf), N, K, prec))
            self.dev.sync()
            for t in (wd, gd, bd, cd):
                if t is not None:
                    t.free()
            fold = (wf, cs, bf, weights, gamma, beta, bias)  # keep the host arrays alive so ids stay unique
            self._b._folds[key] = fold
            while len(self._b._folds) > self._b.MAX_FOLDS:   # least recently used first
                self._b._folds.popitem(last=False)
        wf, cs, bf = fold[:3]
        if isinstance(x, DeviceTensor):
            xd, host = x, False
        else:
            xd, host = self.dev.upload(x, "bf16" if bf16 else "f32"), True   # raw rows: the statistics need them unrounded
        M = xd.size // K
        y = self.dev.empty((M, N))
        stats = self.dev.empty((2 * M,))
        self.dev.check(self.lib.grilly_layernorm_linear(self.ctx, _p(xd), _p(wf), _p(cs), _p(bf), _p(y), _p(stats), M, N, K,
                                                        float(eps), L.NORM_RMS if mode == "rms" else L.NORM_LAYER,
                                                        L.ACT_NONE, prec, 0))
        out = self._out(y, host, x_shape[:-1] + (N,))
        stats.free()
        return out

    def gemm(self, A, B, precision=None):
        """C = A @ B, row-major (M,K) x (K,N): backend/fnn.py:104-166, gemm_mnk.glsl:35-88."""
        if len(A.shape) != 2 or len(B.shape) != 2 or A.shape[1] != B.shape[0]:
            raise AssertionError(f"K mismatch: {tuple(A.shape)} @ {tuple(B.shape)}")  # the reference asserts (fnn.py:118)
        mode = self._mode(precision)
        M, K = (int(s) for s in A.shape)
        N = int(B.shape[1])
        q = 8 if mode == "bf16" else 4
        kpad, npad = (-K) % q, (-N) % q
        if (kpad or npad) and (isinstance(A, DeviceTensor) or isinstance(B, DeviceTensor)):
            raise ValueError("device-resident gemm operands need K and N to be multiples of 16 bytes")
        if kpad or npad:
            A = np.pad(np.asarray(A, np.float32), ((0, 0), (0, kpad)))
            B = np.pad(np.asarray(B, np.float32), ((0, kpad), (0, npad)))
        ad, host_a = self._act_in(A, mode=mode)
        bd, host_b = self._act_in(B, mode=mode)
        c = self.dev.empty((M, N + npad))
        self.dev.check(self.lib.grilly_gemm_mnk(self.ctx, _p(ad), _p(bd), _p(c), M, K + kpad, N + npad, _PREC[mode], 0))
        if host_a or host_b:
            out = c.numpy()
            return np.ascontiguousarray(out[:, :N]) if npad else out
        return c

    gemm_mnk = gemm

    # ---- normalisation ----------------------------------------------------------------------
    def linear_backward(self, grad_output, x, weights, bias=None):
        """(grad_input, grad_weight, grad_bias) of y = x W^T + b as three products on the tensor cores, the way the
        reference's GEMM branch does it (backend/fnn.py:1501-1573): grad_output @ W, grad_output^T @ x, and the
        column sums of grad_output as ones(1, rows) @ grad_output. Each operand is uploaded once; the transpose of
        grad_output is taken on the device. grad_bias is None when there is no bias."""
        go = np.asarray(grad_output, dtype=np.float32)
        xs = np.asarray(x, dtype=np.float32)
        w = np.asarray(weights, dtype=np.float32)
        if go.ndim not in (2, 3) or xs.ndim != go.ndim or go.shape[:-1] != xs.shape[:-1]:
            raise ValueError("grad_output (.., out) and x (.., in) must be 2-D or 3-D with the same leading shape")
        if w.shape != (go.shape[-1], xs.shape[-1]):
            raise ValueError(f"weights must have shape {(go.shape[-1], xs.shape[-1])}")
        go2, x2 = go.reshape(-1, go.shape[-1]), xs.reshape(-1, xs.shape[-1])
        rows, n_out, n_in = go2.shape[0], go2.shape[1], x2.shape[1]
        q = 8 if self._bf16 else 4
        if rows % q or n_out % q or n_in % q:
            # ragged sizes: the padded host path
            grad_input = self.gemm(go2, w).reshape(xs.shape)
            grad_weight = self.gemm(np.ascontiguousarray(go2.T), x2)
            grad_bias = self.gemm(np.ones((1, rows), np.float32), go2).reshape(-1) if bias is not None else None
            return grad_input, grad_weight, grad_bias
        god = self.dev.upload(go2)                       # raw fp32: rounded copies are made below
        got = self.dev.empty((n_out, rows))
        self.dev.check(self.lib.grilly_transpose_2d(self.ctx, _p(god), _p(got), rows, n_out))
        go_m, got_m = self.to_mma(god), self.to_mma(got)
        grad_input = self.gemm(go_m, self._b.to_device(w)).numpy().reshape(xs.shape)
        grad_weight = self.gemm(got_m, self._b.to_device(x2)).numpy()
        grad_bias = None
        if bias is not None:
            grad_bias = self.gemm(self._b.to_device(np.ones((1, rows), np.float32)), go_m).numpy().reshape(-1)
        return grad_input, grad_weight, grad_bias

    def to_mma(self, t: DeviceTensor) -> DeviceTensor:
        """A raw fp32 device tensor in the form the backend's MMAs consume: tf32-rounded fp32, or bf16."""
        out = self.dev.empty(t.shape, "bf16" if self._bf16 else "f32")
        if self._bf16:
            self.dev.check(self.lib.grilly_cast_f32_to_bf16(self.ctx, _p(t), _p(out), t.size))
        else:
            self.dev.check(self.lib.grilly_round_tf32(self.ctx, _p(t), _p(out), t.size))
        return out

    def layernorm_backward(self, grad_output, x, gamma, mean=None, var=None, eps=1e-5):
        """(grad_input, grad_gamma, grad_beta) of LayerNorm over the last dim: backend/fnn.py:1701-1847. ``mean`` and
        ``var`` are the forward pass's statistics (shape (..., 1) or (...)); computed when not given."""
        xs = np.asarray(x, dtype=np.float32)
        go = np.asarray(grad_output, dtype=np.float32)
        if go.shape != xs.shape:
            raise ValueError("grad_output and x must have the same shape")
        F = int(xs.shape[-1])
        rows = xs.size // F
        if gamma is not None and int(np.prod(np.shape(gamma))) != F:
            raise ValueError(f"gamma has {int(np.prod(np.shape(gamma)))} entries, expected {F}")
        xd, god = self.dev.upload(xs.reshape(rows, F)), self.dev.upload(go.reshape(rows, F))
        md = self.dev.upload(np.asarray(mean, np.float32).reshape(rows)) if mean is not None else None
        vd = self.dev.upload(np.asarray(var, np.float32).reshape(rows)) if var is not None else None
        gi, gg, gb = self.dev.empty((rows, F)), self.dev.empty((F,)), self.dev.empty((F,))
        self.dev.check(self.lib.grilly_layernorm_backward(self.ctx, _p(god), _p(xd), _p(self._vec(gamma)), _p(md), _p(vd), _p(gi),
                                                          _p(gg), _p(gb), rows, F, float(eps)))
        return gi.numpy().reshape(xs.shape), gg.numpy(), gb.numpy()

    def softmax_backward(self, grad_output, softmax_output, dim=-1):
        """softmax_output * (grad_output - sum(grad_output * softmax_output)) along ``dim``: backend/fnn.py:1849-1933."""
        go = np.asarray(grad_output, dtype=np.float32)
        y = np.asarray(softmax_output, dtype=np.float32)
        if go.shape != y.shape:
            raise ValueError("grad_output and softmax_output must have the same shape")
        ax = dim % go.ndim
        if ax != go.ndim - 1:
            moved = self.softmax_backward(np.ascontiguousarray(np.moveaxis(go, ax, -1)), np.ascontiguousarray(np.moveaxis(y, ax, -1)))
            return np.ascontiguousarray(np.moveaxis(moved, -1, ax))
        cols = int(go.shape[-1])
        god, yd = self.dev.upload(go), self.dev.upload(y)
        gi = self.dev.empty(go.shape)
        self.dev.check(self.lib.grilly_softmax_backward(self.ctx, _p(god), _p(yd), _p(gi), go.size // cols, cols))
        return gi.numpy()

    def _norm(self, x, gamma, beta, eps, mode, residual=None):
        x_shape = tuple(x.shape)
        F = int(x_shape[-1])
        xd, host = self._act_in(x, mma_operand=False)
        rd = None
        if residual is not None:
            rd, _ = self._act_in(residual, mma_operand=False)
        for name, v in (("gamma", gamma), ("beta", beta)):
            if v is not None and int(np.prod(v.shape)) != F:
                raise ValueError(f"{name} has {int(np.prod(v.shape))} entries, expected {F}")
        rows = xd.size // F
        y = self.dev.empty((rows, F))
        self.dev.check(self.lib.grilly_layernorm(self.ctx, _p(xd), _p(rd), _p(self._vec(gamma)), _p(self._vec(beta)), _p(y),
                                                 rows, F, float(eps), mode, 0))
        return self._out(y, host, x_shape)

    def layernorm(self, x, gamma=None, beta=None, eps=1e-5):
        """gamma (x - mean) / sqrt(var + eps) + beta over the last dim: backend/fnn.py:1285-1389."""
        return self._norm(x, gamma, beta, eps, L.NORM_LAYER)

    def rmsnorm(self, x, gamma=None, eps=1e-5):
        """x / sqrt(mean(x^2) + eps) * gamma: snn-rmsnorm.glsl:34-75."""
        return self._norm(x, gamma, None, eps, L.NORM_RMS)

    def residual_layernorm(self, x, module_output, gamma=None, beta=None, eps=1e-5):
        """LayerNorm(x + module_output) in one pass (the post-LN step of utils/vulkan_sentence_transformer.py:1004)."""
        return self._norm(x, gamma, beta, eps, L.NORM_LAYER, residual=module_output)

    # ---- activations ------------------------------------------------------------------------
    def _eltwise(self, op, a, b=None, half=0):
        shape = tuple(a.shape)
        ad, host = self._act_in(a, mma_operand=False)
        bd = None
        if b is not None:
            if tuple(b.shape) != shape:
                raise ValueError(f"shape mismatch: {shape} vs {tuple(b.shape)}")
            bd, _ = self._act_in(b, mma_operand=False)
        out_shape = shape if op != L.ELT_SWIGLU else shape[:-1] + (half,)
        y = self.dev.empty(out_shape)
        self.dev.check(self.lib.grilly_eltwise(self.ctx, op, _p(ad), _p(bd), _p(y), y.size, half))
        return self._out(y, host)

    def activation_gelu(self, input_data):
        """tanh-approximation GELU: backend/fnn.py:285-342."""
        return self._eltwise(L.ELT_GELU, input_data)

    def activation_silu(self, input_data):
        """x * sigmoid(x): backend/fnn.py:344-400."""
        return self._eltwise(L.ELT_SILU, input_data)

    def activation_relu(self, input_data):
        """max(0, x): backend/fnn.py:232-283."""
        return self._eltwise(L.ELT_RELU, input_data)

    def activation_swiglu(self, input_data):
        """x1 * silu(x2) on halves of the last dim: backend/fnn.py:499-572."""
        if input_data.shape[-1] % 2:
            raise ValueError("SwiGLU needs an even last dimension")
        return self._eltwise(L.ELT_SWIGLU, input_data, half=int(input_data.shape[-1]) // 2)

    swiglu = activation_swiglu  # the name the reference's README uses (README.md:108)

    def activation_softmax(self, input_data, axis=-1):
        """softmax over ``axis``: backend/fnn.py:574-663."""
        nd = len(input_data.shape)
        ax = axis % nd
        if ax != nd - 1:
            if isinstance(input_data, DeviceTensor):
                raise ValueError("device-resident softmax runs over the last axis only")
            moved = np.moveaxis(np.asarray(input_data, np.float32), ax, -1)
            return np.ascontiguousarray(np.moveaxis(self.activation_softmax(np.ascontiguousarray(moved)), -1, ax))
        shape = tuple(input_data.shape)
        xd, host = self._act_in(input_data, mma_operand=False)
        y = self.dev.empty(shape)
        cols = int(shape[-1])
        self.dev.check(self.lib.grilly_softmax(self.ctx, _p(xd), _p(y), xd.size // cols, cols))
        return self._out(y, host)

    def residual(self, x, module_output):
        """x + module_output: backend/fnn.py:1950-2014."""
        return self._eltwise(L.ELT_ADD, x, module_output)


class Attention(_Namespace):
    """backend/attention.py ``VulkanAttention``."""

    architecture = None

    def flash_attention2(self, queries, keys, values, num_heads=None, head_dim=None, tile_size_q=64, tile_size_k=64,
                         scale=None, mask=None, causal=False, use_rope=False, rope_base=10000.0, rope_scaling=1.0,
                         rope_style="interleaved"):
        """softmax(scale Q K^T + mask) V on (B, S, H, D) or (B, S, H*D) inputs: backend/attention.py:361-597.

        ``mask`` is a (B, S) key-padding mask, 1 = keep. ``causal`` masks keys after the query. ``tile_size_*`` are
        accepted for signature compatibility; the kernel tiles 128 x 128. With ``use_rope`` the scores are taken
        on rotated q, k (flash-attention2-rope.glsl; ``rope_style`` 'interleaved' or 'rotate_half')."""
        shape = tuple(queries.shape)
        if len(shape) == 4:
            B, S, H, D = (int(s) for s in shape)  # a 4-D input's own shape wins (attention.py:410)
        elif len(shape) == 3:
            if num_heads is None or head_dim is None:
                raise ValueError("3-D inputs need num_heads and head_dim")
            B, S, _ = (int(s) for s in shape)
            H, D = int(num_heads), int(head_dim)
            if shape[2] != H * D:
                raise ValueError(f"last dimension {shape[2]} != num_heads * head_dim = {H * D}")
        else:
            raise ValueError("queries must be (B, S, H, D) or (B, S, H*D)")
        if tuple(keys.shape) != shape or tuple(values.shape) != shape:
            raise ValueError("queries, keys and values must have the same shape")
        if mask is not None and tuple(mask.shape) != (B, S):
            raise ValueError(f"mask must have shape {(B, S)}")
        if self._b.precision == "tf32x3":
            return self._attention_fp32(queries, keys, values, B, S, H, D, scale, mask, causal, use_rope, rope_base,
                                        rope_scaling, rope_style)
        qd, host = self._act_in(queries)
        kd, _ = self._act_in(keys)
        vd, _ = self._act_in(values)
        md = None
        if mask is not None:
            md, _ = self._act_in(np.asarray(mask, dtype=np.float32) if not isinstance(mask, DeviceTensor) else mask,
                                 mma_operand=False)
        rope = L.ROPE_NONE
        if use_rope:
            if rope_style not in ("interleaved", "rotate_half"):
                raise ValueError("rope_style must be 'interleaved' or 'rotate_half'")
            rope = L.ROPE_INTERLEAVED if rope_style == "interleaved" else L.ROPE_ROTATE_HALF
        sc = float(scale) if scale is not None else 1.0 / math.sqrt(D)
        Dk = self._kernel_head_dim(D, S, bool(causal) or rope != L.ROPE_NONE)
        if Dk != D:
            # a head dim between the kernels' sizes runs zero-padded: zero columns of q, k add nothing to a score and
            # zero columns of v give output columns that are dropped again (all on the device)
            if rope != L.ROPE_NONE:
                raise ValueError(f"use_rope needs head_dim in {self._head_dims(S, True)} ({self._b.precision} mode)")
            qd, kd, vd = (self._pad_heads(t, B * S * H, D, Dk) for t in (qd, kd, vd))
        out = self.dev.empty((B, S, H, Dk))
        self.dev.check(self.lib.grilly_flash_attention(
            self.ctx, _p(qd), _p(kd), _p(vd), _p(out), B, S, H, Dk, H * Dk, H * Dk, None, B * S, _p(md), sc, int(bool(causal)),
            rope, float(rope_base), float(rope_scaling), L.PREC_BF16 if self._bf16 else L.PREC_TF32, 0))
        if Dk != D:
            out = self._pad_heads(out, B * S * H, Dk, D)
        return self._out(out, host, (B, S, H, D))

    def _head_dims(self, S: int, general: bool):
        """Head dims the attention kernels are instantiated for."""
        if not self._bf16:
            return (32, 64, 96, 128)
        return (64, 128) if (general or S > 128) else (32, 64, 128)

    def _kernel_head_dim(self, D: int, S: int, general: bool) -> int:
        for d in self._head_dims(S, general):
            if D <= d:
                return d
        raise ValueError(f"head_dim {D} exceeds 128")

    def _pad_heads(self, t: DeviceTensor, rows: int, d_from: int, d_to: int) -> DeviceTensor:
        """(rows, d_from) -> (rows, d_to) on the device: zero-padded when d_to > d_from, cut when smaller."""
        elt = 2 if t.dtype == "bf16" else 4
        out = self.dev.empty((rows, d_to), t.dtype)
        if d_to > d_from:
            self.dev.check(self.lib.grilly_memset(self.ctx, _p(out), 0, rows * d_to * elt))
        self.dev.check(self.lib.grilly_copy_2d(self.ctx, _p(out), d_to * elt, _p(t), d_from * elt, min(d_from, d_to) * elt, rows))
        return out

    def _attention_fp32(self, queries, keys, values, B, S, H, D, scale, mask, causal, use_rope, rope_base, rope_scaling,
                        rope_style):
        """The exact-index mode of a 'tf32x3' backend: the same attention from the fp32 FMA kernels of the unfused
        pipeline (scores, mask, softmax, output; every product and sum in fp32, no tensor-core rounding), all on the
        device. It materialises the (B, H, S, S) scores, so it is meant for checking indices, not for long sequences."""
        if use_rope and rope_style not in ("interleaved", "rotate_half"):
            raise ValueError("rope_style must be 'interleaved' or 'rotate_half'")
        qd, host = self._act_in(queries, mma_operand=False)
        kd, _ = self._act_in(keys, mma_operand=False)
        vd, _ = self._act_in(values, mma_operand=False)
        if use_rope:
            style = L.ROPE_INTERLEAVED if rope_style == "interleaved" else L.ROPE_ROTATE_HALF
            qr, kr = self.dev.empty((B, S, H, D)), self.dev.empty((B, S, H, D))
            for src, dst in ((qd, qr), (kd, kr)):
                self.dev.check(self.lib.grilly_apply_rope(self.ctx, _p(src), _p(dst), None, B, S, H, D, S, float(rope_base),
                                                          float(rope_scaling), style))
            qd, kd = qr, kr
        sc = float(scale) if scale is not None else 1.0 / math.sqrt(D)
        scores = self.dev.empty((B, H, S, S))
        self.dev.check(self.lib.grilly_attention_scores(self.ctx, _p(qd), _p(kd), _p(scores), B, S, H, D, sc))
        if causal:
            self.dev.check(self.lib.grilly_attention_mask(self.ctx, _p(scores), None, B, H, S, 1, -1e9))
        if mask is not None:
            md, _ = self._act_in(np.asarray(mask, dtype=np.float32) if not isinstance(mask, DeviceTensor) else mask,
                                 mma_operand=False)
            self.dev.check(self.lib.grilly_attention_mask(self.ctx, _p(scores), _p(md), B, H, S, 0, -1e9))
        self.dev.check(self.lib.grilly_softmax(self.ctx, _p(scores), _p(scores), B * H * S, S))
        out = self.dev.empty((B, S, H, D))
        self.dev.check(self.lib.grilly_attention_output(self.ctx, _p(scores), _p(vd), _p(out), B, S, H, D))
        return self._out(out, host)

    def flash_attention2_rope(self, queries, keys, values, num_heads=None, head_dim=None, scale=None, mask=None,
                              causal=False, rope_base=10000.0, rope_scaling=1.0, rope_style="interleaved"):
        """flash-attention2-rope.glsl:74-149,165-247 (the reference ships the shader without a Python wrapper)."""
        return self.flash_attention2(queries, keys, values, num_heads, head_dim, scale=scale, mask=mask, causal=causal,
                                     use_rope=True, rope_base=rope_base, rope_scaling=rope_scaling, rope_style=rope_style)

    def apply_rope(self, q_or_k, position_ids=None, rope_base=10000.0, rope_scaling=1.0):
        """Rotate-half RoPE on (B, S, H, D): backend/attention.py:599-676, rope.glsl:52-126."""
        shape = tuple(q_or_k.shape)
        if len(shape) != 4 or shape[-1] % 2:
            raise ValueError("apply_rope expects (B, S, H, D) with an even D")
        B, S, H, D = (int(s) for s in shape)
        xd, host = self._act_in(q_or_k, mma_operand=False)
        pid, max_pos = None, S
        if position_ids is not None:
            ph = np.ascontiguousarray(position_ids, dtype=np.int32)
            if ph.shape != (B, S):
                raise ValueError(f"position_ids must have shape {(B, S)}")
            if ph.min() < 0:
                raise ValueError("position_ids must be non-negative")
            max_pos = int(ph.max()) + 1
            pid = self.dev.upload(ph, "i32")
        y = self.dev.empty(shape)
        self.dev.check(self.lib.grilly_apply_rope(self.ctx, _p(xd), _p(y), _p(pid), B, S, H, D, max_pos, float(rope_base),
                                                  float(rope_scaling), L.ROPE_ROTATE_HALF))
        return self._out(y, host)

    # ---- the unfused pipeline (what VulkanSentenceTransformer._attention_gpu calls): kept for drop-in use;
    #      flash_attention2 computes the same result without the (B,H,S,S) tensor
    def _bshd(self, t, num_heads, head_dim):
        shape = tuple(t.shape)
        if len(shape) == 4:
            return tuple(int(s) for s in shape)
        if len(shape) == 3 and shape[2] == num_heads * head_dim:
            return int(shape[0]), int(shape[1]), int(num_heads), int(head_dim)
        raise ValueError("expected (B, S, H, D) or (B, S, H*D)")

    def attention_scores(self, queries, keys, num_heads, head_dim, scale=None):
        """scale * Q K^T -> (B, H, S, S): backend/attention.py:41-126."""
        B, S, H, D = self._bshd(queries, num_heads, head_dim)
        if tuple(keys.shape) != tuple(queries.shape):
            raise ValueError("queries and keys must have the same shape")
        qd, host = self._act_in(queries, mma_operand=False)
        kd, _ = self._act_in(keys, mma_operand=False)
        out = self.dev.empty((B, H, S, S))
        sc = float(scale) if scale is not None else 1.0 / math.sqrt(D)
        self.dev.check(self.lib.grilly_attention_scores(self.ctx, _p(qd), _p(kd), _p(out), B, S, H, D, sc))
        return self._out(out, host)

    def attention_mask(self, attention_scores, use_causal=True, mask_value=-1e9, custom_mask=None):
        """Causal or key-padding mask on (B, H, S, S) scores: backend/attention.py:128-203."""
        shape = tuple(int(s) for s in attention_scores.shape)
        if len(shape) != 4 or shape[2] != shape[3]:
            raise ValueError("attention_scores must be (B, H, S, S)")
        B, H, S, _ = shape
        if not use_causal and custom_mask is None:
            return np.asarray(attention_scores, dtype=np.float32) if not isinstance(attention_scores, DeviceTensor) else attention_scores
        if isinstance(attention_scores, DeviceTensor):
            sd, host = attention_scores, False
        else:
            sd, host = self.dev.upload(np.asarray(attention_scores, np.float32)), True
        md = None
        if not use_causal:
            if tuple(custom_mask.shape) != (B, S):
                raise ValueError(f"custom_mask must have shape {(B, S)}")
            md, _ = self._act_in(np.asarray(custom_mask, np.float32) if not isinstance(custom_mask, DeviceTensor) else custom_mask,
                                 mma_operand=False)
        self.dev.check(self.lib.grilly_attention_mask(self.ctx, _p(sd), _p(md), B, H, S, int(bool(use_causal)), float(mask_value)))
        return self._out(sd, host)

    def attention_output(self, attention_weights, values, num_heads, head_dim):
        """weights @ V -> (B, Sq, H, D): backend/attention.py:205-300. As the reference picks a shader by the backend's
        architecture (backend/attention.py:226-229, backend/shader_registry.py:154-156), 'gpt' / 'granite' sum the keys
        k <= q only (attention-output-gpt.glsl) and 't5' takes weights (B, H, Sq, Sk) over encoder values
        (B, Sk, H, D) (attention-output-t5.glsl); every other architecture is the square bidirectional form."""
        wshape = tuple(int(s) for s in attention_weights.shape)
        if len(wshape) != 4:
            raise ValueError("attention_weights must be (B, H, S, S)")
        B, H, Sq, Sk = wshape
        arch = (self.architecture or "").lower()
        if arch != "t5" and Sq != Sk:
            raise ValueError("attention_weights must be (B, H, S, S)")
        vB, vS, vH, D = self._bshd(values, num_heads, head_dim)
        if (vB, vS, vH) != (B, Sk, H):
            raise ValueError("values do not match the attention weights")
        wd, host = self._act_in(attention_weights, mma_operand=False)
        vd, _ = self._act_in(values, mma_operand=False)
        out = self.dev.empty((B, Sq, H, D))
        causal = int(arch in ("gpt", "granite"))
        self.dev.check(self.lib.grilly_attention_output_ex(self.ctx, _p(wd), _p(vd), _p(out), B, Sq, Sk, H, D, causal))
        return self._out(out, host)

    def attention_backward(self, grad_output, q, k, v, attn_weights, scale):
        """(grad_q, grad_k, grad_v) of out = attn_weights @ v with attn_weights = softmax(scale q k^T): tensors in the
        (B, H, S, D) layout and attn_weights (B, H, S, S), as backend/autograd_core.py:609-646 takes them
        (shaders/attention-backward.glsl)."""
        go, qs, ks, vs = (np.asarray(t, dtype=np.float32) for t in (grad_output, q, k, v))
        aw = np.asarray(attn_weights, dtype=np.float32)
        if qs.ndim != 4 or ks.shape != qs.shape or vs.shape != qs.shape or go.shape != qs.shape:
            raise ValueError("grad_output, q, k, v must all be (B, H, S, D)")
        B, H, S, D = (int(s) for s in qs.shape)
        if aw.shape != (B, H, S, S):
            raise ValueError(f"attn_weights must have shape {(B, H, S, S)}")
        up = self.dev.upload
        god, qd, kd, vd, ad = up(go), up(qs), up(ks), up(vs), up(aw)
        gq, gk, gv = self.dev.empty(qs.shape), self.dev.empty(qs.shape), self.dev.empty(qs.shape)
        self.dev.check(self.lib.grilly_attention_backward(self.ctx, _p(god), _p(qd), _p(kd), _p(vd), _p(ad), _p(gq), _p(gk), _p(gv),
                                                          B, H, S, D, float(scale)))
        return gq.numpy(), gk.numpy(), gv.numpy()

    def attention_concat_heads(self, attention_output):
        """(B, S, H, D) -> (B, S, H*D): backend/attention.py:302-359 (a reshape in this layout)."""
        B, S, H, D = (int(s) for s in attention_output.shape)
        return attention_output.reshape(B, S, H * D)


class Pooling(_Namespace):
    """backend/pooling.py ``VulkanPooling`` (sequence pooling only)."""

    def _pool(self, embeddings, mask, normalize):
        shape = tuple(embeddings.shape)
        if len(shape) != 3:
            raise ValueError("embeddings must be (batch, seq_len, dim)")
        B, S, F = (int(s) for s in shape)
        if mask is not None and tuple(mask.shape) != (B, S):
            raise ValueError(f"mask must have shape {(B, S)}")
        xd, host = self._act_in(embeddings, mma_operand=False)
        md = None
        if mask is not None:
            md, _ = self._act_in(np.asarray(mask, np.float32) if not isinstance(mask, DeviceTensor) else mask, mma_operand=False)
        out = self.dev.empty((B, F))
        self.dev.check(self.lib.grilly_mean_pool(self.ctx, _p(xd), _p(md), None, _p(out), B, S, F, int(normalize)))
        return self._out(out, host)

    def mean_pool(self, embeddings, mask=None):
        """Masked mean over the sequence axis (mask > 0.5 counts; zero vector when nothing counts):
        backend/pooling.py:22-142, embedding-pool.glsl:61-81."""
        return self._pool(embeddings, mask, False)

    def mean_pool_normalize(self, embeddings, mask=None):
        """mean_pool followed by x / (||x|| + 1e-8) (functional/embedding.py:42-68) in the same kernel."""
        return self._pool(embeddings, mask, True)


class Learning(_Namespace):
    """backend/learning.py ``VulkanLearning`` (embedding lookup only)."""

    def embedding_lookup(self, token_ids, embedding_table):
        """Row gather; ids outside the table give zero rows: backend/learning.py:811-877."""
        if len(embedding_table.shape) != 2:
            raise ValueError("embedding_table must be (vocab, dim)")
        V, F = (int(s) for s in embedding_table.shape)
        ids = np.ascontiguousarray(token_ids, dtype=np.int64)
        ids32 = np.where((ids < 0) | (ids >= V), -1, ids).astype(np.int32)
        idd = self.dev.upload(ids32, "i32")
        td = self.dev.weight(embedding_table, "f32", round_tf32=False, tag="table")
        out = self.dev.empty(tuple(ids.shape) + (F,))
        self.dev.check(self.lib.grilly_embedding_lookup(self.ctx, _p(idd), _p(td), _p(out), ids.size, V, F))
        return out.numpy()


    def adam_update(self, weights, gradients, moment1, moment2, learning_rate, beta1=0.9, beta2=0.999, epsilon=1e-8,
                    beta1_t=0.0, beta2_t=0.0, clear_grad=False):
        """One Adam step: (updated_weights, updated_moment1, updated_moment2), new arrays of the inputs' shape
        (backend/learning.py:967-1077, adam-update.glsl). ``beta1_t`` / ``beta2_t`` are beta^t for the bias
        correction. ``clear_grad`` is accepted for signature compatibility: the caller's gradient array is a host
        array and is left as it is, as on the reference's GPU branch."""
        w = np.asarray(weights, dtype=np.float32)
        arrs = [np.asarray(a, dtype=np.float32) for a in (gradients, moment1, moment2)]
        if any(a.size != w.size for a in arrs):
            raise ValueError("All arrays must have the same size")
        wd, gd, m1, m2 = (self.dev.upload(a.reshape(-1)) for a in (w, *arrs))
        self.dev.check(self.lib.grilly_adam_update(self.ctx, _p(wd), _p(gd), _p(m1), _p(m2), w.size, float(learning_rate), float(beta1),
                                                   float(beta2), float(epsilon), float(beta1_t), float(beta2_t), int(bool(clear_grad))))
        return wd.numpy().reshape(w.shape), m1.numpy().reshape(w.shape), m2.numpy().reshape(w.shape)


class Faiss(_Namespace):
    """backend/faiss.py ``VulkanFAISS``: pairwise distances and exact top-k selection."""

    _TYPES = {"l2": L.DIST_L2, "cosine": L.DIST_COSINE, "dot": L.DIST_DOT}

    def compute_distances(self, queries, database, distance_type="cosine"):
        """(num_queries, num_database) distances: 'l2' sqrt(sum (q-d)^2), 'cosine' 1 - q.d/(|q||d| + 1e-8), 'dot'
        -(q.d); an unknown name means cosine, as in the reference (backend/faiss.py:25-104, faiss-distance.glsl:29-83).
        The dot products run on the tensor cores over tf32 hi/lo splits, so they carry fp32 accuracy. A NumPy
        database is cached on the device like a weight (``backend.invalidate(database)`` after an in-place change)."""
        if not isinstance(queries, DeviceTensor):
            queries = np.asarray(queries, dtype=np.float32)
            if queries.ndim == 1:
                queries = queries.reshape(1, -1)
        if len(queries.shape) != 2 or len(database.shape) != 2:
            raise ValueError("queries must be (num_queries, dim) or (dim,), database (num_database, dim)")
        nq, dim = (int(s) for s in queries.shape)
        ndb, dim_db = (int(s) for s in database.shape)
        if dim != dim_db:
            raise ValueError(f"dimension mismatch: queries have {dim}, database has {dim_db}")
        qd, host = self._act_in(queries, mma_operand=False)
        dd = self.dev.weight(database, "f32", round_tf32=False, tag="faiss-db")
        out = self.dev.empty((nq, ndb))
        code = self._TYPES.get(distance_type, L.DIST_COSINE)
        self.dev.check(self.lib.grilly_faiss_distances(self.ctx, _p(qd), _p(dd), _p(out), nq, ndb, dim, code))
        return self._out(out, host)

    def search(self, queries, database, k, distance_type="cosine"):
        """``topk(compute_distances(queries, database, distance_type), k)`` in one call that never materialises the
        (num_queries, num_database) matrix: the database is walked in L2-sized chunks, each reduced to its k best at
        once. Returns (indices uint32, distances fp32), each (num_queries, k), identical to the two-call form."""
        if not isinstance(queries, DeviceTensor):
            queries = np.asarray(queries, dtype=np.float32)
            if queries.ndim == 1:
                queries = queries.reshape(1, -1)
        if len(queries.shape) != 2 or len(database.shape) != 2:
            raise ValueError("queries must be (num_queries, dim) or (dim,), database (num_database, dim)")
        nq, dim = (int(s) for s in queries.shape)
        ndb, dim_db = (int(s) for s in database.shape)
        if dim != dim_db:
            raise ValueError(f"dimension mismatch: queries have {dim}, database has {dim_db}")
        k = min(int(k), ndb)
        if k <= 0:
            raise ValueError("k must be positive")
        qd, _ = self._act_in(queries, mma_operand=False)
        dd = self.dev.weight(database, "f32", round_tf32=False, tag="faiss-db")
        idx, val = self.dev.empty((nq, k), "i32"), self.dev.empty((nq, k))
        code = self._TYPES.get(distance_type, L.DIST_COSINE)
        self.dev.check(self.lib.grilly_faiss_search(self.ctx, _p(qd), _p(dd), nq, ndb, dim, k, code, _p(idx), _p(val)))
        return idx.numpy().view(np.uint32), val.numpy()

    def topk(self, distances, k):
        """(indices uint32, distances fp32), each (num_queries, k): the k smallest entries of every row in ascending
        order, ties by ascending index (backend/faiss.py:106-195). k is clipped to the row length as in the
        reference; k above 1024 is not supported on the device."""
        if not isinstance(distances, DeviceTensor):
            distances = np.asarray(distances, dtype=np.float32)
            if distances.ndim == 1:
                distances = distances.reshape(1, -1)
        if len(distances.shape) != 2:
            raise ValueError("distances must be (num_queries, num_database)")
        nq, ndb = (int(s) for s in distances.shape)
        k = min(int(k), ndb)
        if k <= 0:
            raise ValueError("k must be positive")
        dd, _ = self._act_in(distances, mma_operand=False)
        idx = self.dev.empty((nq, k), "i32")
        val = self.dev.empty((nq, k))
        self.dev.check(self.lib.grilly_faiss_topk(self.ctx, _p(dd), nq, ndb, k, _p(idx), _p(val)))
        return idx.numpy().view(np.uint32), val.numpy()


class _PoolView:
    """``backend.fnn.buffer_pool.get_stats()`` (tutorials/06_transformer_components.py:142-145)."""

    def __init__(self, dev: Device):
        self._dev = dev

    def get_stats(self) -> dict:
        """The keys ``BufferPool.get_stats`` returns (backend/buffer_pool.py:627-640): a *hit* is an acquire the pool
        served from memory it already held, ``allocations`` counts the acquires that made the pool grow (= misses),
        ``total_pooled_memory`` is what the pool holds beyond the live buffers. The stream-ordered pool has no size
        buckets and never evicts (release threshold = unlimited). The native counters follow under their own names."""
        return reference_pool_stats(self._dev.pool_stats())


def reference_pool_stats(native: dict) -> dict:
    """Maps the library's pool counters to the reference's ``get_stats`` dictionary (plus the native ones)."""
    acquired, hits = int(native.get("acquired", 0)), int(native.get("pool_hits", 0))
    misses = max(acquired - hits, 0)
    stats = {
        "hits": hits, "misses": misses, "allocations": misses, "evictions": 0,
        "total_acquired": acquired, "total_released": int(native.get("released", 0)),
        "total_pooled_memory": max(int(native.get("pool_reserved_bytes", 0)) - int(native.get("bytes_in_use", 0)), 0),
        "buckets": {}, "hit_rate": hits / max(1, hits + misses), "vma_enabled": False,
    }
    stats.update({k: v for k, v in native.items() if k not in stats})
    return stats


class _CoreView:
    """What callers read from ``backend.core`` (backend/core.py:14-439) without touching Vulkan: the table of available
    shaders, by the reference's shader names (``nn.Linear.forward`` takes its GEMM path when 'gemm_mnk' is listed,
    nn/modules.py:146-152), and the device name. There are no Vulkan handles behind it."""

    SHADERS = ("fnn-linear", "fused-linear-gelu", "fused-linear-relu", "fused-linear-silu", "fused-linear-gcu",
               "fused-linear-roswish", "fused-qkv-projection", "fused-layernorm-linear", "fused-swiglu", "fused-geglu",
               "gemm_mnk", "fnn-layernorm", "snn-rmsnorm", "fnn-residual", "activation-gelu", "activation-silu",
               "activation-relu", "activation-softmax", "activation-swiglu", "activation-gcu", "activation-roswish",
               "flash-attention2", "flash-attention2-rope", "rope", "attention-scores", "attention-mask",
               "attention-output", "attention-output-gpt", "attention-output-t5", "attention-backward",
               "embedding-lookup", "embedding-pool", "faiss-distance", "faiss-topk", "fnn-linear-backward",
               "fnn-layernorm-backward", "activation-softmax-backward", "adam-update")

    def __init__(self, device):
        self.shaders = {name: b"" for name in self.SHADERS}
        self.device_name = "NVIDIA B200 (sm_100a), device %d" % device.index


class Compute:
    """Drop-in for ``grilly.Compute()`` (``VulkanCompute``, backend/compute.py:23-128) on one B200.

    precision: 'tf32' (fp32 storage, tf32 tensor-core products, fp32 accumulate), 'bf16', or 'tf32x3': like 'tf32',
    but linear / fused_linear_* / fused_qkv_projection / gemm split every operand into tf32 hi + lo and run three
    products, which gives fp32-level results -- the mode for callers that compare argmax / top-k indices with an fp32
    implementation (tf32 alone cannot order values closer than its rounding noise).
    """

    def __init__(self, shader_dir=None, device: int = 0, precision: str = "tf32"):
        if precision not in ("tf32", "bf16", "tf32x3"):
            raise ValueError("precision must be 'tf32', 'bf16' or 'tf32x3'")
        self.precision = precision
        self.device = Device(device)
        self.architecture = None
        self._folds: OrderedDict = OrderedDict()   # folded LayerNorm->linear weights, least recently used first
        self.fnn = FNN(self)
        self.attention = Attention(self)
        self.pooling = Pooling(self)
        self.learning = Learning(self)
        self.faiss = Faiss(self)
        self.core = _CoreView(self.device)
        self._alias()

    def _alias(self):
        # flat aliases the reference exposes (backend/compute.py:99,116-128,153-195,324-326)
        f = self.fnn
        for name in ("linear", "layernorm", "residual", "activation_relu", "activation_gelu", "activation_silu",
                     "activation_swiglu", "activation_softmax", "fused_linear_gelu", "fused_linear_relu",
                     "fused_linear_silu", "gemm"):
            setattr(self, name, getattr(f, name))
        self.flash_attention2 = self.attention.flash_attention2
        self.apply_rope = self.attention.apply_rope
        self.mean_pool = self.pooling.mean_pool
        self.embedding_lookup = self.learning.embedding_lookup
        self.faiss_compute_distances = self.faiss.compute_distances   # backend/compute.py:143-150
        self.faiss_topk = self.faiss.topk
        self.faiss_search = self.faiss.search

    def set_architecture(self, architecture: str):
        """backend/compute.py:70-128: selects the form of ``attention.attention_output`` ('gpt' / 'granite' causal,
        't5' decoder-over-encoder); everything else takes causal masking as a flag."""
        self.architecture = architecture
        self.attention.architecture = architecture

    def to_device(self, arr, mma_operand: bool = True) -> DeviceTensor:
        """Stage an array on the GPU once; ops given DeviceTensors return DeviceTensors."""
        if self.precision == "bf16" and mma_operand:
            return self.device.upload(arr, "bf16")
        return self.device.upload(arr, "f32", round_tf32=mma_operand and self.precision != "tf32x3")

    MAX_FOLDS = 32

    def register_weight(self, arr):
        """Keep ``arr``'s device copies cached for the backend's lifetime (see :meth:`Device.register_weight`)."""
        self.device.register_weight(arr)

    def invalidate(self, arr=None):
        """Forget cached device copies of a weight that was modified in place (all weights if None), including the
        folded LayerNorm->linear weights that were built from it (as weights, gamma, beta or bias)."""
        self.device.invalidate(arr)
        if arr is None:
            self._folds.clear()
            return
        ptr = np.asarray(arr).__array_interface__["data"][0]

        def same(h):
            return h is not None and (h is arr or np.asarray(h).__array_interface__["data"][0] == ptr)

        for k in [k for k, f in self._folds.items() if any(same(h) for h in f[3:])]:
            del self._folds[k]

    def synchronize(self):
        self.device.sync()

    def cleanup(self):
        """backend/compute.py:56-68."""
        self._folds.clear()
        self.device.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.cleanup()
