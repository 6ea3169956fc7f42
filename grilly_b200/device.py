"""Device context, device tensors and the persistent weight cache.

Replaces the reference's ``VulkanCore`` buffer plumbing (backend/core.py:304-360)
and ``BufferPool`` (backend/buffer_pool.py:466-651): allocations come from the
library's stream-ordered ``cudaMallocAsync`` pool, weights stay on the device
between calls instead of being re-uploaded (backend/fnn.py:1437-1489 uploads W
on every call).
"""
from __future__ import annotations

import ctypes as C
import weakref

import numpy as np

from . import _lib as L


class DeviceTensor:
    """A contiguous array in device memory. dtype is 'f32', 'bf16' or 'i32'."""

    __slots__ = ("dev", "ptr", "shape", "dtype", "_owned", "__weakref__")
    _ITEMSIZE = {"f32": 4, "bf16": 2, "i32": 4}

    def __init__(self, dev: "Device", ptr: int, shape, dtype: str, owned: bool = True):
        self.dev, self.ptr, self.shape, self.dtype, self._owned = dev, ptr, tuple(int(s) for s in shape), dtype, owned

    @property
    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        return self.size * self._ITEMSIZE[self.dtype]

    def reshape(self, *shape) -> "DeviceTensor":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = list(shape)
        if -1 in shape:
            known = 1
            for s in shape:
                if s != -1:
                    known *= s
            shape[shape.index(-1)] = self.size // max(known, 1)
        t = DeviceTensor(self.dev, self.ptr, shape, self.dtype, owned=False)
        if t.size != self.size:
            raise ValueError(f"cannot reshape {self.shape} to {tuple(shape)}")
        # a view keeps its base alive
        object.__setattr__(t, "_owned", self)
        return t

    def numpy(self) -> np.ndarray:
        return self.dev.download(self)

    def free(self) -> None:
        if self._owned is True and self.ptr:
            self.dev.free_ptr(self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Device:
    """One context per (process, GPU): stream, memory pool, launch counter."""

    def __init__(self, index: int = 0):
        self.lib = L.load()
        n = C.c_int(0)
        rc = self.lib.grilly_device_count(C.byref(n))
        if rc != L.OK or n.value == 0:
            raise RuntimeError("grilly_b200: no CUDA device available (this package has no CPU fallback)")
        h = C.c_void_p()
        rc = self.lib.grilly_init(index, C.byref(h))
        if rc == L.ERR_UNSUPPORTED:
            raise RuntimeError("grilly_b200: the kernels are built for sm_100a (B200) only")
        if rc != L.OK:
            raise RuntimeError(f"grilly_b200: grilly_init({index}) failed with status {rc}")
        self.ctx = h
        self.index = index
        self._weights: dict = {}
        self._pinned: dict = {}
        self._closed = False

    # ------------------------------------------------------------------ plumbing
    def check(self, rc: int) -> None:
        L.check(self.ctx, rc)

    def sync(self) -> None:
        self.check(self.lib.grilly_sync(self.ctx))

    def set_stream(self, cuda_stream_ptr: int | None) -> None:
        self.check(self.lib.grilly_set_stream(self.ctx, C.c_void_p(cuda_stream_ptr or 0)))

    def set_tuning(self, name: str, value: int) -> None:
        """Kernel-selection knob of this context (``grilly_set_tuning``): tests and sweeps use it to force a tile
        width or the CTA-pair kernel; 0 (``gemm_pair``/``gemm_swap``: -1) restores the default choice."""
        self.check(self.lib.grilly_set_tuning(self.ctx, name.encode(), int(value)))

    def launch_count(self) -> int:
        n = C.c_uint64(0)
        self.check(self.lib.grilly_launch_count(self.ctx, C.byref(n)))
        return n.value

    def alloc_ptr(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.check(self.lib.grilly_alloc(self.ctx, nbytes, C.byref(p)))
        return p.value

    def free_ptr(self, ptr: int) -> None:
        if not self._closed:
            self.lib.grilly_free(self.ctx, C.c_void_p(ptr))

    def empty(self, shape, dtype: str = "f32") -> DeviceTensor:
        t = DeviceTensor(self, 0, shape, dtype)
        t.ptr = self.alloc_ptr(max(t.nbytes, 16))
        return t

    def upload(self, arr: np.ndarray, dtype: str = "f32", round_tf32: bool = False) -> DeviceTensor:
        """Copy a NumPy array to the device as fp32 (optionally rounded to tf32), bf16 or int32."""
        if dtype == "i32":
            host = np.ascontiguousarray(arr, dtype=np.int32)
            t = self.empty(host.shape, "i32")
            self.check(self.lib.grilly_upload(self.ctx, t.ptr, host.ctypes.data, host.nbytes))
            self.sync()
            return t
        host = np.ascontiguousarray(arr, dtype=np.float32)
        t = self.empty(host.shape, "f32")
        self.check(self.lib.grilly_upload(self.ctx, t.ptr, host.ctypes.data, host.nbytes))
        if dtype == "bf16":
            tb = self.empty(host.shape, "bf16")
            self.check(self.lib.grilly_cast_f32_to_bf16(self.ctx, t.ptr, tb.ptr, t.size))
            self.sync()  # host buffer and the fp32 staging copy may now go away
            t.free()
            return tb
        if round_tf32:
            self.check(self.lib.grilly_round_tf32(self.ctx, t.ptr, t.ptr, t.size))
        self.sync()
        return t

    def download(self, t: DeviceTensor) -> np.ndarray:
        if t.dtype == "bf16":
            tf = self.empty(t.shape, "f32")
            self.check(self.lib.grilly_cast_bf16_to_f32(self.ctx, t.ptr, tf.ptr, t.size))
            out = self.download(tf)
            tf.free()
            return out
        out = np.empty(t.shape, dtype=np.int32 if t.dtype == "i32" else np.float32)
        self.check(self.lib.grilly_download(self.ctx, out.ctypes.data, t.ptr, out.nbytes))
        return out

    # ------------------------------------------------------------------ weights
    def weight(self, arr, dtype: str = "f32", round_tf32: bool = True, transform=None, tag: str = "") -> DeviceTensor:
        """Device copy of a weight array, cached by the identity of the host buffer.

        The key is (data pointer, shape, strides, dtype, requested device dtype, tag) and the entry lives as long as
        the ndarray that owns the buffer (a weak reference to the root of the view chain), so a freed and reused
        address can never serve stale weights. An in-place change of the host array is not seen until
        :meth:`invalidate` is called for it. Anything that is not an ndarray (a list, a buffer object) is converted
        and uploaded on every call.
        """
        if isinstance(arr, DeviceTensor):
            return arr
        cacheable = isinstance(arr, np.ndarray)
        a = np.asarray(arr)
        key = (a.__array_interface__["data"][0], a.shape, a.strides, a.dtype.str, dtype, round_tf32, tag)
        hit = self._weights.get(key)
        if hit is not None:
            ref, t = hit
            if ref() is not None:
                return t
            self._weights.pop(key)[1].free()   # the owner died: the address may belong to another array now
        host = transform(a) if transform is not None else a
        t = self.upload(host, dtype=dtype, round_tf32=round_tf32 and dtype == "f32")
        if not cacheable:
            return t
        root = a
        while isinstance(root.base, np.ndarray):
            root = root.base
        self._weights[key] = (weakref.ref(root), t)
        if len(self._weights) > 512:
            self._prune()
        return t

    def register_weight(self, arr) -> None:
        """Pin an ndarray so that its device copies stay cached until :meth:`invalidate`, even if the caller drops
        every reference: the device keeps one, which keeps the buffer and therefore the cache key valid."""
        if not isinstance(arr, np.ndarray):
            raise TypeError("register_weight expects a numpy.ndarray (other array-likes are converted per call)")
        self._pinned[arr.__array_interface__["data"][0]] = arr

    def _prune(self) -> None:
        dead = [k for k, (ref, _) in self._weights.items() if ref() is None]
        for k in dead:
            self._weights.pop(k)[1].free()

    def invalidate(self, arr=None) -> None:
        """Drop cached device copies of ``arr`` (or of every weight when ``arr`` is None)."""
        if arr is None:
            for _, t in self._weights.values():
                t.free()
            self._weights.clear()
            self._pinned.clear()
            return
        ptr = np.asarray(arr).__array_interface__["data"][0]
        self._pinned.pop(ptr, None)
        for k in [k for k in self._weights if k[0] == ptr]:
            self._weights.pop(k)[1].free()

    def timer_start(self) -> None:
        """Record the start event of the device-side stopwatch on the context's stream."""
        self.check(self.lib.grilly_timer_start(self.ctx))

    def timer_stop(self) -> float:
        """Record the stop event, wait for it and return the elapsed device time in milliseconds."""
        ms = C.c_float(0)
        self.check(self.lib.grilly_timer_stop(self.ctx, C.byref(ms)))
        return ms.value

    PROFILE_CLASSES = ("gemm", "attention", "norm", "embedding", "pooling", "other")

    def profile_begin(self) -> None:
        """Start bracketing every launch with CUDA events on the launching stream."""
        self.check(self.lib.grilly_profile_begin(self.ctx))

    def profile_end(self) -> dict:
        """Stop and return {class: {launches, ms, flops, bytes}} summed over the bracketed launches."""
        out = (C.c_double * (len(self.PROFILE_CLASSES) * 4))()
        self.check(self.lib.grilly_profile_end(self.ctx, out))
        res = {}
        for i, name in enumerate(self.PROFILE_CLASSES):
            res[name] = {"launches": int(out[4 * i]), "ms": out[4 * i + 1], "flops": out[4 * i + 2], "bytes": out[4 * i + 3]}
        return res

    def pool_stats(self) -> dict:
        out = (C.c_uint64 * 8)()
        self.check(self.lib.grilly_pool_stats(self.ctx, out))
        names = ["acquired", "released", "bytes_in_use", "peak_bytes", "pool_reserved_bytes",
                 "tensor_map_hits", "tensor_map_misses", "pool_hits"]
        d = {n: int(out[i]) for i, n in enumerate(names)}
        self._prune()   # entries whose host array has died are not cached weights any more (their key may be reused)
        d["cached_weights"] = len(self._weights)
        return d

    def close(self) -> None:
        if not self._closed:
            self.invalidate()
            self._closed = True
            self.lib.grilly_shutdown(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

