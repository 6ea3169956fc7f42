"""grilly_b200: a B200-native (sm_100a) implementation of grilly's dense transformer hot path.

``Compute()`` mirrors ``grilly.Compute()`` (backend/compute.py:23-128 of the reference) for the GEMM family,
flash-attention and the encoder glue around them; ``SentenceEncoder`` is the device-resident counterpart of
``VulkanSentenceTransformer.encode`` (utils/vulkan_sentence_transformer.py:1109-1219).

Importing the package does not load the CUDA library: that happens when the first ``Device`` / ``Compute`` is
created, or when ``CUDA_AVAILABLE`` is read.
"""
from __future__ import annotations

from . import _lib
from .compute import Compute
from .device import Device, DeviceTensor
from .encoder import SentenceEncoder, EncoderWeights

__version__ = "0.2.0"
VULKAN_AVAILABLE = False  # nothing here goes through Vulkan

__all__ = ["Compute", "Device", "DeviceTensor", "SentenceEncoder", "EncoderWeights", "CUDA_AVAILABLE", "VULKAN_AVAILABLE"]


def _probe() -> bool:
    try:
        import ctypes as C

        lib = _lib.load()
        n = C.c_int(0)
        return lib.grilly_device_count(C.byref(n)) == _lib.OK and n.value > 0
    except Exception:
        return False


def __getattr__(name: str):
    # CUDA_AVAILABLE: True when the CUDA library is built and a GPU is visible (the reference's VULKAN_AVAILABLE,
    # backend/base.py:8-48). Evaluated on first use, so that importing the package maps no shared library.
    if name == "CUDA_AVAILABLE":
        value = _probe()
        globals()["CUDA_AVAILABLE"] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
