"""grilly_b200: a B200-native (sm_100a) implementation of grilly's dense transformer hot path.

``Compute()`` mirrors ``grilly.Compute()`` (backend/compute.py:23-128 of the reference) for the GEMM family,
flash-attention and the encoder glue around them; ``SentenceEncoder`` is the device-resident counterpart of
``VulkanSentenceTransformer.encode`` (utils/vulkan_sentence_transformer.py:1109-1219).
"""
from __future__ import annotations

from . import _lib

__version__ = "0.1.0"


def _probe() -> bool:
    try:
        import ctypes as C

        lib = _lib.load()
        n = C.c_int(0)
        return lib.grilly_device_count(C.byref(n)) == _lib.OK and n.value > 0
    except Exception:
        return False


#: True when the CUDA library is built and a GPU is visible (the reference's VULKAN_AVAILABLE, backend/base.py:8-48)
CUDA_AVAILABLE = _probe()
VULKAN_AVAILABLE = False  # nothing here goes through Vulkan

from .compute import Compute  # noqa: E402
from .device import Device, DeviceTensor  # noqa: E402
from .encoder import SentenceEncoder, EncoderWeights  # noqa: E402

__all__ = ["Compute", "Device", "DeviceTensor", "SentenceEncoder", "EncoderWeights", "CUDA_AVAILABLE", "VULKAN_AVAILABLE"]
