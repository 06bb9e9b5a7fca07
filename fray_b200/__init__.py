"""B200-native drop-in for the flash-attention forward path of Fray.

Same import surface as the reference package for that path (fray/__init__.py:1-5):
``jit``, ``jit_kernels.flash_attn_cute``, ``bench_kineto`` and ``calc_diff``.
"""
import torch  # noqa: F401  (the reference imports torch first as well)

from . import jit
from . import jit_kernels
from .utils import bench_kineto, calc_diff, count_bytes
