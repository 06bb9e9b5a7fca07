"""Import-name shim: ``import fray`` resolves to the B200-native package.

Lets code written against the reference (``fray.jit_kernels.flash_attn_cute``,
``fray.bench_kineto``, ``fray.calc_diff``, ``fray.jit``) run unchanged.
"""
import sys

import fray_b200 as _impl
from fray_b200 import *  # noqa: F401,F403
from fray_b200 import bench_kineto, calc_diff, count_bytes, jit, jit_kernels, utils  # noqa: F401

for _name in ("jit", "jit_kernels", "utils", "jit.template", "jit.compiler", "jit.runtime",
              "jit_kernels.tuner", "jit_kernels.flashattn_cute", "multi_gpu"):
    __import__(f"fray_b200.{_name}")
    sys.modules[f"fray.{_name}"] = sys.modules[f"fray_b200.{_name}"]
