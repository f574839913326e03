"""The bfloat16 kernel set used for serving: fast kernels where one exists for the
shape at hand, the plain kernel (same arithmetic, bfloat16 storage) otherwise."""
from __future__ import annotations

from .kernel_sets import PlainKernels


class FastKernels(PlainKernels):
    name = "fast"
