"""kernelforge for B200: the two inference hot paths of KernelForge (fused attention forward, INT4 weight-only
linear) as hand-written sm_100a kernels behind the reference's operator surface.

`kernelforge.ops`, `kernelforge.quantize` and `kernelforge.modules` keep the reference's names and call
conventions (kernelforge/__init__.py:1-8 of the reference lists the same modules); the compiled part is the
C-ABI library `libkfb200.so` next to this file (declared in include/kfb200.h, bound in `_capi`), which takes
the place of the reference's pybind11 extension `kernelforge._C`.  Importing the package loads nothing: the
library is opened at the first kernel call and a missing build raises ImportError there.
"""

__version__ = "0.2.0"
