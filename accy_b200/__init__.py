"""accy_b200: B200 (sm_100a) execution target for recorded Accy tensor programs.

`accy_b200.tensor` mirrors the reference's recording API (`tensor.define`, `Value` methods) and
its execution entry points (`runCpu` -> `run_cuda`, `Cpu` -> `Cuda`, `Session`) on top of the C ABI
in `include/accy_b200.h`.  Everything executes in hand-written CUDA kernels; the package fails
loudly when the native library cannot be loaded, and there is no CPU fallback.
"""
from . import _native  # noqa: F401  (loads libaccy_b200.so or raises)
from . import tensor  # noqa: F401

__all__ = ["tensor"]
