"""Python faces of the CUDA entry points.

Each function checks what only the host can check (devices, dtypes, contiguity, shapes),
passes raw pointers and the current stream to the `extern "C"` entry point, and raises
`KernelError` when the kernel refuses a size.  There is no other implementation behind
these functions: a tensor that is not on a CUDA device, or a library that cannot be
built, is an error.
"""
from .bindings import *      # noqa: F401,F403
from .bindings import KernelError  # noqa: F401
