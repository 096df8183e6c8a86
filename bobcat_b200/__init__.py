"""bobcat-cuda: B200 (sm_100a) decode and prefill for bobcat's Q4_0 hybrid language models.

The product is ``libbobcat_cuda.so`` (hand-written CUDA kernels and C++ host code behind the C ABI
of ``include/bobcat_cuda.h``). This package is the Python mirror of that ABI, with the class and
method names of the reference's Rust API, used by the tests and the benchmark. There is no CPU
path: every class here needs the shared library and a CUDA device.
"""

from . import errors
from .backend import ACCUMULATE, F16, F32, OVERWRITE, Q4_0, Q6_K, Q8_0, SWIGLU, Buffer, Cuda, Norm, View
from .models import BatchCuda, Checkpoint, Engine, Lfm2Cuda, Model, Qwen35Cuda, SeqCuda, Trace

__all__ = [
    "errors", "Cuda", "Buffer", "View", "Norm", "Model", "Trace", "Checkpoint", "SeqCuda", "Lfm2Cuda", "Qwen35Cuda", "BatchCuda", "Engine",
    "F32", "F16", "Q4_0", "Q8_0", "Q6_K", "OVERWRITE", "ACCUMULATE", "SWIGLU",
]
