"""yule_b200 — a B200 (sm_100a) CUDA backend for Yule's quantized-inference hot path.

The product is ``libyule_cuda.so`` (C ABI in ``include/yule_cuda.h``); this package is its host-side
mirror of Yule's ``ComputeBackend`` trait and ``ModelRunner`` for tests, benchmarks and Python users.
"""

from .dtype import DType, matvec_bytes  # noqa: F401
from .backend import BufferHandle, CudaB200Backend, YuleGpuError, is_available  # noqa: F401
from .runner import CudaTransformerRunner, ModelConfig  # noqa: F401
from .gguf import GgufFile, GgufTensor, load_runner  # noqa: F401
