"""B200-native implementation of numba-mlir's data-parallel GPU offload path.

The decorator names of numba_mlir/numba_mlir/__init__.py and kernel.py are the
user-facing surface; underneath, device work goes through the gpux* C-ABI of
libnumba_mlir_gpu_runtime_cuda.so (include/numba_mlir_gpu_runtime_cuda.h).
"""

from . import runtime  # noqa: F401
from .decorators import jit, njit, njit_replace_parfors, vectorize  # noqa: F401
from .device_array import (  # noqa: F401
    DeviceArray,
    as_device_array,
    empty,
    from_host,
    pinned_empty,
    zeros,
)

from .streaming import HostPipeline, map_host  # noqa: F401,E402

__version__ = "0.1.0"
