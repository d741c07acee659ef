"""Kernel-programming API, the names of numba_mlir/numba_mlir/kernel.py:5-22."""

from .kernel_impl import (  # noqa: F401
    DEFAULT_LOCAL_SIZE,
    GLOBAL_MEM_FENCE,
    LOCAL_MEM_FENCE,
    Kernel,
    atomic,
    barrier,
    get_global_id,
    get_global_size,
    get_group_id,
    get_local_id,
    get_local_size,
    group,
    kernel,
    kernel_func,
    local,
    mem_fence,
    private,
)
