"""Drop-in import name: `import numba_mlir` / `from numba_mlir import njit`
resolve to the B200 offload implementation (numba_mlir/numba_mlir/__init__.py:5
exports the decorators the same way)."""

from numba_mlir_b200 import *  # noqa: F401,F403
from numba_mlir_b200 import __version__, jit, njit, njit_replace_parfors, vectorize  # noqa: F401
