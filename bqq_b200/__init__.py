"""bqq_b200: B200 (sm_100a) implementation of the BinaryQuadratic linear forward.

`bqq_b200.bqq_modules` mirrors the reference module of the same name; `install()`
registers it as the top-level module `bqq_modules` so that pickled models that
record `bqq_modules.BinaryQuadratic` load onto this implementation.
"""
import sys

from . import _cabi  # noqa: F401  (fails loudly when the CUDA library is missing)
from . import bqq_modules
from .bqq_modules import (BinaryQuadratic, PackedBinaryQuadratic, PartialBQQLinear, PlaneBinaryQuadratic,  # noqa: F401
                          get_matrices, merge_binary_quadratic, merge_binaryquadratic_recursive,
                          pack_binaryquadratic_model, replace_linear_with_bqq, shard_rows)


def install() -> None:
    """Make `import bqq_modules` / unpickling resolve to this package's module, and
    `import bqq_cuda_ext` (what the reference's packed layer imports in its forward,
    src/bqq_modules.py:217-219) to this package's stand-in for the extension loader."""
    from . import bqq_cuda_ext
    sys.modules['bqq_modules'] = bqq_modules
    sys.modules['bqq_cuda_ext'] = bqq_cuda_ext
