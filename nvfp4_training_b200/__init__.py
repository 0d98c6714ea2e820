"""B200-native (sm_100a) NVFP4 linear-layer hot path: quantizers + tcgen05 block-scaled FP4 GEMM
behind the reference's `nvq` / `fp4ops` Python API.  The CUDA library is built ahead of time by
`python -m nvfp4_training_b200.build`; importing the operator modules does not need a GPU, calling
them does (there is no CPU path)."""
import sys


def install_as_reference_modules():
    """Register this package's `nvq` and `fp4ops` under the reference's top-level module names so
    that unmodified reference code (`import nvq`, `import fp4ops as F`) resolves to them."""
    from . import fp4ops, nvq
    sys.modules["nvq"] = nvq
    sys.modules["fp4ops"] = fp4ops
    return nvq, fp4ops
