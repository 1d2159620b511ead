"""idrak_b200 — a Blackwell-native deep-learning framework with the capabilities of Idrak.

PyTorch is the tensor/autograd layer; the hot operations are hand-written sm_100a kernels
(``idrak_b200/csrc``) loaded through a flat C ABI; collectives run over NVLink peer memory from inside
kernels and are fused with the compute next to them.
"""
__version__ = "0.1.0"

from . import _native  # noqa: F401


def native_available() -> bool:
    """True when the compiled kernel library is present (it is required on a GPU machine)."""
    return _native.available()
