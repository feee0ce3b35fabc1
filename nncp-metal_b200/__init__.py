"""B200-native backend for NNCP's Transformer-XL train step (package root).

The product is the C-ABI shared library built from csrc/ (include/nncu.h) and
the C host code in host/; the Python modules here are the thin loader the
tests and the benchmark use to reach that ABI.
"""
from . import abi  # noqa: F401
from .loader import library, build_library, build_dropin, LibraryMissing, DROPIN_BIN  # noqa: F401
from .model import TrfModel  # noqa: F401
from . import host  # noqa: F401
from . import dist  # noqa: F401
