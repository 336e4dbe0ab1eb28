"""Python access to libiris_b200.so for tests and the benchmark driver.

The product is the C-ABI shared library built from csrc/ (see include/*.h);
this package only loads it through ctypes and declares its signatures. There
is no Python or CPU implementation behind these names: loading fails loudly
when the library has not been built, and every operation fails when no
sm_100 device is present.
"""
from .binding import Lib, load, LIB_PATH, IrisB200Error  # noqa: F401
