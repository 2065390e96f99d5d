"""maple_runtime_b200 -- Maple's mixture-of-experts layer on B200 (sm_100a) behind the reference's C plug-in ABI.

The product is the C library ``libgpre_cuda.so`` (sources in ``csrc/``, prototypes in ``include/gpre.h`` and
``include/gmoe.h``).  This package is a thin ctypes binding used by the tests and the benchmark: it loads the
library, declares every exported prototype, and fails loudly when the library is missing.  It contains no
arithmetic of its own and no CPU fallback.
"""
from .lib import Gpre, load, build, LIB_PATH, DECLS, CONST  # noqa: F401
