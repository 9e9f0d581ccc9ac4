"""B200-native Nengo simulator backend with the nengo_ocl planning surface.

``Simulator`` is the public entry point (same API as ``nengo_ocl.Simulator``).
Importing the package does not touch the GPU; the CUDA library is loaded on
first use and there is no CPU fallback.
"""

import logging

__version__ = "0.1.0"

logging.getLogger(__name__).addHandler(logging.NullHandler())


def __getattr__(name):
    if name == "Simulator":
        from nengo_ocl_b200.simulator import Simulator

        return Simulator
    raise AttributeError(name)
