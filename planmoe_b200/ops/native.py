"""Loader for the in-tree native extension ``planmoe_b200/_C*.so``.

The extension holds every sm_100a kernel, the symmetric-heap runtime and the CPU C++
reference ops.  It is built in-tree by ``planmoe_b200.utils.build`` (never pip-installed),
so the shared object travels with the source tree.

``lib()`` returns the module or raises with the build command; ``available()`` probes.
GPU code paths call ``lib()`` so that a missing extension is a loud error, never a silent
fallback to eager PyTorch.
"""

import importlib
import os

_LIB = None
_ERR = None


def _try_load():
    global _LIB, _ERR
    if _LIB is not None or _ERR is not None:
        return
    try:
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        _LIB = importlib.import_module("planmoe_b200._C")
    except Exception as ex:  # ImportError or a loader error
        _ERR = ex


def available():
    _try_load()
    return _LIB is not None


def lib():
    _try_load()
    if _LIB is None:
        raise RuntimeError(
            "planmoe_b200 native extension is not built or failed to load (%r). "
            "Build it with:  python -m planmoe_b200.utils.build" % (_ERR,))
    return _LIB


def maybe_lib():
    """The module, or None when it is absent (CPU-only fallbacks may use this)."""
    _try_load()
    return _LIB


def force_python_fallback():
    """True when env PLANMOE_NO_NATIVE=1 asks CPU paths to avoid the extension."""
    return os.environ.get("PLANMOE_NO_NATIVE", "0") == "1"
