"""planmoe_b200 — a Blackwell-native (sm_100a) Mixture-of-Experts training framework.

Public modules mirror the reference package (``PlanMoE/__init__.py:4``): ``moe``, ``net``,
``system``, ``jit``, ``gates``, ``experts``, ``impls``, ``parted``, ``launcher``, ``examples``;
the packages ``planmoe`` and ``schemoe`` are import aliases of this one.  ``models``, ``ops``,
``parallel`` and ``utils`` hold the B200-specific machinery (GPT-MoE model, kernels' Python
bindings, symmetric-heap transport / scheduler, build and timing helpers).
"""

__version__ = "0.1.0"

from . import net      # noqa: F401
from . import system   # noqa: F401
from . import moe      # noqa: F401
from . import jit      # noqa: F401
