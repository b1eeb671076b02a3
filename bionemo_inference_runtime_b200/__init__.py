"""B200-native triangle attention and pair transition behind the reference's module API.

``from bionemo_inference_runtime_b200 import TriangleAttentionStartingNode, TriangleAttentionEndingNode,
Transition`` gives drop-in replacements of the reference layers of the same names; every forward runs
hand-written sm_100a kernels from ``libb200ta.so`` (C ABI in ``include/b200ta.h``).  There is no fallback:
importing the layers without the built library raises.
"""

from . import _lib

_lib.load()  # fail loudly at import when the extension has not been built

from . import ops  # noqa: E402
from .layers import *  # noqa: E402,F401,F403
from .layers import __all__ as _layers_all  # noqa: E402
from .host_pipeline import HostPipeline, bind_to_gpu_numa_node  # noqa: E402

__all__ = ["ops", "HostPipeline", "bind_to_gpu_numa_node", *_layers_all]
