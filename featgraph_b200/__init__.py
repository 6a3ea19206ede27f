"""featgraph_b200: vanilla SpMM / SDDMM for NVIDIA B200 (sm_100a) behind the module
interface of dglai/FeatGraph (``featgraph.module``, ``featgraph.util``)."""
from . import util
from .placeholder import Placeholder, placeholder

__all__ = ["util", "module", "placeholder", "Placeholder"]


def __getattr__(name):
    # the module layer needs torch; import it on first use so that the host-side
    # utilities stay importable on their own
    if name in ("module", "op", "graphgen", "sharded"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
