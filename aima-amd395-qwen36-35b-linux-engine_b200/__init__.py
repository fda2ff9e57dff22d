"""B200 (sm_100a) routed mixture-of-experts provider for the Qwen3.6-35B-A3B
class model: Python binding of libaima_moe_b200.so.

The directory name is not a Python identifier; load it with
``importlib`` (see ``__graft_entry__.load_package``) or put this directory's
parent on ``sys.path`` and import it through ``importlib.import_module``.
"""
from .provider import (  # noqa: F401
    AimaMoeError,
    MoeLibrary,
    LmHead,
    MoeProvider,
    StripedImage,
    library_path,
    load_library,
)
from . import synth  # noqa: F401

__all__ = ["AimaMoeError", "LmHead", "MoeLibrary", "MoeProvider", "StripedImage", "library_path", "load_library", "synth"]
