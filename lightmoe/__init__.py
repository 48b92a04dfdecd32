"""``lightmoe`` import name for code written against the reference package.

``import lightmoe``, ``lightmoe.gemm``, ``lightmoe.inference``,
``lightmoe.kernels.routing.combine`` ... resolve to the very same module
objects as ``nvfp4moe_b200`` and its submodules, so existing callers switch by
changing nothing but the installed package.
"""

import importlib
import pkgutil
import sys

import nvfp4moe_b200 as _impl

for _info in pkgutil.walk_packages(_impl.__path__, _impl.__name__ + "."):
    if _info.name.rsplit(".", 1)[-1].startswith("lib"):
        continue  # the CUDA shared library sits in the package folder; it is not a Python module
    _module = importlib.import_module(_info.name)
    sys.modules[__name__ + _info.name[len(_impl.__name__):]] = _module

sys.modules[__name__] = _impl
