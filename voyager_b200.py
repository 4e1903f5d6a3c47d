"""Import alias for the package in ``voyager-compiler-2_b200/``.

The package directory carries the project's name, which is not a valid Python
identifier, so this module loads it under the name ``voyager_b200``::

    import voyager_b200            # registers torch.ops.quantized_ops.* (CUDA)
    voyager_b200.build()           # compile the sm_100a library in-tree
"""

import importlib.util
import os
import sys

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "voyager-compiler-2_b200")


def _load():
    spec = importlib.util.spec_from_file_location(
        __name__, os.path.join(_DIR, "__init__.py"), submodule_search_locations=[_DIR])
    module = importlib.util.module_from_spec(spec)
    sys.modules[__name__] = module
    spec.loader.exec_module(module)
    return module


_load()
