"""``import conductor`` -- drop-in import name of the reference package.

The implementation lives in :mod:`conductor_b200`; this module aliases it, and every
submodule (``conductor.optimization.graph_analyzer`` ...), so code written against the
reference's import paths keeps working and ``import conductor`` registers the ``gcu``
backend exactly as the reference's ``conductor/__init__.py:36-41`` does.
"""
import importlib
import pkgutil
import sys

import conductor_b200 as _impl

for _m in pkgutil.walk_packages(_impl.__path__, prefix="conductor_b200."):
    if ".csrc" in _m.name:
        continue
    try:
        importlib.import_module(_m.name)
    except Exception:  # optional pieces (e.g. sharding without torch.distributed) stay lazy
        pass
for _name, _mod in list(sys.modules.items()):
    if _name == "conductor_b200" or _name.startswith("conductor_b200."):
        sys.modules["conductor" + _name[len("conductor_b200"):]] = _mod
