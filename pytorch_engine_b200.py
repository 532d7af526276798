"""Import alias: ``import pytorch_engine_b200`` gives the package in the folder ``pytorch-engine_b200``
(whose name is not a Python identifier).  Every submodule is aliased too, so nothing loads twice."""
import importlib
import sys

_pkg = importlib.import_module("pytorch-engine_b200")
for _name, _mod in list(sys.modules.items()):
    if _name == "pytorch-engine_b200" or _name.startswith("pytorch-engine_b200."):
        sys.modules["pytorch_engine_b200" + _name[len("pytorch-engine_b200"):]] = _mod
sys.modules[__name__] = _pkg
