"""Import alias: ``import attnfuse`` resolves to ``attentionfuse_b200``.

Code written against the reference package (its tests, examples and the
``attnfuse.integrations.hf`` import that registers the HuggingFace backend) keeps working
unmodified: every ``attnfuse.x.y`` module is the corresponding ``attentionfuse_b200.x.y``.
"""
import importlib
import importlib.abc
import importlib.util
import sys

import attentionfuse_b200 as _real

_PREFIX, _TARGET = __name__ + ".", _real.__name__ + "."


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real_name = _TARGET + fullname[len(_PREFIX):]
        if importlib.util.find_spec(real_name) is None:
            return None
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        return importlib.import_module(_TARGET + spec.name[len(_PREFIX):])

    def exec_module(self, module):
        pass


sys.meta_path.insert(0, _AliasFinder())
sys.modules[__name__] = _real
for _name, _mod in list(sys.modules.items()):
    if _name.startswith(_TARGET):
        sys.modules[_PREFIX + _name[len(_TARGET):]] = _mod
