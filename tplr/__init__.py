"""``import tplr``: the reference's package name as an alias of :mod:`templar_b200`.

Code written against the reference (``import tplr``, ``tplr.Comms``, ``tplr.compress.TopKCompressor``,
``from tplr.neurons import outer_step``, ``tplr.muon.Muon`` ...; src/tplr/__init__.py:22-40) runs on this
framework unchanged.  Every submodule is registered under both names as the SAME module object, so there is
one copy of each module's state (the ``dist_helper`` singleton, the logger, the native library handle).
"""

import importlib
import pkgutil
import sys

import templar_b200 as _impl

_self = sys.modules[__name__]
for _attr in dir(_impl):
    if not _attr.startswith("__") or _attr == "__version__":
        setattr(_self, _attr, getattr(_impl, _attr))

for _info in pkgutil.walk_packages(_impl.__path__, prefix="templar_b200."):
    try:
        _mod = importlib.import_module(_info.name)
    except Exception:  # noqa: BLE001  (an optional dependency of that submodule is absent: it stays unaliased)
        continue
    sys.modules["tplr." + _info.name[len("templar_b200."):]] = _mod
