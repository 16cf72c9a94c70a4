"""Import alias for the package directory ``spikingbrain-7b_b200/``.

The directory name carries a hyphen, which Python cannot import. This module
turns itself into that package: it points ``__path__`` at the directory and runs
its ``__init__.py``, so ``import spikingbrain_7b_b200.ops`` resolves to
``spikingbrain-7b_b200/ops.py``.
"""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "spikingbrain-7b_b200")]
__file__ = _os.path.join(__path__[0], "__init__.py")
with open(__file__, "r", encoding="utf-8") as _f:
    exec(compile(_f.read(), __file__, "exec"))
del _f, _os
