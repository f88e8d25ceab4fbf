"""What a checkout of the reference needs to run on this library: `monoserve_b200.compat._C`
exports the names of the reference's native extension `monoserve._C`
(csrc/bindings.cpp:171-384), and `install()` registers it under that name."""
import sys


def install():
    """Make `import monoserve._C` (and `monoserve._C.control`) resolve to this library's
    drop-in module.  Call before the reference's Python package is imported."""
    from monoserve_b200.compat import _C
    sys.modules["monoserve._C"] = _C
    sys.modules["monoserve._C.control"] = _C.control
    parent = sys.modules.get("monoserve")
    if parent is not None:
        parent._C = _C
    return _C
