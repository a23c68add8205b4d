"""Import paths of the reference's native extension (``monarch._rust_bindings.*``) over this
package's runtime.

The reference binds a Rust runtime through one PyO3 extension whose submodules Python code
and tests import directly (monarch_extension/src/lib.rs:60-231; stubs under
python/monarch/_rust_bindings/).  Here the runtime is C++ (``monarch_b200._native``,
``monarch_b200._tensor_worker``) with its Python layer in ``monarch_b200.actor``; these
modules give the same names at the same paths.  What a name maps to is stated in each
module; names of the reference's legacy v0 system (``client``, ``controller``) that have no
counterpart here are absent, and importing them raises ``ImportError``.
"""
from . import monarch_extension, monarch_hyperactor, monarch_messages, rdma  # noqa: F401


def has_tensor_engine() -> bool:
    """Whether distributed tensors are available (the tensor worker's native core builds)."""
    try:
        from .. import _tensor_worker  # noqa: F401
        return True
    except ImportError:
        return False
