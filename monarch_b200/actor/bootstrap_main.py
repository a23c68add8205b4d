"""Entry point of a proc spawned by the process allocator.

Parity: python/monarch/_src/actor/bootstrap_main.py + hyperactor_mesh/src/bootstrap.rs.
The native bootstrap loop dials the allocator (``HYPERACTOR_MESH_BOOTSTRAP_ADDR``),
announces itself, creates the proc with its mesh agent when told to, and exits when the
allocator says so or disappears.
"""
import base64
import os
import sys


def main() -> int:
    for mod in filter(None, os.environ.get("MB200_PREIMPORT", "").split(",")):
        try:
            __import__(mod)     # on the main thread, before any actor thread exists
        except ImportError:
            pass
    fn = os.environ.get("MB200_BOOTSTRAP_FN")
    if fn:
        import cloudpickle
        cloudpickle.loads(base64.b64decode(fn))()
    from monarch_b200 import _native as N
    import monarch_b200.actor  # noqa: F401  (registers the python actor type)
    return N.bootstrap_main()


if __name__ == "__main__":
    sys.exit(main())
