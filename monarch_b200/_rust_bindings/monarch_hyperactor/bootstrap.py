"""Entry of a proc started by an allocator (monarch_hyperactor/src/bootstrap.rs:22).
"""
from ..._native import bootstrap_attach, bootstrap_main  # noqa: F401
