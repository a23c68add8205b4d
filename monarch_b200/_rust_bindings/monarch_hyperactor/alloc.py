"""Allocation specs and allocators (monarch_hyperactor/src/alloc.rs:59-470).
"""
from ...actor.allocator import Alloc, AllocConstraints, AllocSpec  # noqa: F401
from ...actor.allocator import LocalAllocator as LocalAllocatorBase  # noqa: F401
from ...actor.allocator import ProcessAllocator as ProcessAllocatorBase  # noqa: F401
from ...actor.allocator import RemoteAllocator as RemoteAllocatorBase  # noqa: F401
from ...actor.allocator import SimAllocator as SimAllocatorBase  # noqa: F401
from ...actor.allocator import _AllocatorBase as AllocatorBase  # noqa: F401
