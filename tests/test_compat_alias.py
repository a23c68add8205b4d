"""``import monarch`` works as an alias of ``monarch_b200`` (same module objects)."""


def test_reference_style_imports_resolve_to_this_package():
    import monarch
    import monarch_b200
    from monarch.actor import Actor, endpoint, this_host  # noqa: F401
    from monarch.tensor_engine import RDMABuffer
    import monarch.actor
    import monarch.parallel.pipelining as pp
    import monarch_b200.actor
    import monarch_b200.parallel.pipelining

    assert monarch.actor is monarch_b200.actor
    assert Actor is monarch_b200.actor.Actor
    assert RDMABuffer is monarch_b200.tensor_engine.RDMABuffer
    assert pp is monarch_b200.parallel.pipelining
    assert monarch.remote is monarch_b200.remote and monarch.DeviceMesh is monarch_b200.DeviceMesh
    assert monarch.timer is monarch_b200.timer
    import pytest
    with pytest.raises(AttributeError):
        monarch.rust_mast_mesh
    with pytest.raises(ImportError):
        import monarch.no_such_module  # noqa: F401
