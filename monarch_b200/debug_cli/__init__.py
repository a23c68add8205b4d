"""``python -m monarch_b200.debug_cli`` -- console for the distributed debugger."""
