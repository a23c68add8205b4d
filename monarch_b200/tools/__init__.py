"""Operator tooling: the process-allocator daemon, the job CLI and the admin views."""
