"""Low-level attention operator wrappers."""
