"""Token-sparse attention: grouping, selection, state machine and operator wrappers."""
