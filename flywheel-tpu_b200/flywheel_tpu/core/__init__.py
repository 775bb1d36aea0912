"""Hardware facts and integer helpers."""
