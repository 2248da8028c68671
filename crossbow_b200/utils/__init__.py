"""Small host-side helpers (counter-based RNG, logging, measurement tools)."""
