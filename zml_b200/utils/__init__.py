"""Small host-side utilities (flags, formatting, logging, timing)."""
