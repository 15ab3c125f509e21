"""Single-device workflows (cp = 1)."""
