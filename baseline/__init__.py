"""Baselines this library is measured against: the unmodified reference vendored beside it."""
