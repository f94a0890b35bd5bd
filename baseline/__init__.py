"""Measurement-only helpers around the reference checkout (never imported by the shipped package)."""
