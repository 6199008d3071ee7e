"""Shared constants (same literals as the reference's runtime/constants.py:3)."""

TRITON_SCORING_REQUIRED_MARKER = "TRIATTN_FATAL_TRITON_SCORING_REQUIRED"
