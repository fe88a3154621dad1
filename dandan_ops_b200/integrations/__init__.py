"""Adapters between inference engines and the W4A16 operator."""
