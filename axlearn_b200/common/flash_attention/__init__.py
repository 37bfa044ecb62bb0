"""Fused attention layer and kernel selection."""
