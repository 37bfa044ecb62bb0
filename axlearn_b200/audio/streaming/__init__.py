"""Streaming (chunk-by-chunk) variants of audio layers."""
