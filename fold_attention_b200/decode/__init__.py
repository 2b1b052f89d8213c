"""Quantised paged-KV decode (host side)."""
