"""Command lines."""
