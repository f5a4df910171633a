"""Tracing, logging and statistics helpers."""
