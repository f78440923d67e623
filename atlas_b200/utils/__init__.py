"""Utilities: metrics, tracing, fault latch, environment config."""
