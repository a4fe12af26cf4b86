"""Helpers for turning raw recordings into a dataset before an upload (the upload itself needs a network)."""
