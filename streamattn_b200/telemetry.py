"""Sequence-length bucketing shared by the routing records (reference ``telemetry.py:17-22``)."""

from .decode import seq_bucket

__all__ = ["seq_bucket"]
