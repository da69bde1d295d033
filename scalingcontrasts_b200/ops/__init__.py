"""Kernel-backed operations: the streamed loss and its helpers."""
