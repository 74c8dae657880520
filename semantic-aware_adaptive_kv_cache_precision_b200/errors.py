"""Errors that more than one part of the library raises."""

from __future__ import annotations


class OutOfDeviceMemory(RuntimeError):
    """The device could not give the memory that the weights or the cache need. What was
    being built is dropped whole: an engine that raised this holds no half-loaded model
    and no half-built cache. The reference has the same typed error for its allocations
    (`src/core_kernels/include/microinfer/check.h:18-73`)."""


def allocate(make, what: str, nbytes: int):
    """`make()`, with the allocator's out-of-memory error turned into `OutOfDeviceMemory`
    that says what was asked for."""
    import torch
    try:
        return make()
    except torch.OutOfMemoryError as exc:
        raise OutOfDeviceMemory(f"the device has no room for {what} ({nbytes:,} bytes); "
                                "nothing of it was kept") from exc
