"""Stream capture without the garbage collector.

While a stream is being captured, destroying another CUDA graph is an operation that CUDA refuses, and
the refusal invalidates the capture: the next launch fails with "operation failed due to a previous
error during capture".  An engine and its graphs refer to one another, so an engine that its owner has
dropped lives on until Python's cycle collector runs, and the collector runs whenever enough objects
have been allocated: in the middle of a capture too.  `no_collection` collects first, so that dropped
engines and their graphs go before the capture begins, and keeps the collector off until the capture
has ended.
"""
from __future__ import annotations

import contextlib
import gc


@contextlib.contextmanager
def no_collection():
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        yield
    finally:
        if was_enabled:
            gc.enable()
