"""brainstorm_b200: an NVIDIA B200 (sm_100a) backend for the brainstorm Handler API.

    from brainstorm_b200 import B200Handler
    net.set_handler(B200Handler())

Importing the package loads ``libb200handler.so`` (build it with
``python -m brainstorm_b200.build``); there is no CPU fallback.
"""
from ._lib import B200Error, lib  # noqa: F401
from .array import B200Array  # noqa: F401
from .handler import B200Handler  # noqa: F401

__all__ = ['B200Handler', 'B200Array', 'B200Error']
