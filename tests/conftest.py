"""pytest configuration: markers and import paths.

``gpu`` marks every test that needs a CUDA device; everything else runs on CPU.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'tests', 'golden')):
    if p not in sys.path:
        sys.path.insert(0, p)
# The importable install of the reference (layers, Network, Trainer: the callers
# of the handler).  Optional: tests that need it skip when it is absent.
REF = os.path.join(ROOT, 'baseline', '_ref')
if os.path.isdir(os.path.join(REF, 'brainstorm')) and REF not in sys.path:
    sys.path.insert(0, REF)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: test needs a CUDA device (B200)')


def has_reference():
    try:
        import brainstorm  # noqa: F401
        return True
    except Exception:
        return False


needs_reference = pytest.mark.skipif(
    not has_reference(), reason='reference install (baseline/_ref) not present')
