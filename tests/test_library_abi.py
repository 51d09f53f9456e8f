"""The shared library loads without a GPU and exports exactly what the header
declares; calls that need a device fail with a clear error, not a crash."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported():
    from brainstorm_b200._lib import PROTOTYPES, lib, HEADER
    with open(HEADER) as f:
        declared = set(re.findall(r'\b(b200_\w+)\s*\(', f.read()))
    assert declared == set(PROTOTYPES), declared ^ set(PROTOTYPES)
    assert len(declared) > 60
    for name in declared:
        assert getattr(lib, name) is not None
    out = subprocess.run(['nm', '-D', '--defined-only',
                          os.path.join(ROOT, 'brainstorm_b200', 'libb200handler.so')],
                         capture_output=True, text=True).stdout
    exported = set(re.findall(r'\bT (b200_\w+)', out))
    assert exported == declared, exported ^ declared


def test_prototypes_parse_pointer_and_scalar_types():
    from brainstorm_b200._lib import PROTOTYPES
    ret, args = PROTOTYPES['b200_clip_t']
    assert ret is ctypes.c_int
    assert args == [ctypes.c_void_p, ctypes.c_float, ctypes.c_float, ctypes.c_void_p,
                    ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
    assert PROTOTYPES['b200_last_error'] == (ctypes.c_char_p, [])
    assert PROTOTYPES['b200_sum_t_scratch_floats'][0] is ctypes.c_int64


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip('a GPU is present')
    from brainstorm_b200 import B200Handler, B200Error
    with pytest.raises(B200Error):
        B200Handler()


def test_calls_before_init_fail_cleanly():
    code = ("import ctypes,sys; sys.path.insert(0, %r); from brainstorm_b200._lib import lib; "
            "rc = lib.b200_add_tt(0, 0, 0, 1, 8, 8, 8, 8); "
            "print(rc, lib.b200_last_error().decode())" % ROOT)
    out = subprocess.run(['python', '-c', code], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert out.stdout.startswith('2 ') and 'b200_init' in out.stdout


def test_scratch_size_query_needs_no_device():
    from brainstorm_b200._lib import lib
    assert lib.b200_sum_t_scratch_floats(65536, 4096, 4096, 1) == 0
    n0 = lib.b200_sum_t_scratch_floats(65536, 4096, 4096, 0)
    assert n0 > 0 and n0 % 4096 == 0
    assert lib.b200_sum_t_scratch_floats(0, 4096, 4096, 0) == 0


def test_peer_allreduce_entry_points_refuse_to_run_unconfigured():
    """No GPU here: the peer all-reduce must say what is missing instead of crashing."""
    from brainstorm_b200._lib import lib
    assert lib.b200_peer_window_bytes() == 2 * 65536 * 4 + 256 + 16 * 512 * 8    # two slots, the counters, the per-group counters
    assert lib.b200_peer_max_floats() == 65536
    assert lib.b200_peer_allreduce(None, None, 4, 0) != 0
    assert lib.b200_peer_teardown() == 0          # nothing set up: nothing to do
