"""Host-side pieces of bench.py that need no GPU: the op table, the byte
accounting, the CPU leg and the reference arm's JSON line."""
import json
import os
import subprocess
import sys

import numpy as np

from conftest import ROOT

sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_suite_and_byte_table_agree():
    from oracle.numpy_oracle import OracleHandler, op_suite_inputs
    rows, cols = 64, 48
    d = op_suite_inputs(rows, cols, 3)
    t = {k: d[k] for k in ('a', 'b', 'dy', 'div', 'row', 'col')}
    t.update(labels=d['labels'].astype(np.float32), out=np.zeros((rows, cols), np.float32),
             y=np.tanh(d['a']), absa=np.abs(d['a']), s0=np.zeros((1, cols), np.float32),
             s1=np.zeros((rows, 1), np.float32), sall=np.zeros((), np.float32),
             picked=np.zeros((rows, 1), np.float32))
    suite = bench.make_suite(OracleHandler(np.float32), t)
    table = bench.suite_bytes(rows, cols)
    assert [n for n, _ in suite] == [n for n, _ in table]
    for _, fn in suite:
        fn()                                   # every thunk runs on the CPU handler
    n = rows * cols * 4
    by = dict(table)
    assert by['add_tt'] == 3 * n and by['sigmoid'] == 2 * n and by['sum_t_all'] == n + 4
    assert np.allclose(t['s0'], d['a'].sum(0, keepdims=True), rtol=1e-5, atol=1e-4)


def test_cpu_leg_reports_throughput():
    gbs, dt, kind = bench.cpu_suite_time(256, 128, 1, 2, 1, 0)
    assert gbs > 0 and dt > 0 and kind in ('reference', 'port')


def test_reference_arm_prints_one_json_line(monkeypatch):
    env = dict(os.environ, RANK='0')
    code = ("import sys; sys.argv=['bench.py','--impl','reference','--steps','1','--warmup','0'];"
            "import bench; bench.CPU_SAMPLE_ROWS=128; bench.CPU_LSTM_BATCH=2; bench.main()")
    out = subprocess.run([sys.executable, '-c', code], capture_output=True, text=True, cwd=ROOT, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line['impl'] == 'reference' and line['value'] > 0 and line['unit'] == 'GB/s'
    assert line['cpu_baseline']['cores'] >= 1 and line['e2e']['h2d_bytes_per_step'] == 0
    # the LSTM half of the metric on the reference's own stack (when its install is present)
    assert 'unavailable' in line['lstm'] or (line['lstm']['sequences_per_s'] > 0 and line['lstm']['batch'] == 2)
    other = subprocess.run([sys.executable, '-c', code], capture_output=True, text=True, cwd=ROOT,
                           env=dict(env, RANK='1'))
    assert other.returncode == 0 and other.stdout.strip() == ''      # other ranks do no work
