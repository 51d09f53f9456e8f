#!/usr/bin/env python
"""Benchmark of the B200 handler hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): the handler op suite on fp32 (65536, 4096) operands (1 GiB each),
(1, 4096) / (65536, 1) broadcast vectors and 65536 labels in [0, 4096).  One
"step" runs every op of the suite once.  The metric is the suite's algorithmic
HBM bytes per second.  With N > 1 ranks (one process per GPU, launched with
torch.distributed.run) every rank runs the suite on its own (65536, 4096) row
shard (weak scaling: the global batch is 65536*N rows) and the axis-0 sum is
completed across shards by an NCCL all-reduce of the (1, 4096) partial sums.

`value` is measured with the operands resident in HBM; `e2e` runs the same suite
through the public handler API from page-locked HOST buffers, with the
host->device copies of the operands and the device->host read of the reduction
results inside the timed region.

`--impl reference` times the CPU restatement of the reference's NumpyHandler
(oracle/numpy_oracle.py) on a bounded row sample of the same workload, spread
over all host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS = 65536, 4096
SEED = 1
CPU_SAMPLE_ROWS = 16384          # bounded sample for the CPU legs (same columns)
METRIC = 'handler_op_suite_throughput'
UNIT = 'GB/s'


# ------------------------------------------------------------------ op suite
def suite_bytes(rows, cols):
    """Algorithmic HBM bytes of each op (4-byte elements): every operand that
    must be read once plus every result that must be written once."""
    n = rows * cols
    e = 4
    table = [
        ('add_tt', 3 * n), ('subtract_tt', 3 * n), ('mult_tt', 3 * n), ('divide_tt', 3 * n),
        ('add_mv_row', 2 * n + cols), ('add_mv_col', 2 * n + rows),
        ('mult_mv_row', 2 * n + cols), ('mult_mv_col', 2 * n + rows),
        ('mult_st', 2 * n),
        ('sigmoid', 2 * n), ('sigmoid_deriv', 3 * n), ('tanh', 2 * n), ('tanh_deriv', 3 * n),
        ('rel', 2 * n), ('rel_deriv', 3 * n), ('el', 2 * n), ('el_deriv', 3 * n),
        ('sum_t_axis0', n + cols), ('sum_t_axis1', n + rows), ('sum_t_all', n + 1),
        ('softmax_m', 2 * n), ('clip_t', 2 * n), ('abs_t', 2 * n), ('sign_t', 2 * n),
        ('sqrt_t', 2 * n), ('binarize_v', n + rows), ('index_m_by_v', 3 * rows),
    ]
    return [(name, cnt * e) for name, cnt in table]


def make_suite(H, t):
    """[(name, thunk)] running each op once on the arrays in dict t."""
    a, b, dy, div, out, y, absa = t['a'], t['b'], t['dy'], t['div'], t['out'], t['y'], t['absa']
    row, col, labels = t['row'], t['col'], t['labels']
    s0, s1, sall, picked = t['s0'], t['s1'], t['sall'], t['picked']
    return [
        ('add_tt', lambda: H.add_tt(a, b, out)),
        ('subtract_tt', lambda: H.subtract_tt(a, b, out)),
        ('mult_tt', lambda: H.mult_tt(a, b, out)),
        ('divide_tt', lambda: H.divide_tt(a, div, out)),
        ('add_mv_row', lambda: H.add_mv(a, row, out)),
        ('add_mv_col', lambda: H.add_mv(a, col, out)),
        ('mult_mv_row', lambda: H.mult_mv(a, row, out)),
        ('mult_mv_col', lambda: H.mult_mv(a, col, out)),
        ('mult_st', lambda: H.mult_st(0.37, a, out)),
        ('sigmoid', lambda: H.sigmoid(a, out)),
        ('sigmoid_deriv', lambda: H.sigmoid_deriv(a, y, dy, out)),
        ('tanh', lambda: H.tanh(a, out)),
        ('tanh_deriv', lambda: H.tanh_deriv(a, y, dy, out)),
        ('rel', lambda: H.rel(a, out)),
        ('rel_deriv', lambda: H.rel_deriv(a, y, dy, out)),
        ('el', lambda: H.el(a, out)),
        ('el_deriv', lambda: H.el_deriv(a, y, dy, out)),
        ('sum_t_axis0', lambda: H.sum_t(a, 0, s0)),
        ('sum_t_axis1', lambda: H.sum_t(a, 1, s1)),
        ('sum_t_all', lambda: H.sum_t(a, None, sall)),
        ('softmax_m', lambda: H.softmax_m(a, out)),
        ('clip_t', lambda: H.clip_t(a, -1.0, 1.0, out)),
        ('abs_t', lambda: H.abs_t(a, out)),
        ('sign_t', lambda: H.sign_t(a, out)),
        ('sqrt_t', lambda: H.sqrt_t(absa, out)),
        ('binarize_v', lambda: H.binarize_v(labels, out)),
        ('index_m_by_v', lambda: H.index_m_by_v(a, labels, picked)),
    ]


def host_inputs(rows, cols, seed, alloc=None):
    """The workload's seeded synthetic operands: the full draw of
    ``workloads.op_suite_inputs`` (uniform[-4, 4]; divisors uniform[0.5, 4] with a random
    sign; labels uniform in [0, cols)), labels as the fp32 column the handler takes."""
    from brainstorm_b200.workloads import op_suite_inputs
    d = op_suite_inputs(rows, cols, seed, alloc=alloc)
    d['labels'] = d['labels'].astype(np.float32)
    return d


# ------------------------------------------------------------------ clocks
class ClockSampler(object):
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(gpu_index), '--query-gpu=' + self.QUERY,
                 '--format=csv,noheader,nounits', '-lms', '100'],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for ts, line in self.rows:
            if ts < t0 or ts > t1 + 0.2:
                continue
            f = [x.strip() for x in line.split(',')]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': float(np.median(sm)) if sm else None, 'sm_max_mhz': mx,
                'reasons': sorted(reasons), 'samples': len(sm)}


# ------------------------------------------------------------------ CPU legs
def cpu_handler():
    """The CPU side of the comparison: the reference's own NumpyHandler when an
    install of the reference is present (kind 'reference'), else the oracle port of it
    (kind 'port')."""
    ref = os.path.join(ROOT, 'baseline', '_ref')
    if os.path.isdir(os.path.join(ref, 'brainstorm')) and ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            from brainstorm.handlers import NumpyHandler
        return NumpyHandler(np.float32), 'reference'
    except Exception:
        from oracle.numpy_oracle import OracleHandler
        return OracleHandler(np.float32), 'port'


def cpu_suite_time(rows, cols, seed, threads, steps, warmup):
    """Times the CPU handler (see cpu_handler) on `rows` rows, split into row chunks
    over `threads` host threads (numpy releases the GIL).  Returns GB/s, seconds per
    step and the kind of handler used."""
    from concurrent.futures import ThreadPoolExecutor
    from brainstorm_b200.workloads import op_suite_inputs
    O, kind = cpu_handler()
    d = op_suite_inputs(rows, cols, seed)
    labels = d['labels'].astype(np.float32)
    y = np.zeros_like(d['a'])
    O.tanh(d['a'], y)
    absa = np.abs(d['a'])
    bounds = np.linspace(0, rows, threads + 1).astype(int)
    chunks = []
    for i in range(threads):
        lo, hi = bounds[i], bounds[i + 1]
        if hi <= lo:
            continue
        t = {k: d[k][lo:hi] for k in ('a', 'b', 'dy', 'div')}
        t.update(out=np.zeros((hi - lo, cols), np.float32), y=y[lo:hi], absa=absa[lo:hi],
                 row=d['row'], col=d['col'][lo:hi], labels=labels[lo:hi],
                 s0=np.zeros((1, cols), np.float32), s1=np.zeros((hi - lo, 1), np.float32),
                 sall=np.zeros((), np.float32), picked=np.zeros((hi - lo, 1), np.float32))
        chunks.append(make_suite(O, t))

    def run_chunk(suite):
        for _, fn in suite:
            fn()

    def step(pool):
        list(pool.map(run_chunk, chunks))

    with ThreadPoolExecutor(max_workers=threads) as pool:
        for _ in range(warmup):
            step(pool)
        t0 = time.perf_counter()
        for _ in range(steps):
            step(pool)
        dt = (time.perf_counter() - t0) / steps
    nbytes = sum(b for _, b in suite_bytes(rows, cols))
    return nbytes / dt / 1e9, dt, kind


CPU_LSTM_BATCH = 32     # sequences per step of the reference arm's LSTM sample


def reference_lstm_step(batch=None, steps=1):
    """The character-LSTM training step (time 100, 205 symbols, 2 x 1000 units, SGD) on the
    reference's own stack: NumpyHandler, LstmLayerImpl, SgdStepper, unchanged.  A bounded
    sample: `batch` sequences per step instead of 128 (a step costs about batch / 16 seconds
    of host time; numpy's BLAS uses all cores)."""
    batch = batch or CPU_LSTM_BATCH
    ref = os.path.join(ROOT, 'baseline', '_ref')
    if os.path.isdir(os.path.join(ref, 'brainstorm')) and ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        import brainstorm  # noqa: F401
        from brainstorm.handlers import NumpyHandler
    except Exception as e:
        return {'unavailable': 'the reference install (baseline/_ref) is not importable: %s' % e}
    import importlib.util
    spec = importlib.util.spec_from_file_location('b200_workloads', os.path.join(ROOT, 'brainstorm_b200', 'workloads.py'))
    workloads = importlib.util.module_from_spec(spec)    # the network builder only: no GPU library is loaded
    spec.loader.exec_module(workloads)
    net, data, stepper = workloads.lstm(time=100, batch=batch)
    net.set_handler(NumpyHandler(np.float32))
    st = stepper()
    st.start(net)

    def step():
        net.provide_external_data(data)
        st.run()
        return float(net.get_loss_values()['total_loss'])

    step()
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = step()
    dt = (time.perf_counter() - t0) / steps
    return {'sequences_per_s': round(batch / dt, 2), 'ms_per_step': round(dt * 1e3, 1), 'time_steps': 100,
            'batch': batch, 'hidden': 1000, 'layers': 2, 'steps': steps, 'loss': round(loss, 4), 'kind': 'reference',
            'cores': os.cpu_count() or 1,
            'sample': '%d sequences per step instead of 128, %d step(s) after 1 warm-up' % (batch, steps)}


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    if args.only == 'lstm':
        res = reference_lstm_step()
        print(json.dumps({'impl': 'reference', 'metric': 'lstm_train_sequences_per_s',
                          'value': res.get('sequences_per_s'), 'unit': 'sequences/s', 'n_gpus': args.gpus, 'lstm': res}))
        return
    steps = max(1, min(args.steps, 5))
    gbs, dt, kind = cpu_suite_time(CPU_SAMPLE_ROWS, COLS, SEED, threads, steps, min(args.warmup, 1))
    sample = '%d of %d rows per step (same %d columns, same ops), %d steps' % (
        CPU_SAMPLE_ROWS, ROWS, COLS, steps)
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': round(gbs, 3), 'unit': UNIT,
        'n_gpus': args.gpus, 'steps': steps, 'warmup': min(args.warmup, 1),
        'ms_per_step': round(dt * 1e3, 3), 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic (seeded)',
        'config': {'workload': 'handler op suite, fp32 (%d, %d) operands' % (ROWS, COLS),
                   'sample_rows': CPU_SAMPLE_ROWS, 'cols': COLS, 'seed': SEED},
        'cpu_baseline': {'value': round(gbs, 3), 'unit': UNIT, 'cores': threads, 'kind': kind,
                         'sample': sample},
        'e2e': {'value': round(gbs, 3), 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    if args.only == 'all':
        line['lstm'] = reference_lstm_step()
    print(json.dumps(line))


# ------------------------------------------------------------------ training workloads
def _reference_on_path():
    ref = os.path.join(ROOT, 'baseline', '_ref')
    if os.path.isdir(os.path.join(ref, 'brainstorm')) and ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        import brainstorm  # noqa: F401
        return None
    except Exception as e:
        return 'brainstorm (the caller of the handler) is not importable: %s' % e


def _max_over_ranks(value, world):
    if world == 1:
        return value
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], device='cuda', dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _timed_steps(step, steps, barrier, world, warm=3):
    """ms per step: host wall clock around `steps` whole updates (each ends with the loss
    read-back), bracketed by a barrier and a synchronisation, max over ranks."""
    for _ in range(warm):
        loss = step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = step()
    barrier()
    return _max_over_ranks((time.perf_counter() - t0) / steps, world) * 1e3, loss


def _pipelined_ms(net, run, H, host_data, batch, total, warm, barrier, world):
    """ms per update with the next batch uploaded during the step and the loss read one call
    late (PrefetchingIterator + defer_loss_readback): `total` minibatches, the first `warm` untimed."""
    import brainstorm as bs
    from brainstorm_b200.pipeline import PrefetchingIterator, defer_loss_readback
    many = {k: np.concatenate([v] * total, axis=1) for k, v in host_data.items()}
    it = PrefetchingIterator(bs.data_iterators.Minibatches(batch, shuffle=False, **many))
    deferred = defer_loss_readback(net)
    barrier()
    t0, k = None, 0
    for b in it(handler=H):
        if k == warm:
            barrier()
            t0 = time.perf_counter()
        net.provide_external_data(b)
        run()
        net.get_loss_values()
        k += 1
    deferred.flush()
    barrier()
    ms = _max_over_ranks((time.perf_counter() - t0) / (k - warm), world) * 1e3
    deferred.restore()
    return ms


def lstm_training(H, world, rank, steps, barrier, lib):
    """Second half of the metric: training sequences per second of the character LSTM
    (time 100, batch 128 per GPU, 205 symbols, 2 x 1000 units, SoftmaxCE, SGD) through the
    reference's unchanged Network / SgdStepper on this handler with the fused LSTM layer
    and 16-byte aligned hubs.  Every step uploads its batch from page-locked host memory
    and reads the loss back, as Trainer does.  Timed twice: every rank on its own (the
    one-GPU figure, no exchange), then data-parallel with the gradient all-reduce."""
    why = _reference_on_path()
    if why:
        return {'unavailable': why}
    from brainstorm_b200 import workloads
    from brainstorm_b200.fused_lstm import fuse_lstm_layers
    T, B = 100, 128
    net, data, stepper = workloads.lstm(time=T, batch=B, data_seed=rank)
    pinned = {}
    for k, v in data.items():
        pinned[k] = H.pinned_empty(v.shape, np.float32)
        pinned[k][...] = v
    net.set_handler(H)
    fuse_lstm_layers(net)
    st = stepper()
    st.start(net)

    def step():
        net.provide_external_data(pinned)
        st.run()
        return float(net.get_loss_values()['total_loss'])

    out = {'T': T, 'batch_per_gpu': B, 'global_batch': world * B, 'hidden': 1000, 'layers': 2, 'steps': steps}
    ms1, loss = _timed_steps(step, steps, barrier, 1)
    out['n1_ms'] = round(ms1, 3)
    out['n1_sequences_per_s'] = round(B / ms1 * 1e3, 1)
    ms = ms1
    if world > 1:
        from brainstorm_b200.parallel import Comm, data_parallel
        data_parallel(net, Comm())
        l0 = lib.b200_launch_count()
        ms, loss = _timed_steps(step, steps, barrier, world)
        out['launches_per_step'] = int((lib.b200_launch_count() - l0) // (steps + 3))
        out['allreduce_floats'] = int(net.buffer.parameters.size)
    out['ms_per_step'] = round(ms, 3)
    out['sequences_per_s'] = round(world * B / ms * 1e3, 1)
    out['vs_n1'] = round(out['sequences_per_s'] / out['n1_sequences_per_s'], 3)
    out['loss'] = round(loss, 4)
    # the same updates with the next batch uploaded during the step and the loss read one call late
    out['pipelined_ms'] = round(_pipelined_ms(net, lambda: st.run(), H, data, B, steps + 3, 3, barrier, world), 3)
    out['h2d_bytes_per_step'] = int(sum(v.nbytes for v in pinned.values()))
    return out


def other_training(name, H, world, rank, barrier, lib, new_event, elapsed, blocks=10):
    """The other training workloads.  'mlp': the MNIST-style MLP, batch 100 per GPU
    (weak scaling), momentum SGD.  'cifar10_cnn': the convolutional network of the reference's
    examples/cifar10_cnn.py, batch 100 per GPU, momentum SGD; rank 0 also times two updates of
    the same network on the reference's NumpyHandler.  'highway_bn': ten Highway + BatchNorm blocks of width
    4096, batch 8192 in total (strong scaling: 8192 / N rows per GPU), BatchNorm statistics
    completed across the shards inside sum_t(axis=0).  Plain stepper and the same step
    replayed from a recording; at N > 1 the Highway step also reports its phases."""
    why = _reference_on_path()
    if why:
        return {'unavailable': why}
    from brainstorm_b200 import GraphedStepper, workloads
    if name == 'mlp':
        net, data, stepper = workloads.mlp(batch=100, data_seed=rank)
        global_batch, steps, mode = 100 * world, 50, 'local'
    elif name == 'cifar10_cnn':
        net, data, stepper = workloads.cifar10_cnn(batch=100, data_seed=rank)
        global_batch, steps, mode = 100 * world, 50, 'local'
    else:
        net, data, stepper = workloads.highway_bn(batch=8192 // world, blocks=blocks, data_seed=rank)
        global_batch, steps, mode = 8192, 3 if world == 1 else 6, 'avg'
    pinned = {}
    for k, v in data.items():                     # host batches live in page-locked memory, as in lstm_training
        pinned[k] = H.pinned_empty(v.shape, np.float32)
        pinned[k][...] = v
    host_data, data = data, pinned
    net.set_handler(H)
    phase_events, phases_on = {}, [False]

    def mark(tag):
        if phases_on[0]:
            phase_events[tag] = H.record_event(phase_events.get(tag))

    if world > 1:
        from brainstorm_b200.parallel import Comm, data_parallel
        comm = Comm()
        data_parallel(net, comm, axis0_reduce=mode, peer=(name == 'highway_bn'),
                      on_phase=mark if name == 'highway_bn' else None)
    st = stepper()
    st.start(net)

    def step():
        net.provide_external_data(data)
        st.run()
        return float(net.get_loss_values()['total_loss'])

    l0 = lib.b200_launch_count()
    ms, _ = _timed_steps(step, steps, barrier, world)
    out = {'samples_per_s': round(global_batch / ms * 1e3, 1), 'ms_per_step': round(ms, 3), 'global_batch': global_batch,
           'launches_per_step': int((lib.b200_launch_count() - l0) // (steps + 3))}
    if world > 1 and name == 'highway_bn':
        # one more step with the phases bracketed by events on the library stream
        phases_on[0] = True
        fwd0 = net.forward_pass

        def forward_pass(*a, **k):
            mark('start')
            fwd0(*a, **k)
            mark('forward_done')
        net.forward_pass = forward_pass
        step()
        mark('updated')
        phases_on[0] = False
        net.forward_pass = fwd0
        H.synchronize()
        order = ['start', 'forward_done', 'backward_queued', 'reduced', 'updated']
        names = ['forward', 'backward', 'allreduce_tail', 'update']
        out['phases_ms'] = {n: round(_max_over_ranks(elapsed(phase_events[a], phase_events[b]), world), 3)
                            for n, a, b in zip(names, order[:-1], order[1:])}
        # time the host needs to queue one step (no waiting): a step cannot be shorter than this
        H.synchronize()
        t0 = time.perf_counter()
        net.provide_external_data(data)
        st.run()
        out['host_queue_ms'] = round(_max_over_ranks((time.perf_counter() - t0), world) * 1e3, 3)
        H.synchronize()
    if name == 'highway_bn':
        # the same network with the Highway, BatchNorm and FullyConnected layers in their fused forms and the
        # stepper's update as one call (same bits); the recorded step below runs them too
        from brainstorm_b200.fused_layers import fuse_layers
        from brainstorm_b200.steppers import FusedSgdStepper
        fuse_layers(net)
        lr = st.learning_rate
        stepper = lambda: FusedSgdStepper(learning_rate=lr)          # the update as one kernel, same bits
        st = stepper()
        st.start(net)
        l0 = lib.b200_launch_count()
        ms, _ = _timed_steps(step, steps, barrier, world)
        out['fused_layers'] = {'ms_per_step': round(ms, 3), 'samples_per_s': round(global_batch / ms * 1e3, 1),
                               'launches_per_step': int((lib.b200_launch_count() - l0) // (steps + 3))}
        ms = _pipelined_ms(net, lambda: st.run(), H, host_data, data['default'].shape[1], steps + 3, 3, barrier, world)
        out['fused_layers']['pipelined_ms_per_step'] = round(ms, 3)
    if name in ('mlp', 'cifar10_cnn') or world > 1:
        gs = GraphedStepper(stepper(), eager_steps=1)
        gs.start(net)
        st = gs
        ms, _ = _timed_steps(step, steps, barrier, world)
        if gs._step is not None:
            out['recorded_ms_per_step'] = round(ms, 3)
            out['recorded_samples_per_s'] = round(global_batch / ms * 1e3, 1)
        if name == 'mlp' and gs._step is not None:
            # the recorded step with the next batch uploaded during the step and the loss read one call late
            ms = _pipelined_ms(net, lambda: st.run(), H, host_data, data['default'].shape[1], 200, 20, barrier, world)
            out['recorded_pipelined_ms_per_step'] = round(ms, 3)
            out['recorded_pipelined_samples_per_s'] = round(global_batch / ms * 1e3, 1)
        gs.invalidate()
    if name == 'cifar10_cnn' and rank == 0:
        from brainstorm.handlers import NumpyHandler
        ref, rdata, rstepper = workloads.cifar10_cnn(batch=100, data_seed=rank)
        ref.set_handler(NumpyHandler(np.float32))
        rs_ = rstepper()
        rs_.start(ref)
        t0 = time.perf_counter()
        for _ in range(2):
            ref.provide_external_data(rdata)
            rs_.run()
            float(ref.get_loss_values()['total_loss'])
        out['numpy_handler_ms_per_step'] = round((time.perf_counter() - t0) / 2 * 1e3, 1)
    return out


# ------------------------------------------------------------------ GEMM block
GEMM_CASES = [('NT', 8192, 4096, 4096, False, True), ('NN', 8192, 4096, 4096, False, False),
              ('TN', 8192, 4096, 4096, True, False), ('NT_step', 128, 4000, 1000, False, True)]


def gemm_block(H, lib, check, new_event, elapsed, local_rank, peaks):
    """dot_mm on the tensor cores at the shapes of the training workloads: one call timed on
    its own and 400 calls back to back (the power cap then sets the clock), with the SM
    clock seen during the loop.  frac = TFLOP/s over a third of half the measured bf16
    rate (TF32 runs at half the bf16 rate; three TF32 products per fp32 product)."""
    rs = np.random.RandomState(7)
    out = {}
    burst = float(peaks.get('bf16_tflops', 1590.0)) / 6.0
    sustained = float(peaks.get('bf16_tflops_sustained', 1400.0)) / 6.0
    for name, M, N, K, ta, tb in GEMM_CASES:
        a = H.create_from_numpy(rs.uniform(-1, 1, (K, M) if ta else (M, K)).astype(np.float32))
        b = H.create_from_numpy(rs.uniform(-1, 1, (N, K) if tb else (K, N)).astype(np.float32))
        c = H.zeros((M, N))
        for _ in range(3):
            H.dot_mm(a, b, c, transa=ta, transb=tb)
        single = []
        e0, e1 = new_event(), new_event()
        for _ in range(5):
            H.synchronize()
            time.sleep(0.02)
            check(lib.b200_event_record(e0))
            H.dot_mm(a, b, c, transa=ta, transb=tb)
            check(lib.b200_event_record(e1))
            single.append(elapsed(e0, e1))
        reps = 400 if M * N * K > 1e9 else 2000
        sampler = ClockSampler(local_rank)
        H.synchronize()
        t0 = time.time()
        check(lib.b200_event_record(e0))
        for _ in range(reps):
            H.dot_mm(a, b, c, transa=ta, transb=tb)
        check(lib.b200_event_record(e1))
        loop_ms = elapsed(e0, e1) / reps
        clk = sampler.stop(t0, time.time())
        flop = 2.0 * M * N * K
        tf1, tfl = flop / min(single) / 1e9, flop / loop_ms / 1e9
        out['%s_%dx%dx%d' % (name, M, N, K)] = [round(tf1, 1), round(tfl, 1), round(tf1 / burst, 3),
                                                round(tfl / sustained, 3), clk.get('sm_mhz')]
        del a, b, c
    out['columns'] = 'single-call TFLOP/s, loop TFLOP/s, single/burst peak, loop/sustained peak, SM MHz in the loop'
    out['peak_tflops'] = [round(burst, 1), round(sustained, 1)]
    return out


def pin_to_gpu_numa_node(local_rank):
    """With several ranks on one host, run this rank (and so first-touch its page-locked
    buffers) on the CPUs next to its GPU: the e2e leg moves 4.3 GB per step and rank
    across PCIe, and eight ranks otherwise share whichever memory controller the
    kernel happened to pick.  Returns the CPU list used, or None if nothing was changed."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev = torch.cuda.get_device_properties(local_rank).pci_device_id
        path = '/sys/bus/pci/devices/%04x:%02x:%02x.0/local_cpulist' % (dom, bus, dev)
        with open(path) as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(','):
            lo, _, hi = part.partition('-')
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        pin_to_gpu_numa_node.allowed = allowed
        use = cpus & allowed
        if not use or use == allowed:
            return None
        os.sched_setaffinity(0, use)
        return '%d of %d allowed CPUs' % (len(use), len(allowed))
    except Exception:
        return None


# ------------------------------------------------------------------ GPU arm
def run_b200(args):
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit('--gpus %d needs WORLD_SIZE=%d (launch with torch.distributed.run)' % (args.gpus, args.gpus))
    import torch
    import torch.distributed as dist
    from brainstorm_b200 import B200Handler, lib
    from brainstorm_b200._lib import check

    torch.cuda.set_device(local_rank)
    numa = pin_to_gpu_numa_node(local_rank) if world > 1 else None
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local_rank))
    H = B200Handler(seed=SEED + rank, device=local_rank)
    peaks, peak_src = {}, 'fallback'
    try:
        with open(os.path.join(ROOT, 'MEASURED_PEAKS.json')) as f:
            peaks = json.load(f)
        peak, peak_src = float(peaks['hbm_gbs']), 'measured'
    except Exception:
        peak = 6650.0

    def barrier():
        check(lib.b200_sync())
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def new_event():
        e = ctypes.c_uint64()
        check(lib.b200_event_create(ctypes.byref(e)))
        return e.value

    def elapsed(e0, e1):
        ms = ctypes.c_float()
        check(lib.b200_event_elapsed_ms(e0, e1, ctypes.byref(ms)))
        return ms.value

    def finish(line):
        if rank == 0:
            print(json.dumps(line))
        if world > 1:
            barrier()
            dist.destroy_process_group()

    if args.only == 'gemm':
        return run_gemm(args, H, lib, check, new_event, elapsed)
    if args.only == 'ops':
        return run_ops(args, H, lib, check, new_event, elapsed)
    if args.only == 'gemms':
        return finish({'metric': 'dot_mm_fp32_tflops', 'n_gpus': world,
                       'gemm': gemm_block(H, lib, check, new_event, elapsed, local_rank, peaks)})
    if args.only in ('mlp', 'highway_bn', 'cifar10_cnn'):
        res = other_training(args.only, H, world, rank, barrier, lib, new_event, elapsed, blocks=args.blocks)
        return finish({'metric': '%s_train_samples_per_s' % args.only, 'value': res.get('samples_per_s'),
                       'unit': 'samples/s', 'n_gpus': world, 'detail': res})
    if args.only == 'lstm':
        lstm = lstm_training(H, world, rank, max(1, args.steps), barrier, lib)
        return finish({'metric': 'lstm_train_sequences_per_s', 'value': lstm.get('sequences_per_s'),
                       'unit': 'sequences/s', 'n_gpus': world, 'lstm': lstm})
    ROWS = args.rows
    # ---- operands: page-locked host copies (for e2e) and device-resident arrays
    host = host_inputs(ROWS, COLS, SEED + rank, alloc=H.pinned_empty)
    t = {k: H.create_from_numpy(v) for k, v in host.items()}
    t['out'] = H.zeros((ROWS, COLS))
    t['y'] = H.zeros((ROWS, COLS))
    t['absa'] = H.zeros((ROWS, COLS))
    H.tanh(t['a'], t['y'])
    H.abs_t(t['a'], t['absa'])
    t['s0'] = H.zeros((1, COLS))
    t['s1'] = H.zeros((ROWS, 1))
    t['sall'] = H.zeros(())
    t['picked'] = H.zeros((ROWS, 1))
    suite = make_suite(H, t)
    nbytes = dict(suite_bytes(ROWS, COLS))
    step_bytes = sum(nbytes.values())

    # ---- sharded rows: sum_t(axis=0) is completed across the shards by the handler itself
    # (H.set_comm: stream-ordered, no host wait), over the library's peer-memory kernel
    peer_ok, comm = None, None
    if world > 1:
        from brainstorm_b200.parallel import Comm
        comm = Comm()
        peer_on = comm.enable_peer()
        # self-check outside the timed region: the peer kernel against NCCL, replicas bit-equal
        rs = np.random.RandomState(100 + rank)
        x = rs.randn(COLS).astype(np.float32)
        a_peer, a_nccl = H.create_from_numpy(x), H.create_from_numpy(x)
        comm.allreduce(a_peer, 'sum')
        check(lib.b200_comm_allreduce(a_nccl.ptr, a_nccl.size, 0)) if comm._lib_nccl else Comm(library_nccl=False).allreduce(a_nccl, 'sum')
        got, want = H.get_numpy_copy(a_peer), H.get_numpy_copy(a_nccl)
        gathered = [None] * world
        dist.all_gather_object(gathered, got)
        peer_ok = bool(peer_on and all(np.array_equal(g, gathered[0]) for g in gathered) and
                       np.allclose(got, want, rtol=1e-6, atol=1e-6))
        H.set_comm(comm, 'sum')

    def step(events=None):
        for i, (name, fn) in enumerate(suite):
            if events is not None:
                check(lib.b200_event_record(events[i][0]))
            fn()
            if events is not None:
                check(lib.b200_event_record(events[i][1]))

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- device-resident timing: K steps, per-op events inside the timed region
    per_step_events = [[(new_event(), new_event()) for _ in suite] for _ in range(args.steps)]
    e_start, e_stop = new_event(), new_event()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = lib.b200_launch_count()
    waits0 = comm.peer_wait_stats() if peer_ok else None
    barrier()
    t0 = time.time()
    check(lib.b200_event_record(e_start))
    for k in range(args.steps):
        step(per_step_events[k])
    check(lib.b200_event_record(e_stop))
    barrier()
    t1 = time.time()
    axis0_wait_us = None
    if waits0 is not None:
        # how long the exchange inside sum_t(axis=0) waited for the slowest rank: [least, most] patient rank
        calls, waited = comm.peer_wait_stats()
        mine = (waited - waits0[1]) / max(1, calls - waits0[0]) * 1e6
        axis0_wait_us = [round(-_max_over_ranks(-mine, world), 1), round(_max_over_ranks(mine, world), 1)]
    launches = lib.b200_launch_count() - launches0
    total_ms = _max_over_ranks(elapsed(e_start, e_stop), world)
    clocks = sampler.stop(t0, t1) if sampler else None
    ms_per_step = total_ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    op_ms = {}
    for i, (name, _) in enumerate(suite):
        op_ms[name] = float(np.mean([elapsed(*per_step_events[k][i]) for k in range(args.steps)]))
    ops = {name: [round(ms, 4), round(nbytes[name] / (ms * 1e-3) / 1e9)] for name, ms in op_ms.items()}

    if args.only == 'suite':
        return finish({'metric': METRIC, 'value': round(value, 1), 'unit': UNIT, 'n_gpus': world,
                       'steps': args.steps, 'ms_per_step': round(ms_per_step, 4),
                       'config': {'workload': 'handler op suite only, (%d, %d)' % (ROWS, COLS)},
                       'gpu_launches': int(launches), 'peer_ok': peer_ok, 'axis0_exchange_wait_us': axis0_wait_us,
                       'ops_ms_gbs': ops})
    # ---- end to end: host buffers in, results out, every step
    e2e_steps = max(2, min(args.steps, 4))
    results = [np.empty((1, COLS), np.float32), np.empty((ROWS, 1), np.float32),
               np.empty((), np.float32), np.empty((ROWS, 1), np.float32)]
    names = ('a', 'b', 'dy', 'div', 'row', 'col', 'labels')
    h2d = sum(host[k].nbytes for k in names)
    d2h = sum(r.nbytes for r in results)

    # Double-buffered operands: while the suite runs on one set, the next step's host
    # buffers are uploaded into the other set on the upload stream.
    sets = [t, dict(t)]
    for k in names:
        sets[1][k] = H.allocate(t[k].shape)
    suites = [suite, make_suite(H, sets[1])]
    done = [0, 0]

    def upload(which, after):
        for k in names:
            H.upload_async(sets[which][k], host[k], after)

    def e2e_run(n):
        upload(0, 0)                                   # step 0's inputs: nothing to overlap with
        H.upload_join()
        for k in range(n):
            cur, nxt = k % 2, (k + 1) % 2
            if k + 1 < n:
                upload(nxt, done[nxt])                 # after the kernels that last read that set
            for name, fn in suites[cur]:
                fn()
            done[cur] = H.record_event(done[cur] or None)
            for r, key in zip(results, ('s0', 's1', 'sall', 'picked')):
                r[...] = H.get_numpy_copy(sets[cur][key])
            H.upload_join()

    e2e_run(2)
    barrier()
    w0 = time.perf_counter()
    e2e_run(e2e_steps)
    barrier()
    e2e_s = _max_over_ranks((time.perf_counter() - w0) / e2e_steps, world)
    e2e_value = world * step_bytes / e2e_s / 1e9
    H.set_comm(None, 'local')
    del t, suite, suites, sets, host
    import gc
    gc.collect()

    gemm = gemm_block(H, lib, check, new_event, elapsed, local_rank, peaks)
    lstm = lstm_training(H, world, rank, max(3, min(args.steps, 10)), barrier, lib)
    others = {n: other_training(n, H, world, rank, barrier, lib, new_event, elapsed) for n in ('mlp', 'cifar10_cnn', 'highway_bn')}
    if comm is not None:
        comm.close()

    line = None
    if rank == 0:
        traffic = None
        try:
            with open(os.path.join(ROOT, 'profiles', 'ncu_traffic.txt')) as f:
                traffic = json.load(f).get('ew_flat_vec_add_tt_bytes_per_launch_1gib')
        except Exception:
            pass
        dom = 'add_tt'
        achieved = nbytes[dom] / (op_ms[dom] * 1e-3) / 1e9
        threads = os.cpu_count() or 1
        if getattr(pin_to_gpu_numa_node, 'allowed', None):
            os.sched_setaffinity(0, pin_to_gpu_numa_node.allowed)      # the CPU leg uses every host thread
        cgbs, cdt, ckind = cpu_suite_time(CPU_SAMPLE_ROWS, COLS, SEED, threads, 2, 1)
        cpu = {'value': round(cgbs, 3), 'unit': UNIT, 'cores': threads, 'kind': ckind,
               'sample': '%d of %d rows per step (same %d columns, same ops), 2 steps after 1 warm-up, '
                         'row chunks over %d threads' % (CPU_SAMPLE_ROWS, ROWS, COLS, threads)}
        line = {
            'metric': METRIC, 'value': round(value, 1), 'unit': UNIT, 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': round(ms_per_step, 4),
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32',
            'data': 'synthetic (seeded draw of the whole operands)',
            'config': {'workload': 'handler op suite (27 ops), fp32 (%d, %d) operands per GPU, '
                                   '%.3g GiB each' % (ROWS, COLS, ROWS * COLS * 4 / 2.0 ** 30),
                       'rows_per_gpu': ROWS, 'cols': COLS, 'seed': SEED,
                       'l2': 'operands (1 GiB) exceed L2 (126 MB); no flush needed',
                       'sharding': 'rows; axis-0 sum completed across shards inside sum_t (peer-memory kernel)'
                       if world > 1 else 'single GPU', 'numa_pinning': numa},
            'e2e': {'value': round(e2e_value, 1), 'unit': UNIT, 'h2d_bytes_per_step': int(h2d),
                    'd2h_bytes_per_step': int(d2h), 'steps': e2e_steps},
            'gpu_launches': int(launches),
            'clocks': clocks,
            'roofline': {'bound': 'hbm', 'kernel': 'ew_flat_vec<FAdd> (add_tt)', 'achieved': round(achieved, 1),
                         'peak': peak, 'peak_source': peak_src, 'unit': 'GB/s',
                         'frac': round(achieved / peak, 4), 'traffic': traffic},
            'cpu_baseline': cpu,
            'ops_ms_gbs': ops,
            # the short blocks come last: the second half of the metric must survive a truncated record
            'gemm': gemm,
            'other_training': others,
            'peer_ok': peer_ok,
            'axis0_exchange_wait_us': axis0_wait_us,
            'lstm': lstm,
        }
    finish(line)


def run_ops(args, H, lib, check, new_event, elapsed):
    """--only ops --ops a,b,...: the named ops of the suite, each `steps` times back to back,
    on device-generated operands of (rows, 4096); only the operands those ops need are
    allocated.  For profiler captures of single kernels and for launch-shape comparisons."""
    rows = args.rows
    want = [o for o in args.ops.split(',') if o]
    t = {}
    big = lambda: H.allocate((rows, COLS))
    need = {'a'}
    for o in want:
        need |= {'out'} if not o.startswith(('sum_t', 'index')) else set()
        need |= {'b'} if o in ('add_tt', 'subtract_tt', 'mult_tt') else set()
        need |= {'div'} if o == 'divide_tt' else set()
        need |= {'y', 'dy'} if o.endswith('_deriv') else set()
        need |= {'absa'} if o == 'sqrt_t' else set()
    for k in ('a', 'b', 'dy', 'div'):
        if k in need:
            t[k] = big()
            H.fill_gaussian(0.5 if k == 'div' else 0.0, 2.0, t[k])
    for k in ('out', 'y', 'absa'):
        if k in need:
            t[k] = big()
    if 'y' in t:
        H.tanh(t['a'], t['y'])
    if 'absa' in t:
        H.abs_t(t['a'], t['absa'])
    t['row'], t['col'] = H.allocate((1, COLS)), H.allocate((rows, 1))
    H.fill_gaussian(0.0, 1.0, t['row'])
    H.fill_gaussian(0.0, 1.0, t['col'])
    t['labels'] = H.create_from_numpy(np.random.RandomState(SEED).randint(0, COLS, (rows, 1)).astype(np.float32))
    t['s0'], t['s1'], t['sall'], t['picked'] = H.zeros((1, COLS)), H.zeros((rows, 1)), H.zeros(()), H.zeros((rows, 1))
    for k in ('a', 'b', 'dy', 'div', 'out', 'y', 'absa'):
        t.setdefault(k, t['a'])
    suite = dict(make_suite(H, t))
    nbytes = dict(suite_bytes(rows, COLS))
    res = {}
    e0, e1 = new_event(), new_event()
    for o in want:
        for _ in range(max(args.warmup, 1)):
            suite[o]()
        check(lib.b200_event_record(e0))
        for _ in range(args.steps):
            suite[o]()
        check(lib.b200_event_record(e1))
        ms = elapsed(e0, e1) / args.steps
        res[o] = [round(ms, 4), round(nbytes[o] / (ms * 1e-3) / 1e9)]
    print(json.dumps({'metric': 'handler_op_throughput', 'unit': 'GB/s', 'config': {'workload': 'single ops, (%d, %d)' % (rows, COLS)},
                      'steps': args.steps, 'ops_ms_gbs': res}))


def run_gemm(args, H, lib, check, new_event, elapsed):
    """--only gemm: times dot_mm (a . b^T) at one shape on the tensor-core path and
    on the CUDA-core path; used for the ncu captures of the GEMM kernel."""
    M, N, K = [int(v) for v in args.gemm.split(',')]
    rs = np.random.RandomState(SEED)
    a = H.create_from_numpy(rs.uniform(-1, 1, (M, K)).astype(np.float32))
    b = H.create_from_numpy(rs.uniform(-1, 1, (N, K)).astype(np.float32))
    out = H.zeros((M, N))
    res = {}
    for name, path in (('tensor_core_tf32x3', 2), ('cuda_core_fp32', 1)):
        check(lib.b200_set_tuning(2, path))
        for _ in range(3):
            H.dot_mm(a, b, out, transb=True)
        e0, e1 = new_event(), new_event()
        reps = args.steps if path == 2 else max(1, args.steps // 4)
        check(lib.b200_event_record(e0))
        for _ in range(reps):
            H.dot_mm(a, b, out, transb=True)
        check(lib.b200_event_record(e1))
        ms = elapsed(e0, e1) / reps
        res[name] = {'ms': round(ms, 4), 'tflops': round(2.0 * M * N * K / ms / 1e9, 1)}
    check(lib.b200_set_tuning(2, 0))
    print(json.dumps({'metric': 'dot_mm_fp32_tflops', 'value': res['tensor_core_tf32x3']['tflops'],
                      'unit': 'TFLOP/s', 'config': {'workload': 'dot_mm NT %dx%dx%d' % (M, N, K)},
                      'paths': res}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=30)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--only', default='all', choices=['all', 'suite', 'ops', 'gemm', 'gemms', 'lstm', 'mlp', 'cifar10_cnn', 'highway_bn'],
                    help='suite: device-resident op suite only; gemm: one dot_mm shape (for profiling); '
                         'gemms: the GEMM block of the bench line')
    ap.add_argument('--rows', type=int, default=ROWS, help='rows of the op-suite operands (default 65536)')
    ap.add_argument('--gemm', default='8192,4096,4096', help='M,N,K for --only gemm')
    ap.add_argument('--ops', default='add_tt', help='comma-separated op names for --only ops')
    ap.add_argument('--blocks', type=int, default=10, help='Highway + BatchNorm blocks for --only highway_bn (profiler captures use 1)')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_b200(args)


if __name__ == '__main__':
    main()
