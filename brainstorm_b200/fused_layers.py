"""Drop-in fused Highway, BatchNorm and FullyConnected layers for networks that run
on ``B200Handler``.

The reference's layers spell their arithmetic as chains of handler calls
(brainstorm/layers/highway_layer.py:39-71, batch_normalization_layer.py:54-152,
fully_connected_layer.py:51-62).  On a GPU every call of such a chain is a kernel
that streams its operands through HBM once more: ten array streams for the Highway
forward pass where four suffice, nineteen for its backward pass where ten do,
eighteen for the BatchNorm backward pass where six do.  The classes below subclass
the reference's layer classes, keep ``setup`` (parameters, internals, shapes,
memory layout, saved networks) untouched and replace only ``forward_pass`` /
``backward_pass`` by one library call per pass over the data (``b200_highway_*``,
``b200_bn_*``, ``b200_bias_act``).  Every product, sum and quotient is rounded
separately and in the chain's order, so a network computes the same bits with or
without them; every buffer the reference layer leaves filled is filled (the
BatchNorm layer's ``centered`` and ``x_hat`` internals included).

    net.set_handler(B200Handler())
    fuse_layers(net)          # swaps the classes of these layers in place

Operands the kernels cannot take (views that are not contiguous, not 16-byte
aligned, or whose width is not a multiple of 4) go through the reference's own
method of the parent class, call by call.

Data parallelism: the BatchNorm statistics are completed across batch shards exactly
where the chain's ``sum_t(axis=0)`` calls would complete them (``B200Handler.set_comm``).
"""
from __future__ import annotations

from brainstorm.layers.batch_normalization_layer import BatchNormLayerImpl
from brainstorm.layers.fully_connected_layer import FullyConnectedLayerImpl
from brainstorm.layers.highway_layer import HighwayLayerImpl
from brainstorm.utils import flatten_all_but_last, flatten_time_and_features

from ._lib import lib, check
from .array import B200Array
from .handler import B200Handler, _matrix

_ACT = {'sigmoid': 0, 'tanh': 1, 'rel': 2, 'el': 3, 'linear': 4}


def _flat_ok(*arrays):
    """Contiguous, 16-byte aligned, a multiple of 4 elements, all of one size."""
    n = arrays[0].size
    for a in arrays:
        if not isinstance(a, B200Array) or not a._contig or a.ptr % 16 or a.size != n:
            return False
    return n % 4 == 0


def _complete_axis0(handler, dst):
    """What ``B200Handler.sum_t(axis=0)`` does after the local sum: complete it across
    batch shards when a communicator is set."""
    if handler._comm is not None and handler.axis0_reduce != 'local':
        handler._allreduce_axis0(dst)


class FusedHighwayLayerImpl(HighwayLayerImpl):
    """``HighwayLayerImpl`` (brainstorm/layers/highway_layer.py:21) with each pass as one kernel."""

    def forward_pass(self, buffers, training_pass=True):
        x, H, T = buffers.inputs.x, buffers.inputs.H, buffers.inputs.T
        y = buffers.outputs.default
        if not (isinstance(self.handler, B200Handler) and _flat_ok(x, H, T, y)):
            return HighwayLayerImpl.forward_pass(self, buffers, training_pass)
        check(lib.b200_highway_forward(x.ptr, H.ptr, T.ptr, y.ptr, x.size))

    def backward_pass(self, buffers):
        x, H, T = buffers.inputs.x, buffers.inputs.H, buffers.inputs.T
        dx, dH, dT = buffers.input_deltas.x, buffers.input_deltas.H, buffers.input_deltas.T
        dy = buffers.output_deltas.default
        if not (isinstance(self.handler, B200Handler) and _flat_ok(x, H, T, dy, dx, dH, dT)):
            return HighwayLayerImpl.backward_pass(self, buffers)
        check(lib.b200_highway_backward(x.ptr, H.ptr, T.ptr, dy.ptr, dx.ptr, dH.ptr, dT.ptr, x.size))


class FusedBatchNormLayerImpl(BatchNormLayerImpl):
    """``BatchNormLayerImpl`` (brainstorm/layers/batch_normalization_layer.py:23): three passes
    over the data forward (column sums; centering with the sums of squares; normalisation with
    scale and shift) and two backward (both column sums; the input deltas)."""

    _work = None        # (features, sums(2F), vectors(3F)) of the backward pass, made on first use

    def _small(self, features):
        if self._work is None or self._work[0] != features:
            self._work = (features, B200Array.empty((2 * features,), zero=False),
                          B200Array.empty((3 * features,), zero=False))
        return self._work[1], self._work[2]

    def forward_pass(self, buffers, training_pass=True):
        h = self.handler
        sigma_b, centered, x_hat = buffers.internals
        gamma, beta, mu, sigma = buffers.parameters
        inputs = flatten_all_but_last(buffers.inputs.default)
        out = flatten_all_but_last(buffers.outputs.default)
        m, f = inputs.shape
        small = (gamma, beta, mu, sigma, sigma_b)
        if not (isinstance(h, B200Handler) and _flat_ok(inputs, centered, x_hat, out) and f % 4 == 0 and
                all(isinstance(v, B200Array) and v._contig and v.ptr % 16 == 0 for v in small)):
            return BatchNormLayerImpl.forward_pass(self, buffers, training_pass)
        if training_pass:
            mu_b = sigma_b
            h.sum_t(inputs, 0, mu_b)                    # completed across batch shards by the handler
            check(lib.b200_bn_mean(mu_b.ptr, -1.0 / m, self.decay, 1.0 - self.decay, mu_b.ptr, mu.ptr, f))
            sp, sn = h._scratch_for(lib.b200_bn_scratch_floats(m, f))
            sq = self._small(f)[0]
            check(lib.b200_bn_center_sqsum(inputs.ptr, mu_b.ptr, centered.ptr, sq.ptr, m, f, sp, sn))
            _complete_axis0(h, sq[:f])
            check(lib.b200_bn_sigma(sq.ptr, 1.0 / m, self.epsilon, self.decay, 1.0 - self.decay, sigma_b.ptr, sigma.ptr, f))
            sigma = sigma_b
        else:
            h.add_mv(inputs, mu.reshape((1, mu.size)), flatten_all_but_last(centered))
        check(lib.b200_bn_normalize(centered.ptr, sigma.ptr, gamma.ptr, beta.ptr, x_hat.ptr, out.ptr, m, f))

    def backward_pass(self, buffers):
        h = self.handler
        sigma_b, centered, x_hat = buffers.internals
        gamma = buffers.parameters.gamma
        dgamma, dbeta = buffers.gradients.gamma, buffers.gradients.beta
        outdeltas = flatten_all_but_last(buffers.output_deltas.default)
        indeltas = flatten_all_but_last(buffers.input_deltas.default)
        m, f = outdeltas.shape
        small = (gamma, sigma_b, dgamma, dbeta)
        if not (isinstance(h, B200Handler) and _flat_ok(outdeltas, x_hat, indeltas) and f % 4 == 0 and
                all(isinstance(v, B200Array) and v._contig and v.ptr % 16 == 0 for v in small)):
            return BatchNormLayerImpl.backward_pass(self, buffers)
        sums, vec = self._small(f)
        sp, sn = h._scratch_for(lib.b200_bn_scratch_floats(m, f))
        check(lib.b200_bn_backward_sums(outdeltas.ptr, x_hat.ptr, sums.ptr, m, f, sp, sn))
        _complete_axis0(h, sums)
        check(lib.b200_bn_backward_vectors(sums.ptr, 1 / m, gamma.ptr, sigma_b.ptr, dgamma.ptr, dbeta.ptr, vec.ptr, f))
        check(lib.b200_bn_backward_deltas(outdeltas.ptr, x_hat.ptr, vec.ptr, indeltas.ptr, m, f))


class FusedFullyConnectedLayerImpl(FullyConnectedLayerImpl):
    """``FullyConnectedLayerImpl`` (brainstorm/layers/fully_connected_layer.py:21) whose forward pass
    adds the bias and applies the activation in one kernel after the GEMM."""

    def forward_pass(self, buffers, training_pass=True):
        h = self.handler
        W, bias = buffers.parameters
        inputs = flatten_time_and_features(buffers.inputs.default)
        outputs = flatten_time_and_features(buffers.outputs.default)
        act = _ACT.get(self.activation)
        ok = isinstance(h, B200Handler) and act is not None and isinstance(outputs, B200Array) and bias._contig
        if ok:
            try:
                rows, cols, ld = _matrix(outputs)
            except NotImplementedError:
                ok = False
        if not ok or cols % 4 or ld % 4 or outputs.ptr % 16 or bias.ptr % 16:
            return FullyConnectedLayerImpl.forward_pass(self, buffers, training_pass)
        h.dot_mm(inputs, W, outputs, transb=True)
        check(lib.b200_bias_act(outputs.ptr, bias.ptr, rows, cols, ld, act))


_SWAPS = ((HighwayLayerImpl, FusedHighwayLayerImpl), (BatchNormLayerImpl, FusedBatchNormLayerImpl),
          (FullyConnectedLayerImpl, FusedFullyConnectedLayerImpl))


def fuse_layers(net):
    """Swap every Highway, BatchNorm and FullyConnected layer of ``net`` for its fused form, in
    place.  Returns the names of the layers that were swapped."""
    swapped = []
    for name, layer in net.layers.items():
        for plain, fused in _SWAPS:
            if type(layer) is plain:
                layer.__class__ = fused
                swapped.append(name)
    return swapped
