"""Drop-in steppers for networks that run on ``B200Handler``.

``FusedSgdStepper`` is the reference's ``SgdStepper`` (brainstorm/training/steppers.py:46-69)
with the update written as one handler call.  The reference computes
``update = -learning_rate * gradients`` and then ``parameters = update + parameters``:
two kernels and five trips of the flat parameter-sized vector through HBM.
``mult_add_st(-learning_rate, gradients, out=parameters)`` (base_handler.py:284) rounds the
product and then the sum, the same two roundings, in one kernel and three trips, so the
parameters get the same bits.  The stepper's ``update`` buffer is allocated as in the
reference but not written.
"""
from __future__ import annotations

from brainstorm.training.steppers import SgdStepper


class FusedSgdStepper(SgdStepper):
    """Stochastic gradient descent; same arguments, schedules and description as ``SgdStepper``."""

    def run(self):
        self.net.forward_pass(training_pass=True)
        self.net.backward_pass()
        self.net.handler.mult_add_st(-self.learning_rate, self.net.buffer.gradients,
                                     out=self.net.buffer.parameters)
