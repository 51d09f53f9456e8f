"""The abstract ``Handler`` interface that ``B200Handler`` implements.

When the brainstorm library is importable, its own base class
(brainstorm/handlers/base_handler.py:13) is used, so that ``B200Handler`` is a
genuine ``Handler``/``Describable`` for ``Network.set_handler``.  Without it, a
minimal stand-in with the same constructor behaviour (the four activation
dispatch tables of base_handler.py:41-72) lets the backend be used and tested on
its own.  This is interface plumbing only: no arithmetic lives here.
"""
from __future__ import annotations

import numpy as np

try:
    from brainstorm.handlers.base_handler import Handler  # noqa: F401
    from brainstorm.randomness import global_rnd
    HAVE_BRAINSTORM = True

    def new_random_state(seed=None):
        return global_rnd.create_random_state(seed)

except ImportError:
    HAVE_BRAINSTORM = False

    def new_random_state(seed=None):
        return np.random.RandomState(seed)

    class Handler(object):
        """Stand-in for brainstorm's abstract handler base class."""

        def __init__(self):
            self.inplace_act_func = {
                'sigmoid': lambda x: self.sigmoid(x, x),
                'tanh': lambda x: self.tanh(x, x),
                'rel': lambda x: self.rel(x, x),
                'el': lambda x: self.el(x, x),
                'linear': lambda x: None,
            }
            self.inplace_act_func_deriv = {
                'sigmoid': lambda y, dy: self.sigmoid_deriv(y, y, dy, dy),
                'tanh': lambda y, dy: self.tanh_deriv(y, y, dy, dy),
                'rel': lambda y, dy: self.rel_deriv(y, y, dy, dy),
                'el': lambda y, dy: self.el_deriv(y, y, dy, dy),
                'linear': lambda y, dy: None,
            }
            self.act_func = {
                'sigmoid': self.sigmoid, 'tanh': self.tanh, 'rel': self.rel,
                'el': self.el, 'linear': self.copy_to,
            }
            self.act_func_deriv = {
                'sigmoid': self.sigmoid_deriv, 'tanh': self.tanh_deriv,
                'rel': self.rel_deriv, 'el': self.el_deriv,
                'linear': lambda x, y, dy, dx: self.copy_to(dy, dx),
            }

        def __init_from_description__(self, description):
            Handler.__init__(self)
