"""Preconditioned gradient makers (parity: asdl/precondition/__init__.py)."""
from .prec_grad_maker import *  # noqa: F401,F403
from .natural_gradient import *  # noqa: F401,F403
