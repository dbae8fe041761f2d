"""Preconditioned gradient makers (parity: asdl/precondition/__init__.py)."""
from .prec_grad_maker import *  # noqa: F401,F403
from .natural_gradient import *  # noqa: F401,F403
from .shampoo import *  # noqa: F401,F403
from .psgd import *  # noqa: F401,F403
from .smw import *  # noqa: F401,F403
from .newton import *  # noqa: F401,F403
from .kbfgs import *  # noqa: F401,F403
from .curve_ball import *  # noqa: F401,F403
from .seng import *  # noqa: F401,F403
from .kfac_fused import *  # noqa: F401,F403
