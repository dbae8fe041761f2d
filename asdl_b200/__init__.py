"""asdl_b200: second-order gradient preconditioning for PyTorch on Blackwell (sm_100a).

The public surface mirrors the flat namespace of ASDL (asdl/__init__.py:1-17): the
``GradientMaker`` interface, curvature containers, per-layer statistics, Fisher / Hessian /
kernel utilities and the preconditioned gradient makers.
"""
from .utils import *  # noqa: F401,F403
from .vector import *  # noqa: F401,F403
from .symmatrix import *  # noqa: F401,F403
from .matrices import *  # noqa: F401,F403
from .operations import *  # noqa: F401,F403
from .core import *  # noqa: F401,F403
from .grad_maker import *  # noqa: F401,F403
from .mvp import *  # noqa: F401,F403
from .fisher import *  # noqa: F401,F403
from .hessian import *  # noqa: F401,F403
from .gradient import *  # noqa: F401,F403
from .precondition import *  # noqa: F401,F403
from .kernel import *  # noqa: F401,F403
from .counter import *  # noqa: F401,F403
from . import ops, parallel  # noqa: F401

__version__ = '0.1.0'
