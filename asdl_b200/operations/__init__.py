"""Per-layer statistics extractors.  ``get_op_class`` maps an ``nn.Module`` to its extractor.
Parity: asdl/operations/__init__.py:1-79."""
import warnings

from torch import nn

from .operation import *  # noqa: F401,F403
from .operation import __all__ as _operation_all
from .operation import (SHAPE_FULL, SHAPE_LAYER_WISE, SHAPE_KRON, SHAPE_SWIFT_KRON, SHAPE_KFE, SHAPE_UNIT_WISE,  # noqa: F401
                        SHAPE_DIAG, HESSIAN, FISHER_EXACT, FISHER_MC, FISHER_EMP)
from .linear import Linear
from .conv import Conv2d
from .batchnorm import BatchNorm1d, BatchNorm2d
from .layernorm import LayerNorm
from .embedding import Embedding
from .bias import Bias, BiasExt
from .scale import Scale, ScaleExt

__all__ = ['Linear', 'Conv2d', 'BatchNorm1d', 'BatchNorm2d', 'LayerNorm', 'Embedding', 'Bias',
           'Scale', 'BiasExt', 'ScaleExt', 'get_op_class'] + list(_operation_all)

_REGISTRY = [
    (nn.Linear, Linear), (nn.Conv2d, Conv2d), (nn.BatchNorm1d, BatchNorm1d),
    (nn.BatchNorm2d, BatchNorm2d), (nn.LayerNorm, LayerNorm), (nn.Embedding, Embedding),
    (Bias, BiasExt), (Scale, ScaleExt),
]


def get_op_class(module):
    """Extractor class for ``module`` (first matching entry), or None with a warning."""
    for module_cls, op_cls in _REGISTRY:
        if isinstance(module, module_cls):
            return op_cls
    warnings.warn(f'Failed to lookup operations for Module {module}.')
    return None
