"""In-tree build and loading of the sm_100a CUDA extension.

The shared object is compiled next to the sources (``asdl_b200/csrc/_build``) so that it travels
with the source tree; nothing is installed into site-packages and nothing depends on a per-user
JIT cache.  ``load()`` imports an up-to-date binary directly and only invokes ninja/nvcc when a
source file changed.
"""
import hashlib
import importlib.machinery
import importlib.util
import os
import sys
import threading

_NAME = 'asdl_b200_C'
_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'csrc')
_BUILD = os.path.join(_CSRC, '_build')
_lock = threading.Lock()
_module = None

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
    '--expt-relaxed-constexpr', '-Xptxas', '-v',
]


def sources():
    return sorted(os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith('.cu'))


def _digest():
    h = hashlib.sha256()
    for f in sorted(os.listdir(_CSRC)):
        if f.endswith(('.cu', '.cuh', '.h')):
            h.update(f.encode())
            with open(os.path.join(_CSRC, f), 'rb') as fh:
                h.update(fh.read())
    h.update(' '.join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _so_path():
    return os.path.join(_BUILD, _NAME + '.so')


def _import_so():
    import torch  # noqa: F401  (libtorch symbols must be loaded first)
    loader = importlib.machinery.ExtensionFileLoader(_NAME, _so_path())
    spec = importlib.util.spec_from_loader(_NAME, loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules[_NAME] = mod
    return mod


def is_built():
    stamp = os.path.join(_BUILD, 'digest.txt')
    return (os.path.exists(_so_path()) and os.path.exists(stamp)
            and open(stamp).read().strip() == _digest())


def build(verbose=False):
    """Compile every .cu under csrc/ for sm_100a (cross-compiles without a GPU)."""
    from torch.utils import cpp_extension
    digest = _digest()  # of the sources as they are now, not as they are when the build ends
    os.makedirs(_BUILD, exist_ok=True)
    os.environ.setdefault('TORCH_CUDA_ARCH_LIST', '10.0a')
    os.environ.setdefault('MAX_JOBS', str(min(8, os.cpu_count() or 4)))
    cpp_extension.load(name=_NAME, sources=sources(), extra_cuda_cflags=NVCC_FLAGS,
                       extra_cflags=['-O3', '-std=c++17'], build_directory=_BUILD,
                       verbose=verbose, is_python_module=False)
    with open(os.path.join(_BUILD, 'digest.txt'), 'w') as fh:
        fh.write(digest)


def load(allow_build=True):
    """Returns the extension module, building it first if it is missing or stale."""
    global _module
    with _lock:
        if _module is not None:
            return _module
        if not is_built():
            if not allow_build:
                raise ImportError(
                    f'{_NAME} is not built; run `python -c "import __graft_entry__ as g; g.build()"`')
            build()
        _module = _import_so()
        return _module
