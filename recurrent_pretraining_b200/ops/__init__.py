"""Op set: ``reference`` (PyTorch statements / CPU path), ``functional`` (autograd front end),
``cuda`` (ctypes binding of the sm_100a kernel library; imported lazily, GPU only)."""
from . import functional, reference  # noqa: F401
