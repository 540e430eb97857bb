"""Blackwell-native expert-parallel communication library (same public names as ``deep_ep``,
deep_ep/__init__.py:93-107): ``ElasticBuffer``, ``EPHandle``, ``Buffer``, ``Config``, ``EventOverlap``,
``EventHandle``, ``topk_idx_t``, ``get_physical_domain_size``, ``get_logical_domain_size``."""
from . import _native

_native.apply_persistent_envs()      # before anything reads them (topk_idx_t is fixed at import)

from .buffers.elastic import ElasticBuffer, EPHandle, topk_idx_t  # noqa: E402
from .utils.event import EventHandle, EventOverlap  # noqa: E402
from .utils.envs import get_logical_domain_size, get_physical_domain_size  # noqa: E402

__version__ = '0.1.0'

__all__ = ['ElasticBuffer', 'EPHandle', 'EventOverlap', 'EventHandle', 'topk_idx_t',
           'get_physical_domain_size', 'get_logical_domain_size']


def __getattr__(name):
    # the legacy-style API is imported lazily: it pulls in the low-latency kernels
    if name in ('Buffer', 'Config'):
        from .buffers import legacy
        return getattr(legacy, name)
    raise AttributeError(name)
