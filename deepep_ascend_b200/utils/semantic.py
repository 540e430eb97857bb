"""Small helpers shared by the Python layer (parity: deep_ep/utils/semantic.py:5-27)."""
import functools
import weakref
from typing import Any, Callable


def value_or(value: Any, default: Any) -> Any:
    """Return ``value`` unless it is ``None``."""
    return default if value is None else value


def weak_lru(maxsize: int = 128) -> Callable:
    """``functools.lru_cache`` for methods that keeps only a weak reference to ``self``,
    so a cached method never extends the life of the buffer that owns it."""

    def decorator(func: Callable) -> Callable:
        @functools.lru_cache(maxsize)
        def _cached(self_ref, *args, **kwargs):
            return func(self_ref(), *args, **kwargs)

        @functools.wraps(func)
        def wrapper(self, *args, **kwargs):
            return _cached(weakref.ref(self), *args, **kwargs)

        wrapper.cache_clear = _cached.cache_clear
        return wrapper

    return decorator
