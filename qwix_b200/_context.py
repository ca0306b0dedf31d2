"""Per-thread state that stands in for qwix's interception layer on this backend.

The reference patches jax.lax.dot_general & co. while a quantized model runs
(qwix/_src/interception.py:187-410) and finds the calling module through Flax.  Here the
modules call qwix_b200.ops explicitly; this file keeps, per thread, which provider is
active, the path of the module being executed and the per-module op counters
(qwix/_src/aux_data.py, qconfig.py:224-232).
"""

from __future__ import annotations

import contextlib
import threading

_state = threading.local()


def _s():
  if not hasattr(_state, 'provider'):
    _state.provider = None
    _state.modules = []   # stack of (module, path tuple)
    _state.counters = {}  # (id(module), key) -> int
  return _state


def current_provider():
  return _s().provider


def current_module():
  st = _s()
  return st.modules[-1][0] if st.modules else None


def current_module_path() -> tuple[str, ...]:
  st = _s()
  return st.modules[-1][1] if st.modules else ()


@contextlib.contextmanager
def provider_scope(provider):
  """Activates `provider` for ops issued by this thread; not re-entrant on purpose
  (interception.py is non-recursive as well)."""
  st = _s()
  prev, prev_counters = st.provider, st.counters
  st.provider, st.counters = provider, {}
  try:
    yield
  finally:
    st.provider, st.counters = prev, prev_counters


@contextlib.contextmanager
def disabled():
  """Runs ops un-intercepted (the reference's disable_interceptions)."""
  st = _s()
  prev = st.provider
  st.provider = None
  try:
    yield
  finally:
    st.provider = prev


def push_module(module, path: tuple[str, ...]):
  _s().modules.append((module, path))


def pop_module():
  _s().modules.pop()


def next_count(module, key: str, repeated: bool = False) -> int:
  st = _s()
  k = (id(module), key)
  count = st.counters.get(k, 0)
  if repeated:
    return count - 1
  st.counters[k] = count + 1
  return count
