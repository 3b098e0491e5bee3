"""Kinds of cache need: which class of cache spec the manager serves how.

A mixer's ``cache_spec()`` returns an object; its class says what the manager keeps for it:

* ``"paged"`` - tensors that grow with the request, in pages with a block table.  The spec has
  ``page_tensors(page_size) -> {name: shape of one page}`` and ``window`` (None, or the number of
  last positions that are ever read); equal specs share a page pool and block tables.
* ``"state"`` - one tensor of fixed ``shape`` and ``dtype`` per request slot, zeroed when a request
  starts.

``register_cache_kind(SpecClass, "paged" | "state")`` adds a spec class of one's own (a latent per
token, keys and values of different widths, ...) without a change to the manager.  The reference has
one kind only, keys and values of equal shape for every layer (pico_vllm/blockmanager.py:39-42).
"""
from __future__ import annotations

from typing import Dict

from ..errors import PicoError
from ..parts.base import FixedState, PagedKV, PagedTensors

KINDS = ("paged", "state")
_KIND_OF: Dict[type, str] = {}


def register_cache_kind(spec_class: type, kind: str) -> type:
    if kind not in KINDS:
        raise PicoError(f"unknown kind of cache need {kind!r} (have {list(KINDS)})")
    if kind == "paged" and not (hasattr(spec_class, "page_tensors")):
        raise PicoError(f"{spec_class.__name__}: a paged cache spec needs page_tensors(page_size) and window")
    _KIND_OF[spec_class] = kind
    return spec_class


def kind_of(spec) -> str:
    for cls in type(spec).__mro__:
        if cls in _KIND_OF:
            return _KIND_OF[cls]
    raise PicoError(f"unknown kind of cache need {spec!r}: register its class with register_cache_kind")


register_cache_kind(PagedKV, "paged")
register_cache_kind(PagedTensors, "paged")
register_cache_kind(FixedState, "state")
