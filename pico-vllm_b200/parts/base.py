"""What every part of a layer has in common.

A *part* is one piece of a layer: a mixer (attention here), a feed-forward, a norm, a position
encoding, the token embedding, the output head.  A part takes all of its sizes and constants as
constructor arguments, declares the tensors it owns (:class:`Param`) and what cache it needs
(:class:`PagedKV`, :class:`FixedState` or nothing), and never learns which model it is in: the
model builder maps the part's local tensor keys to the tensor names of a model folder.

Interfaces (duck-typed; subclassing :class:`Part` is enough):

* Mixer: ``cache_spec()``, ``forward(h, batch, cache) -> delta`` with h [T, width] in the
  activation dtype, ``batch`` a :class:`~pico_vllm_b200.engine.batch.Batch`, ``cache`` a
  :class:`CacheView` of this call's cache entry; optionally ``plan(shape)`` (scratch and launch
  policy of its own kernels).
* Feed-forward: ``forward(h, batch) -> delta``.
* Norm: ``add_norm(x, delta, rows=None) -> y`` on the float32 residual stream.
* Position encoding: owned by the mixer that uses it; see ``parts/rotary.py``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class Piece:
    """One tensor of the model folder that goes into a parameter."""
    key: str                 # the part's own name for it, e.g. "q.weight"
    shape: Tuple[int, ...]


@dataclass(frozen=True)
class Param:
    """A tensor a part owns: its pieces are concatenated along dimension 0 at load time
    (as the reference fuses q/k/v and gate/up, pico_vllm/weights.py:42-43,58)."""
    attr: str
    pieces: Tuple[Piece, ...]
    kind: str = "matrix"     # "matrix": model dtype unless stored in 32-bit; "vector": float32
    init: str = "normal"     # random-weights rule: "normal" N(0, std) or "one_plus_normal"

    @property
    def shape(self) -> Tuple[int, ...]:
        first = self.pieces[0].shape
        return (sum(p.shape[0] for p in self.pieces),) + tuple(first[1:])


@dataclass(frozen=True)
class PagedKV:
    """The mixer keeps keys and values per token in pages.  ``window``: None = all keys stay
    needed; W = only the last W keys are ever read, older pages may be given back."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def page_tensors(self, page_size: int) -> Dict[str, Tuple[int, ...]]:
        shape = (self.n_kv_heads, page_size, self.head_dim)
        return {"k": shape, "v": shape}


@dataclass(frozen=True)
class PagedTensors:
    """The general paged need: any tensors per page, by name.  ``per_token`` maps a name to the
    shape one token adds (e.g. ``{"latent": (96,)}`` for one compressed vector per token, or
    ``{"k": (2, 64), "v": (2, 128)}`` for keys and values of different widths); a page of the tensor is
    [page_size, *shape].  ``window`` as in :class:`PagedKV`."""
    per_token: Tuple[Tuple[str, Tuple[int, ...]], ...]
    window: Optional[int] = None

    def page_tensors(self, page_size: int) -> Dict[str, Tuple[int, ...]]:
        return {name: (page_size,) + tuple(shape) for name, shape in self.per_token}


@dataclass(frozen=True)
class FixedState:
    """The mixer keeps one tensor of fixed shape per request (zeroed when a request starts)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass
class CacheView:
    """What a mixer call gets of the cache: the tensors of its own cache entry.

    For a paged need: ``tensors`` maps each name of the spec's ``page_tensors`` to
    [num_pages, *page shape] (``k`` and ``v`` are those two when the spec has them: [num_pages,
    n_kv_heads, page_size, head_dim] for :class:`PagedKV`), ``group`` selects
    ``batch.groups[group]`` (slots and block table), ``store`` is False when this call only reads
    an entry that another call fills.  For FixedState: ``state`` is [max_num_seqs, *shape];
    ``batch.seg_slots`` gives each segment's row."""
    group: Optional[int] = None
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    page_size: int = 0
    store: bool = True
    state: Optional[torch.Tensor] = None
    k_map: object = None       # TMA tensor maps over k and v (ops.make_kv_tensor_map), or None
    v_map: object = None
    k_map2d: object = None     # the same pages in [page_size, 64]-boxes (ops.make_kv_tensor_map_2d), or None
    v_map2d: object = None
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)


@dataclass
class StepShape:
    """What a mixer may know of a step before it runs, to plan its kernels (:meth:`Part.plan`)."""
    num_tokens: int                  # tokens of the batch, padding rows of a replayed shape included
    num_segments: int
    q_lens: List[int]                # tokens of each real segment
    starts: List[int]                # tokens each real segment's request already holds
    max_kv: int                      # longest request after this step
    decode_only: bool
    num_sms: int                     # multiprocessors of the device (1 off the GPU)
    engine: object = None            # the EngineConfig (dtype, knobs a mixer may read by name)


@dataclass(frozen=True)
class MixerPlan:
    """A mixer's launch plan for one step; mixers subclass it to add fields of their own.  ``key``
    tells plans apart that need different launches (a recorded step is replayed only for an equal
    key); ``scratch_floats`` is the float32 scratch the mixer's kernels need in this step (the step
    function owns one buffer that every mixer call of the step may use, as calls run one after the
    other)."""
    key: Tuple = ()
    scratch_floats: int = 0


class Part:
    """Base of all parts: declares parameters, receives them from the loader."""

    def params(self) -> List[Param]:
        return []

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        setattr(self, attr, tensor)

    def materialize(self, device: torch.device, dtype: torch.dtype) -> None:
        """Creates device-side constants that are not weights (tables of frequencies …)."""

    def cache_spec(self):
        return None

    def plan(self, shape: "StepShape") -> Optional["MixerPlan"]:
        """A mixer whose kernels need scratch memory or a launch policy that depends on the step
        (splits, tile sharing) returns a :class:`MixerPlan`; the step function calls this once per
        step and per ``plan_key()``, provides the scratch and hands the plan back through
        ``batch.plan(self)``.  None: nothing to plan."""
        return None

    def plan_key(self):
        """Mixers with equal keys get one plan per step (layers of equal sizes share theirs)."""
        return id(self)
