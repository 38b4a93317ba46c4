"""What a part is, and the registries that map a part's kind to its class.

A model is put together from parts of five categories:

``mixer``
    mixes information between the tokens of a request (attention here).  It
    declares the cache it needs (:class:`PagedKVNeed`, :class:`StateNeed` or
    None) and computes ``forward(x, ctx, cache) -> [T, hidden]``.
``feed_forward``
    works on each token alone: ``forward(x, ctx) -> [T, hidden]``.
``norm``
    ``forward(pending, residual, rows=None) -> normalised``: adds the pending
    sublayer output to the 32-bit residual stream and normalises it.
``position``
    position encoding; the attention mixer hands it Q, K, V of the step.
``block``
    the arrangement of the parts above in one layer.

plus ``embedding`` and ``head`` at the two ends of the model.  A part gets its
sizes and constants from its :class:`~einf_b200.config.specs.PartSpec` and its
tensors by their local names; it never sees the model's configuration.

The reference has one class per role inside one file
(``src/einf/executors/torch/qwen.py:125-593``) and no registry.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, ClassVar, Mapping, Optional

import torch

from ..config.specs import PartSpec, TensorSpec

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {category: {} for category in CATEGORIES}


def register_part(category: str, kind: str) -> Callable[[type], type]:
    """Class decorator: make ``kind`` available to specs of ``category``."""
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; known: {CATEGORIES}")

    def decorate(cls: type) -> type:
        known = _REGISTRY[category].get(kind)
        if known is not None and known is not cls:
            raise ValueError(f"{category} kind {kind!r} is already registered to {known.__name__}")
        _REGISTRY[category][kind] = cls
        cls.kind = kind
        return cls

    return decorate


def part_class(category: str, kind: str) -> type:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {}))) or "(none)"
        raise ValueError(f"unknown {category} kind {kind!r}; known: {known}") from None


def known_parts(category: str) -> tuple[str, ...]:
    return tuple(sorted(_REGISTRY[category]))


# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class Runtime:
    """Where and in which precision a model computes."""

    dtype: torch.dtype            # activation dtype: torch.bfloat16 or torch.float32
    device: torch.device

    def matrix(self, tensor: torch.Tensor) -> torch.Tensor:
        """A matrix operand: 32-bit in the 32-bit path, else as the checkpoint keeps it
        (bfloat16, or 32-bit for a tensor stored in 32-bit)."""
        if self.dtype == torch.float32:
            tensor = tensor.to(torch.float32)
        return tensor.to(self.device).contiguous()

    def vector(self, tensor: torch.Tensor) -> torch.Tensor:
        """Norm weights and biases: always 32-bit (they enter 32-bit arithmetic)."""
        return tensor.to(device=self.device, dtype=torch.float32).contiguous()


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every token (or of the last ``window`` tokens), in pages."""

    num_kv_heads: int
    head_size: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A tensor of fixed shape per request, zeroed when the request starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheView:
    """What one run of a layer sees of the cache.

    ``k`` and ``v`` are ``[pages, kv_heads, page_size, head_size]`` for a paged
    need; ``state`` is ``[slots, *shape]`` for a state need.  ``writes`` is false
    for a run that reads another run's cache.
    """

    group: int = -1
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    writes: bool = True
    page_size: int = 0


@dataclass
class StepContext:
    """Device-side description of one step, shared by all parts.

    ``T`` tokens of ``R`` requests are packed in batch order.  All index
    tensors are int32 on the model's device.
    """

    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor          # [T]
    positions: torch.Tensor          # [T] absolute position of each token
    seq_of_token: torch.Tensor       # [T] index of the token's request in the batch
    q_start: torch.Tensor            # [R + 1] prefix sums of the portions' lengths
    context_lens: torch.Tensor       # [R] tokens of the request after this step
    block_tables: list[torch.Tensor]  # per cache group: [R, width] logical -> physical page, -1 = none
    slots: list[torch.Tensor]        # per cache group: [T] physical slot of each token
    state_slots: torch.Tensor        # [R] state slot of each request, -1 = none
    logit_rows: torch.Tensor         # [S] tokens whose logits are wanted
    q_tiles: torch.Tensor            # [tiles, 4] 128-row query tiles of requests with more than one token: request, first token, rows, first position
    single_tokens: torch.Tensor      # [n] packed indices of the tokens of requests that bring exactly one (decoding)
    status: torch.Tensor             # [1] int32, kernels set bits instead of faulting
    # host copies, so that no part reads device memory to size a launch
    q_lens: tuple[int, ...] = ()
    start_positions: tuple[int, ...] = ()
    max_q_len: int = 0
    max_context_len: int = 0
    max_portion_start: int = 0       # most cached tokens before a portion of more than one token
    decode_only: bool = False
    extras: dict[str, Any] = field(default_factory=dict)


class Part:
    """Base of all parts."""

    kind: ClassVar[str] = ""
    #: false for a part whose forward reads device memory on the host (it cannot be
    #: captured in a CUDA graph; the engine then runs every step eagerly)
    graph_safe: ClassVar[bool] = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> Mapping[str, TensorSpec]:
        """Local tensor names (appended to ``spec.prefix``) with shape and role."""
        return {}

    @classmethod
    def kernel_libraries(cls, spec: PartSpec, runtime: Runtime) -> tuple[str, ...]:
        """Names of the kernel libraries this part launches, so that they can be
        compiled side by side before the first step."""
        return ()

    @classmethod
    def nested_parts(cls, spec: PartSpec) -> Mapping[str, str]:
        """Parameters of ``spec`` that are parts themselves (a :class:`PartSpec`, or a tuple of
        them): parameter name -> category.  A part of any category may nest parts; their tensors
        are expected, loaded and handed on like the part's own, and the part builds them with
        :func:`build_nested`.  By default a nested spec's category is its parameter's name
        (``"position"``, ``"norm"`` ...); a part that names its parameters otherwise overrides this."""
        found = {}
        for key, value in spec.params.items():
            values = value if isinstance(value, (tuple, list)) else (value,)
            if values and all(isinstance(v, PartSpec) for v in values):
                if key not in CATEGORIES:
                    raise ValueError(
                        f"{cls.__name__} nests a part under {key!r}, which is no category ({CATEGORIES}); "
                        f"let nested_parts() name its category"
                    )
                found[key] = key
        return found

    def launch_key(self, ctx: "StepContext", page_size: int) -> tuple:
        """What this part's launches take from the step's host-side figures (the longest context,
        say) beyond the shapes of the step's tensors, as a hashable value: steps whose keys differ
        are captured as different CUDA graphs, so a graph never pins a choice made for other
        figures.  ``()``: the launches depend on the shapes alone."""
        return ()

    def launch_group(self):
        """Parts with equal groups give equal launch keys; the runner asks one of each group."""
        return id(self)

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.spec = spec
        self.runtime = runtime


class Mixer(Part):
    """``forward`` returns ``[T, hidden]`` in the activation type, or float32 partial sums
    ``[splits, T, hidden]`` that the next norm adds up (what a split-K product leaves)."""

    def cache_need(self) -> PagedKVNeed | StateNeed | None:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(
        self,
        pending: Optional[torch.Tensor],
        residual: torch.Tensor,
        rows: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        raise NotImplementedError


class PartTensors(dict):
    """A part's own tensors by their local names; ``everything`` is the mapping of all checkpoint
    tensors they were taken from, which a part hands on to the parts it nests."""

    def __init__(self, local: Mapping[str, torch.Tensor], everything: Mapping[str, torch.Tensor]) -> None:
        super().__init__(local)
        self.everything = everything


def build_part(category: str, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> Part:
    """Build the part ``spec`` names from the checkpoint tensors under its prefix."""
    cls = part_class(category, spec.kind)
    local = {}
    for name in cls.tensor_specs(spec):
        full = spec.prefix + name
        if full not in tensors:
            raise KeyError(f"{category} {spec.kind!r} needs tensor {full!r}")
        local[name] = tensors[full]
    return cls(spec, PartTensors(local, tensors), runtime)


def build_nested(category: str, spec: PartSpec, parent_tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> Part:
    """Build a part that another part nests, from the mapping the parent's tensors came from."""
    return build_part(category, spec, getattr(parent_tensors, "everything", {}), runtime)


def walk_part_specs(category: str, spec: PartSpec):
    """``(category, spec)`` of a part and of every part nested in it, at any depth."""
    yield category, spec
    for key, nested_category in part_class(category, spec.kind).nested_parts(spec).items():
        value = spec.params[key]
        for nested in (value if isinstance(value, (tuple, list)) else (value,)):
            yield from walk_part_specs(nested_category, nested)
