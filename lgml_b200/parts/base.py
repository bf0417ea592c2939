"""What a part of a layer is, and the registry of parts by name.

A model is put together from parts: a *norm*, a *mixer* (attention here), a
*feed-forward*, a *position encoding* the mixer uses, and a *block* that says in
which arrangement a layer runs them.  Each part gets its sizes and constants as
constructor arguments, says which tensors it needs, and is looked up by name in
this registry, so a model's builder can choose parts layer by layer from its
configuration and a new kind of part is one ``register_part`` call away.  No
part knows which model it is in.  mischief/lgml keeps its parts the same way,
as plain functions of (graph, sizes, layer): ``M.qkv``, ``M.attend``,
``M.attn_out``, ``M.ffn``, ``M.head`` (``lua/lgml/transformer.lua:1738-1754``,
``:1791-1803``, ``:1849-1859``, ``:2029-2042``, ``:2082-2094``).

Interfaces (tensors are torch tensors on the device; ``rt`` is the ``Runtime``):

* every part:   ``tensor_specs(prefix) -> [TensorSpec]``, ``bind(prefix, tensors, rt)``
* norm:         ``forward(rt, x_f32, out_dtype, delta=None, rows=None) -> h``
                (with ``delta``: x += delta first, the sum stays in x)
* position:     ``apply(rt, qkv, batch, cache, n_heads, n_kv_heads, head_dim) -> q``: it owns what
                happens to q and k between the projection and the cache write, writes this
                step's k and v into ``cache`` and returns q for attention.  A rotation
                (``RotaryPosition``) only gives ``n_rot``, ``pairing``, ``inv_freq`` (device
                float32); any other part calls ``store_kv`` when its own work is done
* mixer:        ``cache_spec() -> PagedKV | FixedState | None``,
                ``forward(rt, h, batch, cache) -> delta``  (h, delta: [tokens, width])
* feed-forward: ``forward(rt, h) -> delta``; optionally ``first_weights() -> [tensor]``
* block:        ``forward(rt, x, pending, batch, cache) -> (x, pending)`` where
                ``pending`` is a delta not yet added to the residual stream x
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List

from ..weights import TensorSpec

KINDS = ("norm", "position", "mixer", "feed_forward", "block")
_PARTS: Dict[str, Dict[str, Callable[..., Any]]] = {k: {} for k in KINDS}


def register_part(kind: str, name: str, factory: Callable[..., Any]) -> None:
    if kind not in _PARTS:
        raise KeyError(f"unknown kind of part '{kind}' (kinds: {', '.join(KINDS)})")
    _PARTS[kind][name] = factory


def make_part(kind: str, name: str, **args) -> Any:
    try:
        factory = _PARTS[kind][name]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(kind, {}))) or "none"
        raise KeyError(f"no {kind} named '{name}' is registered (known: {known})") from None
    return factory(**args)


def registered(kind: str) -> List[str]:
    return sorted(_PARTS[kind])


class Part:
    """Base of all parts: by default no tensors.

    ``graph_safe`` says that ``forward`` only launches work whose shape and addresses are
    fixed by the batch's shape (everything else it reads on the device), so a decode step
    through it can be captured into a CUDA graph and replayed.  A part that loops over
    requests on the host, or reads host values of the batch, leaves it False and the runner
    then runs every step eagerly."""

    graph_safe = False

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return []

    def bind(self, prefix: str, tensors: Dict[str, Any], rt) -> None:
        pass

    def first_weights(self) -> List[Any]:
        """The bound tensors this part reads first, in that order (a block may ask L2 for their
        head while the part before it runs); none by default."""
        return []
