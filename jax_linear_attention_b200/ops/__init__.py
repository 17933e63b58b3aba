"""Linear-attention ops with the call surface of ``jla.ops`` and one implementation: ``"cuda"``.

    o, final_state = linear_attention("gated_deltanet", q, k, v, g=g, beta=beta)

Mirrors ``src/jla/ops/__init__.py`` of the reference: ``KINDS`` (:47-60), ``register`` (:68-90),
``available`` (:113-116) and ``linear_attention`` (:128-173) keep their names, arguments, return values
and error behaviour. The kinds are the ones this hot path covers:

* ``simple_gla`` (``g``): one log-decay per head; Mamba-2's SSD core with ``q=C, k=B, v=dt*x, g=dt*A, scale=1``;
* ``deltanet`` (``beta``); ``gated_deltanet`` (``g, beta``); ``kda`` (``g [B, T, H, K], beta``).

``impl`` is ``"auto"`` or ``"cuda"``: the hand-written sm_100a kernels of ``libjla_b200.so``. There is no
Pallas, Triton, plain-XLA or CPU implementation behind this dispatcher; a call the kernels cannot run raises.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

from . import cuda

__all__ = ["KINDS", "available", "linear_attention", "register", "cuda"]

# kind -> (function name, gate inputs in positional order)
KINDS: dict[str, tuple[str, tuple[str, ...]]] = {
    "simple_gla": ("simple_gla", ("g",)),
    "deltanet": ("delta_rule", ("beta",)),
    "gated_deltanet": ("gated_delta_rule", ("g", "beta")),
    "kda": ("kda", ("g", "beta")),
    "gdn2": ("gdn2", ("g", "b", "w")),
}
_GATE_NAMES = frozenset(name for _, gates in KINDS.values() for name in gates)

_ORDER = ("cuda",)
_Supports = Callable[..., bool]
_REGISTRY: dict[str, dict[str, tuple[Callable[..., Any], _Supports, bool]]] = {name: {} for name in _ORDER}


def register(impl: str, kind: str, fn: Callable[..., Any], supports: _Supports | None = None, *,
             auto: bool = False) -> None:
    """Register ``fn`` as implementation ``impl`` of ``kind`` (same contract as the reference's ``register``).

    ``fn`` takes ``(q, k, v, *gates, **options)`` with the gates in ``KINDS[kind]`` order;
    ``supports(q, k, v, *gates, **options)`` returns False for calls it cannot handle.
    """
    if kind not in KINDS:
        raise ValueError(f"unknown linear-attention kind {kind!r}")
    _REGISTRY.setdefault(impl, {})[kind] = (fn, supports or (lambda *args, **options: True), auto)


def available(kind: str) -> tuple[str, ...]:
    """Registered implementations of ``kind``, fastest first."""
    order = _ORDER + tuple(name for name in _REGISTRY if name not in _ORDER)
    return tuple(impl for impl in order if kind in _REGISTRY.get(impl, {}))


for _kind in KINDS:
    register("cuda", _kind, cuda.FUNCTIONS[_kind], cuda.SUPPORTS[_kind], auto=True)


def linear_attention(kind: str, q, k, v, *, impl: str = "auto", **inputs: Any):
    """Run a linear-attention op; returns ``(o, final_state)``.

    ``inputs`` holds the kind's gates by name (``g``, ``beta``; ``g``, ``b``, ``w`` for ``gdn2``) plus the options passed through: ``scale``,
    ``initial_state``, ``output_final_state``, ``segment_ids``, ``cu_seqlens``, ``use_qk_l2norm`` (delta-rule
    kinds), ``chunk_size`` (must be 64), ``sub_chunk`` (KDA; accepted, unused) and ``precision``
    (``"highest"`` = the fp32 token-scan kernels).
    """
    if kind not in KINDS:
        raise ValueError(f"unknown linear-attention kind {kind!r}; expected one of {sorted(KINDS)}")
    _, gate_names = KINDS[kind]
    missing = [name for name in gate_names if inputs.get(name) is None]
    extra = sorted(name for name in _GATE_NAMES - set(gate_names) if inputs.get(name) is not None)
    if missing or extra:
        raise ValueError(f"{kind} takes gates {gate_names}; missing {missing}, unexpected {extra}")
    gates = [inputs.pop(name) for name in gate_names]
    options = {key: value for key, value in inputs.items() if key not in _GATE_NAMES}
    candidates = _ORDER if impl == "auto" else (impl,)
    for name in candidates:
        entry = _REGISTRY.get(name, {}).get(kind)
        if entry is None:
            continue
        fn, supports, auto_eligible = entry
        if impl == "auto" and not (auto_eligible and supports(q, k, v, *gates, **options)):
            continue
        return fn(q, k, v, *gates, **options)
    if impl == "auto":  # surface the kernels' reason instead of a bare "nothing accepts this call"
        why = cuda.unsupported_reason(kind, q, k, v, tuple(gates), options)
        raise ValueError(f"no implementation of {kind!r} accepts this call (have {available(kind)}): {why}")
    raise ValueError(f"no {impl!r} implementation of {kind!r} accepts this call (have {available(kind)})")
