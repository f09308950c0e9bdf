"""Derived-tensor cache keyed on the identity and version of its source tensors.

Packed weight layouts are derived data: they are never saved in a state_dict and are
rebuilt whenever a caller mutates a source parameter in place (``_version``), replaces it
(``data_ptr``), or moves / casts the module (device, dtype).
"""
from __future__ import annotations

from typing import Callable, Dict, Sequence, Tuple

import torch


def _key(tensors: Sequence[torch.Tensor]) -> Tuple:
    return tuple((t.data_ptr(), t._version, t.dtype, t.device, tuple(t.shape)) for t in tensors)


class DerivedCache:
    def __init__(self) -> None:
        self._slots: Dict[str, Tuple[Tuple, object]] = {}

    def get(self, name: str, sources: Sequence[torch.Tensor], make: Callable[[], object]):
        key = _key(sources)
        hit = self._slots.get(name)
        if hit is not None and hit[0] == key:
            return hit[1]
        with torch.no_grad():
            value = make()
        self._slots[name] = (key, value)
        return value

    def clear(self) -> None:
        self._slots.clear()
