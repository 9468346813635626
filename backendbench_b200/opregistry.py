"""Canonical operator objects <-> spec names ("add.Tensor", "relu").

Same role as BackendBench/opregistry.py:14-110: operators cross process boundaries as
spec-name strings (OpOverload objects do not pickle) and are resolved back to the one
canonical object per name on the other side.
"""

from __future__ import annotations

import logging

import torch

logger = logging.getLogger(__name__)


def _extract_spec_name_from_op(op_obj):
    """"aten::add.Tensor" -> "add.Tensor"; None for objects without a qualified `_name`."""
    name = getattr(op_obj, "_name", None)
    if isinstance(name, str) and "::" in name:
        return name.split("::", 1)[1]
    return None


class OpRegistry:
    def __init__(self):
        self._registry = {}

    def get_operator(self, input_obj):
        if isinstance(input_obj, str):
            return self._from_spec_name(input_obj)
        return self._from_object(input_obj)

    def _from_spec_name(self, spec_name):
        hit = self._registry.get(spec_name)
        if hit is not None:
            return hit
        base, _, overload = spec_name.partition(".")
        try:
            op = getattr(getattr(torch.ops.aten, base), overload or "default")
        except AttributeError as e:
            logger.warning(f"Failed to resolve operator {spec_name}: {e}")
            return None
        self._registry[spec_name] = op
        return op

    def _from_object(self, op_obj):
        spec_name = _extract_spec_name_from_op(op_obj)
        return self._registry.setdefault(spec_name, op_obj)

    def register_operator(self, op_obj):
        return self._from_object(op_obj)

    def get_all_registered_ops(self):
        return dict(self._registry)

    def clear(self):
        self._registry.clear()

    def __len__(self):
        return len(self._registry)

    def __contains__(self, spec_name):
        return spec_name in self._registry

    def __repr__(self):
        return f"OpRegistry({len(self._registry)} ops)"


_op_registry = OpRegistry()


def get_operator(input_obj):
    return _op_registry.get_operator(input_obj)


def register_operator(op_obj):
    return _op_registry.register_operator(op_obj)


def get_registry():
    return _op_registry
