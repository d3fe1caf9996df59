"""Dispatch and layout registries — torchao/dtypes/utils.py:5-65."""
import functools
from collections import defaultdict
from typing import Callable, Dict

# tensor subclass -> {torch function or aten op -> implementation}
_ATEN_OP_OR_TORCH_FN_TABLE: Dict[Callable, Dict[Callable, Callable]] = defaultdict(dict)


def _implements(cls, aten_ops_or_torch_fns):
    """Decorator registering an implementation for aten ops (a list, used from __torch_dispatch__) or a
    torch function (a single object, used from __torch_function__) — torchao/dtypes/utils.py:14-29."""
    if not isinstance(aten_ops_or_torch_fns, (list, tuple)):
        aten_ops_or_torch_fns = [aten_ops_or_torch_fns]

    def decorator(func):
        for op in aten_ops_or_torch_fns:
            @functools.wraps(op)
            def wrapper(*args, **kwargs):
                return func(*args, **kwargs)

            _ATEN_OP_OR_TORCH_FN_TABLE[cls][op] = wrapper
        return func

    return decorator


# tensor subclass -> {extended layout name -> LayoutClass.from_plain}
_LAYOUT_CONSTRUCTOR_TABLE: Dict[Callable, Dict[str, Callable]] = defaultdict(dict)


def _register_layout_cls(cls: Callable, extended_layout: str):
    """torchao/dtypes/utils.py:40-55"""
    def decorator(layout_cls):
        layout_cls.extended_layout = extended_layout
        _LAYOUT_CONSTRUCTOR_TABLE[cls][extended_layout] = layout_cls.from_plain
        return layout_cls

    return decorator


def _get_layout_tensor_constructor(cls: Callable, extended_layout: str) -> Callable:
    """torchao/dtypes/utils.py:57-65"""
    if cls not in _LAYOUT_CONSTRUCTOR_TABLE:
        raise ValueError(f"no registered layout class constructor for: {cls}")
    if extended_layout not in _LAYOUT_CONSTRUCTOR_TABLE[cls]:
        raise ValueError(f"extended_layout: {extended_layout} is not supported yet for {cls}")
    return _LAYOUT_CONSTRUCTOR_TABLE[cls][extended_layout]
