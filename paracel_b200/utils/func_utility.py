"""Callable introspection (reference: include/utils/func_utility.hpp:24-81, which
derives msgpack argument types of a handler at compile time).  In Python the
equivalent information is the signature: arity and annotated types."""
from __future__ import annotations

import inspect
from typing import Any, Callable, Tuple


class f_traits:
    def __init__(self, f: Callable):
        self.f = f
        try:
            sig = inspect.signature(f)
        except (TypeError, ValueError):
            sig = None
        self.signature = sig
        params = [] if sig is None else [
            p for p in sig.parameters.values()
            if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
        self.arity = len(params)
        self.args: Tuple[Any, ...] = tuple(
            (p.annotation if p.annotation is not inspect.Parameter.empty else Any) for p in params)
        self.result_type = Any if sig is None or sig.return_annotation is inspect.Signature.empty \
            else sig.return_annotation
