"""Mirror of sharktank's overridable-op registry for the ops on the MoE path.

Semantics follow sharktank/ops/_registry.py:174-307: an op is a dispatcher;
implementations register with `@op.override(*type_spec, salience=...)`;
candidates are tried from the highest salience down, the latest registration
first among equals, and an implementation declines by returning
`NotImplemented`.  When no candidate accepts, NotImplementedError is raised.
The signatures are those of sharktank/ops/signatures.py (einsum_2args :178-206,
get_index :317-340).

On a machine that has sharktank, `shark_platform_b200.plugin.register()` puts
the same implementations into sharktank's own registry instead.
"""
from __future__ import annotations

import functools
from typing import Any, Callable

import torch

_last_dispatch = None
_track_dispatch = False


def _test_enable_last_op_dispatch(en: bool = True):
    global _track_dispatch, _last_dispatch
    _track_dispatch, _last_dispatch = en, None


def _test_get_last_op_dispatch():
    assert _track_dispatch
    return _last_dispatch


class SignatureDispatcher:
    def __init__(self, sig: Callable, tensor_args: tuple[int, ...]):
        functools.update_wrapper(self, sig)
        self._tensor_args = tensor_args
        self._overrides: list[tuple[int, int, tuple, Callable]] = []
        self._cache: dict[tuple, list[Callable]] = {}
        self._seq = 0

    def override(self, *type_spec, salience: int = 0):
        def deco(f):
            self._seq += 1
            self._overrides.append((salience, self._seq, type_spec, f))
            self._overrides.sort(key=lambda o: (o[0], o[1]))
            self._cache.clear()
            return f

        return deco

    def find_overrides(self, tensors: tuple[Any, ...]):
        key = tuple(type(t) for t in tensors)
        found = self._cache.get(key)
        if found is None:
            found = []
            for _, _, spec, f in self._overrides:
                if len(spec) != len(key):
                    continue
                if all(s is None or issubclass(a, s) for s, a in zip(spec, key)):
                    found.append(f)
            self._cache[key] = found
        return reversed(found)

    def fail(self, tensors):
        raise NotImplementedError(
            f"Overridable operator {self.__name__} does not have an implementation "
            f"for argument types: {[type(t) for t in tensors]}"
        )

    def __call__(self, *args, **kwargs):
        global _last_dispatch
        tensors = tuple(args[i] for i in self._tensor_args)
        for impl in self.find_overrides(tensors):
            result = impl(*args, **kwargs)
            if result is not NotImplemented:
                if _track_dispatch:
                    _last_dispatch = impl
                return result
        self.fail(tensors)


def overridable(*tensor_args: int):
    return lambda sig: SignatureDispatcher(sig, tensor_args)


@overridable(0, 1)
def einsum_2args(input0, input1, einsum_str: str):
    """Executes a given Einstein summation notation string on the provided
    tensors (sharktank/ops/signatures.py:178-206)."""


@overridable(0)
def get_index(tensor, key):
    """Indexes the tensor using the key: `tensor[key]`
    (sharktank/ops/signatures.py:317-340)."""


@overridable(1)
def elementwise(operator, *args, **kwargs):
    """Applies an elementwise operator (sharktank/ops/signatures.py:209-228)."""


@elementwise.override(torch.Tensor)
def _elementwise_tensor(operator, x, *args, **kwargs):
    # ops/default_impls.py:125-128
    return operator(x, *args, **kwargs)


@overridable(0, 1)
def matmul(lhs, rhs, *, transpose_rhs: bool = False):
    """Performs a matmul where the RHS may be an InferenceTensor
    (sharktank/ops/signatures.py:659-688)."""


@overridable(0, 1)
def linear(input, weight, bias=None, *, accum_dtype=None):
    """Applies a linear transformation `input @ weight.T + bias`
    (sharktank/ops/signatures.py:615-656).  The reference dispatches on
    (input, weight[, bias]); the mirror dispatches on (input, weight)."""
