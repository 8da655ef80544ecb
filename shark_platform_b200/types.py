"""Host-side mirror of the sharktank tensor types that cross the MoE boundary.

Same class names, constructor arguments and accessors as the reference
(sharktank/types/tensors.py and sharktank/types/layouts.py) so that code
written against sharktank's `PlanarQuantizedTensor` / `Theta` runs unchanged on
a machine without sharktank.  The kernels accept either these classes or the
reference's own: everything downstream is duck-typed on `.layout_type.__name__`,
`.unpack().planes` and `.shape`.

Only containers live here; arithmetic (`dequant`) calls the CUDA library.
"""
from __future__ import annotations

from typing import Any, Optional, Sequence, Union

import torch

__all__ = [
    "BlockScaledLayout",
    "SuperBlockOffsetScaled_4_6_Layout",
    "QuantizedLayout",
    "InferenceTensor",
    "PrimitiveTensor",
    "DefaultPrimitiveTensor",
    "QuantizedTensor",
    "PlanarQuantizedTensor",
    "ShardedTensor",
    "ReplicatedTensor",
    "SplitPrimitiveTensor",
    "Theta",
    "unbox_tensor",
]


class QuantizedLayout:
    """types/layouts.py `QuantizedLayout`: planes + logical shape."""

    @property
    def planes(self) -> dict[str, torch.Tensor]:
        raise NotImplementedError

    @property
    def shape(self) -> list[int]:
        raise NotImplementedError

    def dequant(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        from . import moe

        return moe.dequant_layout(self, dtype)


class BlockScaledLayout(QuantizedLayout):
    """types/layouts.py:194-299.  `d` [..., K/32, 1] and `qs` [..., K/32, 32];
    `dequant(dtype)` is `d.to(dtype) * qs.to(dtype)`.  Offsets (`m`) are not
    supported by the CUDA path."""

    def __init__(self, shape, d, qs, *, m=None):
        if m is not None:
            raise NotImplementedError("BlockScaledLayout with offsets (m) is not supported")
        self._shape, self._d, self._qs, self._m = list(shape), d, qs, None

    @classmethod
    def serialized_name(cls) -> str:
        return "BlockScaledLayout"

    @property
    def planes(self):
        return {"d": self._d, "qs": self._qs}

    @property
    def shape(self):
        return self._shape

    @property
    def d(self):
        return self._d

    @property
    def m(self):
        return None

    @property
    def qs(self):
        return self._qs


class SuperBlockOffsetScaled_4_6_Layout(QuantizedLayout):
    """types/layouts.py:360-530: the planar form of ggml Q4_K."""

    _NAMES = ("d", "dmin", "sb_scales_high", "sb_scales_low", "sb_mins_high", "sb_mins_low", "qs")

    def __init__(self, shape, *, d, dmin, sb_scales_high, sb_scales_low, sb_mins_high,
                 sb_mins_low, qs):
        self._shape = list(shape)
        self._planes = {
            "d": d, "dmin": dmin,
            "sb_scales_high": sb_scales_high, "sb_scales_low": sb_scales_low,
            "sb_mins_high": sb_mins_high, "sb_mins_low": sb_mins_low,
            "qs": qs,
        }

    @classmethod
    def serialized_name(cls) -> str:
        return "SuperBlockOffsetScaled_4_6_Layout"

    @property
    def planes(self):
        return dict(self._planes)

    @property
    def shape(self):
        return self._shape

    @property
    def d(self):
        return self._planes["d"]

    @property
    def dmin(self):
        return self._planes["dmin"]

    @property
    def qs_bit_packed(self):
        return self._planes["qs"]


class BlockScaledI4Layout(QuantizedLayout):
    """types/layouts.py:303-347: a BlockScaledLayout whose `qs` are packed two
    4-bit values per byte (low nibble first), blocks of 32 with fp16 scale `d`
    and optional fp16 offset `m` (GGUF Q4_1).  Planes: `d`, `m` [..., K/32, 1],
    `qs` [..., K/32, 16] uint8.  Only the unsigned form is supported by the CUDA
    path."""

    def __init__(self, shape, d, qs, *, m=None, signed: bool = False):
        self._shape, self._d, self._qs, self._m, self.signed = list(shape), d, qs, m, signed

    @classmethod
    def serialized_name(cls) -> str:
        return "BlockScaledI4Layout"

    @property
    def planes(self):
        p = {"d": self._d, "qs": self._qs}
        if self._m is not None:
            p["m"] = self._m
        return p

    @property
    def shape(self):
        return self._shape

    @property
    def d(self):
        return self._d

    @property
    def m(self):
        return self._m

    @property
    def qs_bit_packed(self):
        return self._qs


class InferenceTensor:
    """types/tensors.py:189-454 (name, shape, indexing through ops.get_index)."""

    def __init__(self, *, shape, name: str = "<unnamed>"):
        self.name = name
        self.shape = list(shape)

    def __getitem__(self, key):
        from . import ops

        return ops.get_index(self, key)


class PrimitiveTensor(InferenceTensor):
    def as_torch(self, *, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        raise NotImplementedError


class DefaultPrimitiveTensor(PrimitiveTensor):
    """types/tensors.py:507-577."""

    def __init__(self, *, data: torch.Tensor, name: str = "<unnamed>"):
        super().__init__(shape=list(data.shape), name=name)
        self._data = data

    def as_torch(self, *, dtype=None):
        return self._data if dtype is None else self._data.to(dtype)

    @property
    def dtype(self):
        return self._data.dtype

    def to(self, *args, **kwargs):
        return DefaultPrimitiveTensor(data=self._data.to(*args, **kwargs), name=self.name)


class QuantizedTensor(InferenceTensor):
    """types/tensors.py:585-619."""

    def __init__(self, *, shape, layout_type, name: str = "<unnamed>"):
        super().__init__(shape=shape, name=name)
        self.layout_type = layout_type

    def unpack(self) -> QuantizedLayout:
        raise NotImplementedError


class PlanarQuantizedTensor(QuantizedTensor):
    """types/tensors.py:622-735: a quantized tensor whose layout is already
    split into planes."""

    def __init__(self, *, shape, layout: QuantizedLayout, name: str = "<unnamed>"):
        super().__init__(shape=shape, layout_type=type(layout), name=name)
        self.layout = layout

    def unpack(self):
        return self.layout

    def to(self, *args, **kwargs):
        lay = self.layout
        planes = {k: v.to(*args, **kwargs) for k, v in lay.planes.items()}
        if isinstance(lay, BlockScaledLayout):
            new = BlockScaledLayout(lay.shape, planes["d"], planes["qs"])
        else:
            new = type(lay)(lay.shape, **planes)
        return PlanarQuantizedTensor(shape=self.shape, layout=new, name=self.name)


class ShardedTensor(InferenceTensor):
    """types/tensors.py:743-955: a list of per-device shards held by one process."""

    def __init__(self, *, ts: Sequence[Any], shape, shard_dim: Optional[int], name="<unnamed>"):
        super().__init__(shape=shape, name=name)
        self._shards = tuple(ts)
        self.shard_dim = shard_dim

    @property
    def shards(self):
        return self._shards

    @property
    def shard_count(self) -> int:
        return len(self._shards)


class SplitPrimitiveTensor(ShardedTensor):
    """types/tensors.py:957-1096: shards split along `shard_dim`.  Shards may be
    quantized tensors (an expert-sharded `ffn_*_exps.weight`)."""

    def __init__(self, *, ts: Sequence[Any], shard_dim: int, shape=None, name="<unnamed>"):
        if shape is None:
            shape = list(ts[0].shape)
            shape[shard_dim] = sum(int(t.shape[shard_dim]) for t in ts)
        super().__init__(ts=ts, shape=shape, shard_dim=shard_dim, name=name)


class ReplicatedTensor(ShardedTensor):
    """types/tensors.py:1099-1238: the same tensor on every device."""

    def __init__(self, *, ts, shard_count: Optional[int] = None, name="<unnamed>"):
        if isinstance(ts, torch.Tensor) or not isinstance(ts, (list, tuple)):
            assert shard_count is not None
            ts = [ts] * shard_count
        super().__init__(ts=ts, shape=list(ts[0].shape), shard_dim=None, name=name)


def unbox_tensor(t: Union[torch.Tensor, InferenceTensor]) -> torch.Tensor:
    """types/tensors.py:1276-1284 for primitive tensors.  Quantized tensors are
    not silently dequantised here: the kernels consume them in place."""
    if isinstance(t, torch.Tensor):
        return t
    if hasattr(t, "as_torch"):
        return t.as_torch()
    raise TypeError(f"cannot unbox {type(t).__name__}")


def _nest(flat: dict) -> dict:
    """Splits dotted keys into nested dicts and merges them with dicts already
    present ({"a.b": 0, "a": {"c": 1}} -> {"a": {"b": 0, "c": 1}}), as
    types/theta.py:227-270 does.  A tree without dotted keys comes back as is."""
    if not any(isinstance(k, str) and "." in k for k in flat) and not any(
        isinstance(v, dict) for v in flat.values()
    ):
        return flat
    nested: dict = {}

    def add(dst: dict, key, value):
        parts = str(key).split(".")
        for part in parts[:-1]:
            nxt = dst.setdefault(part, {})
            if not isinstance(nxt, dict):
                raise ValueError(f"Name conflict at '{part}' while nesting '{key}'")
            dst = nxt
        leaf = parts[-1]
        if isinstance(value, dict):
            sub = dst.setdefault(leaf, {})
            if not isinstance(sub, dict):
                raise ValueError(f"Name conflict at '{leaf}' while nesting '{key}'")
            for k2, v2 in value.items():
                add(sub, k2, v2)
        else:
            if isinstance(dst.get(leaf), dict):
                raise ValueError(f"Name conflict at '{leaf}' while nesting '{key}'")
            dst[leaf] = value

    for k, v in flat.items():
        add(nested, k, v)
    return nested


class Theta:
    """types/theta.py:71-214: nested dict of inference tensors addressed by
    dotted names."""

    def __init__(self, tree):
        if not isinstance(tree, dict):
            tree = {t.name: t for t in tree}
        self._tree = _nest(tree)

    def flatten(self) -> dict:
        """Leaf tensors keyed by their dotted path (types/theta.py:121-134)."""
        out = {}

        def walk(prefix, node):
            for key, value in node.items():
                path = f"{prefix}.{key}" if prefix else str(key)
                if isinstance(value, dict):
                    walk(path, value)
                else:
                    out[path] = value

        walk("", self._tree)
        return out

    @property
    def keys(self):
        return self._tree.keys()

    @property
    def tree(self):
        return self._tree

    @staticmethod
    def _parts(names):
        out = []
        for n in names:
            out += str(n).split(".")
        return out

    def optional_tensor(self, *names):
        parts = self._parts(names)
        cur = self._tree
        try:
            for part in parts[:-1]:
                cur = cur[part]
        except KeyError:
            raise KeyError(f"Unknown parameter {parts} (in Theta containing {list(self.keys)})")
        return cur.get(parts[-1])

    def tensor(self, *names):
        t = self.optional_tensor(*names)
        if t is None:
            raise KeyError(f"Could not find tensor {'.'.join(self._parts(names))}")
        return t

    def __contains__(self, key) -> bool:
        return key in self._tree

    def __call__(self, *names):
        cur = self._tree
        try:
            for part in self._parts(names):
                cur = cur[part]
        except KeyError:
            raise KeyError(f"Sub-theta {names} not found (of {list(self.keys)})")
        return Theta(cur) if isinstance(cur, dict) else cur

    def to(self, *args, **kwargs) -> "Theta":
        def conv(node):
            if isinstance(node, dict):
                return {k: conv(v) for k, v in node.items()}
            return node.to(*args, **kwargs)

        return Theta(conv(self._tree))
