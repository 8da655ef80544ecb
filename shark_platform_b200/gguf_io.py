"""GGUF files -> tensors the MoE kernels take, unpacked on the GPU.

Mirrors sharktank's loader (sharktank/types/gguf_interop/base.py:141-163,
`load_file`) and its packed tensor classes `Q8_0` / `Q4_K`
(sharktank/types/gguf_interop/layouts.py:31-67 and :70-217): same names, same
constructor arguments, `unpack()` returning the same planar layouts.  What
differs is where the work happens: the raw 34-byte / 144-byte blocks are copied
to the device once and split into planes by `b200moe_gguf_unpack_q8_0` /
`b200moe_gguf_unpack_q4_k`; the reference does it with strided torch views on
the host.

File parsing is the `gguf` package's (`GGUFReader`, memory-mapped), as in the
reference.  ggml stores shapes innermost-first, so the logical shape is the
reversed one (base.py:113-119).
"""
from __future__ import annotations

import ctypes
import os
import warnings
from dataclasses import dataclass, field
from typing import Any, Optional, Union

import numpy as np
import torch

from . import types as T

__all__ = ["Q8_0", "Q4_K", "Dataset", "load_file", "load_properties"]

Q8_0_BLOCK_BYTES = 34  # fp16 d, 32 x int8
Q4_K_BLOCK_BYTES = 144  # fp16 d, fp16 dmin, 12 B of 6-bit scales/mins, 128 B of nibbles

# host -> device staging size for raw blocks (a multiple of both block sizes)
_CHUNK_BYTES = 34 * 144 * 16384  # 80 MB


def _cabi():
    from . import _cabi as C  # raises if the CUDA library is missing

    return C


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _as_bytes(raw) -> torch.Tensor:
    """Flat uint8 view of `raw` (numpy memmap/array or torch tensor of any dtype)."""
    if isinstance(raw, torch.Tensor):
        return raw.contiguous().view(torch.uint8).reshape(-1)
    arr = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    with warnings.catch_warnings():
        # a read-only memory map is only ever read through this tensor
        warnings.simplefilter("ignore", UserWarning)
        return torch.from_numpy(arr)


def _to_device_chunked(raw_bytes: torch.Tensor, device) -> torch.Tensor:
    """Copies a host byte tensor to `device` through pinned staging, `_CHUNK_BYTES` at a time."""
    if raw_bytes.is_cuda:
        return raw_bytes
    n = raw_bytes.numel()
    out = torch.empty(n, dtype=torch.uint8, device=device)
    if n <= _CHUNK_BYTES:
        out.copy_(raw_bytes)
        return out
    stage = torch.empty(_CHUNK_BYTES, dtype=torch.uint8).pin_memory()
    for lo in range(0, n, _CHUNK_BYTES):
        hi = min(n, lo + _CHUNK_BYTES)
        stage[: hi - lo].copy_(raw_bytes[lo:hi])
        out[lo:hi].copy_(stage[: hi - lo], non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the staging buffer is reused
    return out


def _check_shape(kind: str, shape: list[int], block_k: int, block_bytes: int, nbytes: int) -> int:
    if not shape or shape[-1] % block_k != 0:
        raise ValueError(f"{kind}: innermost dimension of {shape} is not a multiple of {block_k}")
    blocks = int(np.prod(shape)) // block_k
    if blocks * block_bytes != nbytes:
        raise ValueError(
            f"{kind}: shape {shape} needs {blocks} blocks = {blocks * block_bytes} bytes, raw data has {nbytes}"
        )
    return blocks


class Q8_0(T.QuantizedTensor):
    """Packed GGUF Q8_0 tensor (gguf_interop/layouts.py:31-67).  `raw` holds
    34-byte blocks in row-major block order; `unpack()` returns a
    BlockScaledLayout with d [..., K/32, 1] fp16 and qs [..., K/32, 32] int8 on
    the device (cached)."""

    def __init__(self, *, raw, shape: list[int], name: str = "<unnamed>", device="cuda"):
        super().__init__(shape=shape, layout_type=T.BlockScaledLayout, name=name)
        self.raw = _as_bytes(raw)
        self._blocks = _check_shape("Q8_0", self.shape, 32, Q8_0_BLOCK_BYTES, self.raw.numel())
        self._device = torch.device(device)
        self._layout: Optional[T.BlockScaledLayout] = None

    def unpack(self) -> T.BlockScaledLayout:
        if self._layout is None:
            C = _cabi()
            with torch.cuda.device(self._device):
                raw = _to_device_chunked(self.raw, self._device)
                d = torch.empty(self._blocks, dtype=torch.float16, device=self._device)
                qs = torch.empty(self._blocks * 32, dtype=torch.int8, device=self._device)
                C.check(C.lib.b200moe_gguf_unpack_q8_0(_ptr(raw), self._blocks, _ptr(d), _ptr(qs), _stream()),
                        "gguf_unpack_q8_0")
            lead = self.shape[:-1] + [self.shape[-1] // 32]
            self._layout = T.BlockScaledLayout(self.shape, d.view(lead + [1]), qs.view(lead + [32]))
            self.raw = self.raw[:0]  # the packed bytes are not needed again
        return self._layout

    def to_planar(self) -> T.PlanarQuantizedTensor:
        return T.PlanarQuantizedTensor(shape=self.shape, layout=self.unpack(), name=self.name)


class Q4_K(T.QuantizedTensor):
    """Packed GGUF Q4_K tensor (gguf_interop/layouts.py:70-217).  `raw` holds
    144-byte super-blocks; `unpack()` returns a
    SuperBlockOffsetScaled_4_6_Layout whose planes have the reference's shapes:
    d, dmin [..., SUP, 1] fp16; sb_scales_high, sb_mins_high [..., SUP, 2];
    sb_scales_low, sb_mins_low [..., SUP, 4]; qs [..., SUP, 8, 16] (uint8)."""

    def __init__(self, *, raw, shape: list[int], name: str = "<unnamed>", device="cuda"):
        super().__init__(shape=shape, layout_type=T.SuperBlockOffsetScaled_4_6_Layout, name=name)
        self.raw = _as_bytes(raw)
        self._blocks = _check_shape("Q4_K", self.shape, 256, Q4_K_BLOCK_BYTES, self.raw.numel())
        self._device = torch.device(device)
        self._layout: Optional[T.SuperBlockOffsetScaled_4_6_Layout] = None

    def unpack(self) -> T.SuperBlockOffsetScaled_4_6_Layout:
        if self._layout is None:
            C = _cabi()
            nb, dev = self._blocks, self._device
            with torch.cuda.device(dev):
                raw = _to_device_chunked(self.raw, dev)
                u8 = lambda n: torch.empty(nb * n, dtype=torch.uint8, device=dev)
                d = torch.empty(nb, dtype=torch.float16, device=dev)
                dmin = torch.empty(nb, dtype=torch.float16, device=dev)
                sch, scl, mnh, mnl, qs = u8(2), u8(4), u8(2), u8(4), u8(128)
                C.check(C.lib.b200moe_gguf_unpack_q4_k(_ptr(raw), nb, _ptr(d), _ptr(dmin), _ptr(sch), _ptr(scl),
                                                       _ptr(mnh), _ptr(mnl), _ptr(qs), _stream()),
                        "gguf_unpack_q4_k")
            lead = self.shape[:-1] + [self.shape[-1] // 256]
            self._layout = T.SuperBlockOffsetScaled_4_6_Layout(
                self.shape,
                d=d.view(lead + [1]), dmin=dmin.view(lead + [1]),
                sb_scales_high=sch.view(lead + [2]), sb_scales_low=scl.view(lead + [4]),
                sb_mins_high=mnh.view(lead + [2]), sb_mins_low=mnl.view(lead + [4]),
                qs=qs.view(lead + [8, 16]),
            )
            self.raw = self.raw[:0]
        return self._layout

    def to_planar(self) -> T.PlanarQuantizedTensor:
        return T.PlanarQuantizedTensor(shape=self.shape, layout=self.unpack(), name=self.name)


_QUANTIZED = {"Q8_0": Q8_0, "Q4_K": Q4_K}
_DENSE = {"F16": np.float16, "F32": np.float32, "F64": np.float64}


@dataclass
class Dataset:
    """types/theta.py:282-356: hyper-parameters plus the root theta."""

    properties: dict = field(default_factory=dict)
    root_theta: Optional[T.Theta] = None


def _scalar(v):
    return v.tolist() if isinstance(v, np.generic) else v


def load_properties(reader) -> dict:
    """The file's key/value metadata as plain Python values (what base.py:64-83
    extracts): strings, numbers, and flat lists of either, plus "schema": "GGUF".
    A scalar of a type the reader has no numpy mapping for is left out; nested or
    otherwise undecodable arrays are an error."""
    from gguf import GGUFValueType

    def element_decoder(kind):
        if kind == GGUFValueType.STRING:
            return lambda part: bytes(part).decode("utf8")
        if kind in reader.gguf_scalar_to_np:
            return lambda part: _scalar(part[0])
        return None

    props: dict[str, Any] = {"schema": "GGUF"}
    for field in reader.fields.values():
        kinds = list(field.types)
        if not kinds:
            raise ValueError(f"GGUF field {field.name!r} carries no value type")
        if kinds[0] != GGUFValueType.ARRAY:
            if len(kinds) != 1:
                raise ValueError(f"GGUF field {field.name!r}: unexpected type chain {kinds}")
            decode = element_decoder(kinds[0])
            if decode is not None:
                props[field.name] = decode(field.parts[-1])
            continue
        decode = element_decoder(kinds[1]) if len(kinds) == 2 else None
        if decode is None:
            raise ValueError(f"GGUF field {field.name!r}: arrays of {kinds[1:]} cannot be decoded")
        props[field.name] = [decode(field.parts[i]) for i in field.data]
    return props


def wrap_tensor(name: str, ggml_shape: list[int], type_name: str, data, device="cuda"):
    """One GGUF tensor as an inference tensor (base.py:107-138).  Dense types
    become DefaultPrimitiveTensor on `device`; Q8_0 / Q4_K become the packed
    classes above (unpacked on first use); anything else raises ValueError, as
    the reference does for types it has no layout for."""
    shape = list(reversed([int(v) for v in ggml_shape]))
    if type_name in _DENSE:
        arr = np.ascontiguousarray(data).view(_DENSE[type_name]).reshape(shape)
        return T.DefaultPrimitiveTensor(name=name, data=torch.from_numpy(arr.copy()).to(device))
    if type_name == "BF16":
        arr = np.ascontiguousarray(data).view(np.int16).reshape(shape)
        return T.DefaultPrimitiveTensor(
            name=name, data=torch.from_numpy(arr.copy()).view(torch.bfloat16).to(device))
    cls = _QUANTIZED.get(type_name)
    if cls is None:
        raise ValueError(f"tensor {name!r}: GGUF type {type_name} has no layout here "
                         f"(dense {sorted(_DENSE)} + BF16, quantized {sorted(_QUANTIZED)})")
    return cls(name=name, raw=data, shape=shape, device=device)


def load_file(gguf_path: Union[str, os.PathLike], device="cuda") -> Dataset:
    """base.py:141-163.  Tensors are keyed by their dotted GGUF names
    (`blk.0.ffn_gate_exps.weight`), so `dataset.root_theta("blk", 0)` is the
    theta a MoE block takes."""
    from gguf import GGUFReader

    reader = GGUFReader(gguf_path)
    tensors = {}
    for t in reader.tensors:
        tensors[t.name] = wrap_tensor(t.name, list(t.shape), t.tensor_type.name, t.data, device=device)
    return Dataset(properties=load_properties(reader), root_theta=T.Theta(tensors))
