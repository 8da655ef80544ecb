"""Stand-in for the `iree` packages so that sharktank's torch-eager path imports.

Test scaffolding only: it exists so that `make_golden.py` and the optional
reference cross-checks can import sharktank from a source checkout on a
machine without iree-turbine.  The IREE custom kernels become callables that
raise, except the rotary-embedding kernel, which has an eager stand-in so that
the reference's whole model can run for the model-level test.  The product never imports this file.
"""
import logging
import sys
import types


class _Anything:
    """Placeholder class: any attribute is another placeholder."""

    def __init__(self, *a, **k):
        pass

    def __class_getitem__(cls, item):
        return cls


class _Trait:
    def __init__(self, *a, **k):
        self.args, self.kwargs = a, k

    @classmethod
    def get(cls, tensor):
        return getattr(tensor, "_stub_trait_" + cls.__name__, None)

    def set(self, tensor):
        setattr(tensor, "_stub_trait_" + type(self).__name__, self)


class DeviceTensorTrait(_Trait):
    pass


class ExternalTensorTrait(_Trait):
    def __init__(self, external_scope="", external_name=""):
        self.external_scope = external_scope
        self.external_name = external_name


class DeviceAffinity(_Anything):
    pass


class ParameterArchive(_Anything):
    pass


class ParameterArchiveEntry(_Anything):
    pass


class ParameterArchiveBuilder(_Anything):
    def add_tensor(self, *a, **k):
        raise NotImplementedError("iree stub: no parameter archives")

    add_blob = save = add_tensor


def _eager_apply_rotary_embedding(input, table):
    """Eager stand-in for the one IREE custom kernel the model-level test cannot
    do without (kernels/rotary.py with templates/rotary_embedding.mlir): for
    input [bs, sl, heads, dim] and angles table [bs, sl, dim], element pairs
    (2i, 2i+1) are rotated, each output element using the angle stored at its
    own index: out[2i] = x[2i]*cos(t[2i]) - x[2i+1]*sin(t[2i]),
    out[2i+1] = x[2i+1]*cos(t[2i+1]) + x[2i]*sin(t[2i+1]).  Not checked against
    IREE's output (iree-turbine is not installable here): the test that uses it
    runs the same stand-in on both sides of its comparison."""
    import torch

    t = table.unsqueeze(2)
    cos, sin = torch.cos(t), torch.sin(t)
    real, imag = input[..., 0::2], input[..., 1::2]
    out = torch.empty_like(input)
    out[..., 0::2] = real * cos[..., 0::2] - imag * sin[..., 0::2]
    out[..., 1::2] = imag * cos[..., 1::2] + real * sin[..., 1::2]
    return out


_EAGER = {"apply_rotary_embedding": _eager_apply_rotary_embedding}


class CustomOp:
    @staticmethod
    def register(*, library=None, **_):
        def deco(cls):
            if cls.__name__ in _EAGER:
                return _EAGER[cls.__name__]

            def unavailable(*a, **k):
                raise RuntimeError(f"iree stub: custom kernel {cls.__name__} unavailable")

            unavailable.__name__ = cls.__name__
            return unavailable

        return deco


def _module(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)

    def _getattr(attr):
        if attr.startswith("__"):
            raise AttributeError(attr)
        return type(attr, (_Anything,), {})

    m.__getattr__ = _getattr
    m.__path__ = []
    sys.modules[name] = m
    return m


def install():
    if "iree.turbine" in sys.modules:
        return
    iree = _module("iree")
    turbine = _module("iree.turbine")
    aot = _module(
        "iree.turbine.aot",
        DeviceTensorTrait=DeviceTensorTrait,
        ExternalTensorTrait=ExternalTensorTrait,
        DeviceAffinity=DeviceAffinity,
        ParameterArchive=ParameterArchive,
        ParameterArchiveEntry=ParameterArchiveEntry,
        ParameterArchiveBuilder=ParameterArchiveBuilder,
    )
    ops = _module("iree.turbine.ops")
    ops_iree = _module(
        "iree.turbine.ops.iree", transfer_to_logical_device=lambda ordinal, t: t
    )
    support = _module("iree.turbine.support")
    slog = _module("iree.turbine.support.logging", get_logger=logging.getLogger)
    irimp = _module("iree.turbine.support.ir_imports")
    runtime = _module("iree.turbine.runtime")
    op_reg = _module(
        "iree.turbine.runtime.op_reg",
        CustomOp=CustomOp,
        def_library=lambda name: name,
    )
    transforms = _module("iree.turbine.transforms")
    merger = _module("iree.turbine.transforms.merger")
    compiler = _module("iree.compiler")
    cir = _module("iree.compiler.ir")
    iree.turbine, iree.compiler = turbine, compiler
    turbine.aot, turbine.ops, turbine.support = aot, ops, support
    turbine.runtime, turbine.transforms = runtime, transforms
    ops.iree = ops_iree
    support.logging, support.ir_imports = slog, irimp
    runtime.op_reg = op_reg
    transforms.merger = merger
    compiler.ir = cir
