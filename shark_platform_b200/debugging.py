"""Debug switches of the B200 blocks, read once from the environment.

    B200MOE_DEBUG="tensor_trace,nan_checks,nvtx,dump_path=/tmp/moe"

Same comma-separated `[+|-]name[=value]` syntax as sharktank's TURBINE_LLM_DEBUG
(utils/debugging.py:28-83), with flags for what this library adds:

  tensor_trace   print routing indices, gates and the layer output of every
                 B200MoeBlock call (the reference prints intermediates the same
                 way through `trace_tensor`)
  nan_checks     raise if a layer output holds a NaN or an infinity
  nvtx           bracket every B200MoeBlock / B200PagedAttentionBlock call with an
                 NVTX range
  dump_path=DIR  save experts / gates / output of every call as
                 DIR/<block>_<call>.pt
  status_checks  read the device status word after every layer call (synchronises)

All of them cost a device synchronisation or more per call; none is on by default.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch

FLAGS_ENV_NAME = "B200MOE_DEBUG"
_PART = re.compile(r"^([+-])?([^=]+)(=(.*))?$")


@dataclass
class DebugFlags:
    tensor_trace: bool = False
    nan_checks: bool = False
    nvtx: bool = False
    status_checks: bool = False
    dump_path: Optional[Path] = None
    calls: int = 0

    @property
    def any(self) -> bool:
        return bool(self.tensor_trace or self.nan_checks or self.nvtx or self.status_checks or self.dump_path)

    def set(self, part: str) -> None:
        m = _PART.match(part)
        if not m:
            raise ValueError(f"{FLAGS_ENV_NAME}: cannot parse {part!r}")
        on, name, value = m.group(1) != "-", m.group(2), m.group(4)
        if name in ("tensor_trace", "nan_checks", "nvtx", "status_checks"):
            setattr(self, name, on)
        elif name == "dump_path":
            self.dump_path = Path(value) if (on and value) else None
        else:
            raise ValueError(f"{FLAGS_ENV_NAME}: unknown flag {name!r}")

    @staticmethod
    def parse(settings: str) -> "DebugFlags":
        f = DebugFlags()
        for part in (p.strip() for p in settings.split(",")):
            if part:
                f.set(part)
        return f


flags = DebugFlags.parse(os.environ.get(FLAGS_ENV_NAME, ""))


def trace_tensor(key: str, t: Optional[torch.Tensor]) -> None:
    if flags.tensor_trace and t is not None:
        print(f"::: TRACE {key}({list(t.shape)}, {t.dtype}) =\n{t!r}")


def after_layer(name: str, y: torch.Tensor, experts=None, gates=None) -> None:
    """Hook the blocks call after a layer when any flag is set."""
    flags.calls += 1
    trace_tensor(f"{name}.experts", experts)
    trace_tensor(f"{name}.gates", gates)
    trace_tensor(f"{name}.output", y)
    if flags.nan_checks and not bool(torch.isfinite(y.float()).all()):
        raise FloatingPointError(f"{name}: the output holds a NaN or an infinity")
    if flags.dump_path is not None:
        flags.dump_path.mkdir(parents=True, exist_ok=True)
        torch.save({"experts": None if experts is None else experts.cpu(),
                    "gates": None if gates is None else gates.cpu(), "output": y.cpu()},
                   flags.dump_path / f"{name}_{flags.calls:06d}.pt")
    if flags.status_checks:
        from . import moe

        moe.device_status()
