"""Registration with sharktank's own `ops` registry and model patching.

    import shark_platform_b200.plugin as b200
    b200.register()              # overrides for get_index / einsum_2args
    b200.patch_moe_blocks(model) # swap every MoeBlock for the fused B200 block

`register()` adds, at a positive salience (no override in sharktank uses one, so
these are consulted first; sharktank/ops/_registry.py:211-244):

* `get_index(QuantizedTensor, key)` — `weights[experts, :, :]` on a Q8_0 /
  Q4_K planar tensor returns a lazy handle instead of failing (the reference
  only implements this for Q4_1, ops/default_impls.py:204-218);
* `einsum_2args(Tensor, GatheredExperts, str)` — the MoE einsums of
  `PreGatherFFNMOE` as grouped products on the GPU;
* the same pair for expert-sharded weights: `get_index(SplitPrimitiveTensor,
  key)` (shard_dim 0, shards = quantized tensors) and `einsum_2args(Tensor |
  ReplicatedTensor, ShardedGatheredExperts, str)` — each shard multiplies the
  pairs routed to its experts on its own device and the disjoint partial results
  are added (one process holding all shards, the reference's sharding model).

Both overrides decline (`NotImplemented`) for CPU tensors and other layouts, so
the reference's own dispatch continues unchanged for everything else.
"""
from __future__ import annotations

import torch

from . import moe

_registered = False


def register(salience: int = 10):
    """Idempotent.  Requires `sharktank` to be importable."""
    global _registered
    if _registered:
        return
    import sharktank.ops as st_ops
    from sharktank.types import QuantizedTensor, ReplicatedTensor, SplitPrimitiveTensor

    moe.register_overrides(st_ops, quantized_type=QuantizedTensor, tensor_type=torch.Tensor,
                           salience=salience, split_type=SplitPrimitiveTensor,
                           replicated_type=ReplicatedTensor)
    # SplitPrimitiveTensor has its own __getitem__ (types/tensors.py:1056-1080)
    # that never consults the registry and refuses any key on the split
    # dimension, so `weights[experts, :, :]` on expert-sharded weights cannot
    # reach the override above.  Ask the override first, fall through otherwise.
    reference_getitem = SplitPrimitiveTensor.__getitem__

    def getitem(self, key):
        result = moe.get_index_split(self, key)
        return reference_getitem(self, key) if result is NotImplemented else result

    SplitPrimitiveTensor.__getitem__ = getitem
    _registered = True


def patch_moe_blocks(model, *, regime: str = "auto") -> int:
    """Replaces every `MoeBlock`-shaped child (anything with `.theta`,
    `.expert_count`, `.expert_used_count` and an `experts.activation`) by a
    `B200MoeBlock` built from the same theta, the way sharktank's own
    `Patch.patch_child_modules` intercepts children (utils/patching.py:12-40).
    Returns the number of blocks replaced."""
    replaced = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, moe.B200MoeBlock):
                continue
            if not all(hasattr(child, a) for a in ("theta", "expert_count", "expert_used_count", "experts")):
                continue
            eps = child.ffn_norm.epsilon
            act = getattr(child.experts, "activation", torch.nn.functional.silu)
            new = moe.B200MoeBlock(child.theta, child.expert_count, child.expert_used_count, eps,
                                   act, regime=regime)
            setattr(parent, name, new)
            replaced += 1
    return replaced
