"""Runs one synthetic MoE layer three times: a small, fixed program to put under
`ncu` (one kernel, a few launches, a few hundred MB on the device).

    python -m shark_platform_b200.profile_case <regime> <tokens> <ffn> [Q8_0|Q4_K|DENSE] [hidden]

regime: auto | stream | tensor.  Hidden defaults to 4096, 8 experts, top-2.
"""
import sys

import torch

from . import moe, synthetic as syn


def main(argv):
    regime, tokens, ffn = argv[0], int(argv[1]), int(argv[2])
    kind = argv[3] if len(argv) > 3 else syn.Q8_0
    hidden = int(argv[4]) if len(argv) > 4 else 4096
    spec = syn.CaseSpec("profile", tokens, hidden, ffn, kind=kind, seed=1)
    case = syn.make_case(spec)
    block = syn.case_block(case, regime=regime)
    h = syn.case_input(case)
    for _ in range(3):
        block(h)
    torch.cuda.synchronize()
    print("device status", moe.device_status())


if __name__ == "__main__":
    main(sys.argv[1:])
