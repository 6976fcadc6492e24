"""Runs the matrix-memory recurrence (or, with --state-space, the state-space one) of given sizes three times, for ncu to
capture one launch of a case that ends by itself:

    python -m research_2_b200.profiling.recurrence_case --heads 12 --dim 32 --vdim 64 --entries 16 --rows 256 &&
    ncu --set full --clock-control none -k regex:outer_scan -s 1 -c 1 -o scan \
        python -m research_2_b200.profiling.recurrence_case --heads 12 --dim 32 --vdim 64 --entries 16 --rows 256

With --time the case is timed inside a CUDA graph of 20 launches and microseconds per launch are printed.
"""
import argparse

import torch

from ..kernels import ops
from .kernel_cases import time_in_graph


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--dim", type=int, default=32, help="rows of a head's state (query/key size; state size N)")
    ap.add_argument("--vdim", type=int, default=64, help="columns of a head's state")
    ap.add_argument("--entries", type=int, default=16)
    ap.add_argument("--rows", type=int, default=256, help="rows of every entry (1: a decode step)")
    ap.add_argument("--state-space", action="store_true")
    ap.add_argument("--time", action="store_true")
    args = ap.parse_args()
    dev, h, dk, dv = "cuda:0", args.heads, args.dim, args.vdim
    t = args.entries * args.rows
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    q_start, slots, fresh = i32([i * args.rows for i in range(args.entries + 1)]), i32(list(range(args.entries))), i32([0] * args.entries)
    if args.state_space:
        xbc = torch.randn(t, h * dv + 2 * dk, device=dev).bfloat16()
        steps, per_head = torch.randn(t, h, device=dev), torch.zeros(h, device=dev)
        state = torch.zeros(args.entries, h * dk * dv, device=dev)
        fn = lambda: ops.ssd_scan(xbc[:, : h * dv], xbc[:, h * dv: h * dv + dk], xbc[:, h * dv + dk:], steps, per_head, per_head, per_head,  # noqa: E731
                                  state, q_start, slots, fresh, h, 1, dk, dv)
    else:
        proj = torch.randn(t, 2 * h * dk + h * dv, device=dev).bfloat16()
        gates = torch.randn(t, 2 * h, device=dev)
        state = torch.zeros(args.entries, h * ops.mlstm_state_floats(dk, dv), device=dev)
        fn = lambda: ops.mlstm_scan(proj[:, : h * dk], proj[:, h * dk: 2 * h * dk], proj[:, 2 * h * dk:], gates, 15.0, dk ** -0.5, state,  # noqa: E731
                                    q_start, slots, fresh, h, dk, dv)
    if args.time:
        print(f"{time_in_graph(fn):.1f} us a launch")
        return 0
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
