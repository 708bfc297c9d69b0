"""Timing of the fused all-reduce + residual add + RMSNorm forms of the rollout step on the ranks of one node (one process per
GPU under ``torch.distributed.run``): one-shot pull and two-shot (reduce-scatter + all-gather) at several row counts, CUDA
events, max over ranks, with the staging kernel that precedes them in the step. Prints one line per (form, rows)."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from pear_b200.ops import decode_ops as K  # noqa: E402
from pear_b200.parallel.symm import SymmWorld  # noqa: E402
from pear_b200.rollout.fast_step import SLOT_STEP_AR  # noqa: E402


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    sw = SymmWorld()
    H, rows_max = 5120, 1024
    g = torch.Generator(device="cuda").manual_seed(rank)
    parts = torch.randn(1, rows_max, H, device="cuda", generator=g) * 0.1
    w = torch.zeros(H, device="cuda")
    ws = sw.alloc((3, rows_max, H), torch.bfloat16)
    h_sym, x_sym = sw.alloc((rows_max, H), torch.bfloat16), sw.alloc((rows_max, H), torch.float32)
    x_sym.tensor.zero_()
    ctr, ticket = sw.device_counter(SLOT_STEP_AR), torch.zeros(1, dtype=torch.int32, device="cuda")
    status = K.status_word()
    sms = K.num_sms()
    buf = rows_max * H
    torch.cuda.synchronize()
    dist.barrier()

    def one(rows):
        K.reduce_parts_bf16(parts, 1, ws.tensor, rows, H, buf, ctr)
        K.ar_add_rmsnorm(ws.c_ptrs, sw.flags.c_ptrs, rank, world, SLOT_STEP_AR, ctr, ticket, x_sym.tensor, 0, w, h_sym.tensor, rows, H, buf, 1e-6, 1 << 22,
                         status, 2 * sms)

    def two(rows):
        K.reduce_parts_bf16(parts, 1, ws.tensor, rows, H, buf, ctr)
        K.ar2_add_rmsnorm(ws.c_ptrs, sw.flags.c_ptrs, h_sym.c_ptrs, x_sym.c_ptrs, rank, world, SLOT_STEP_AR, ctr, ticket, 0, False, w, rows, H, buf, 1e-6,
                          1 << 22, status, 2 * sms)

    def stage_only(rows):
        K.reduce_parts_bf16(parts, 1, ws.tensor, rows, H, buf, None)

    for name, fn in (("stage_only", stage_only), ("one_shot", one), ("two_shot", two)):
        for rows in (128, 256, 512, 1024):
            for _ in range(5):
                fn(rows)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(50):
                fn(rows)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 50 * 1e3], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            K.check_status()
            if rank == 0:
                print(f"TIMING world {world} {name} rows {rows}: {float(t):.1f} us per call", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
