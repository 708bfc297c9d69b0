"""Two trainer ranks on two GPUs: the step with prefetched all-gathers and overlapped reduce-scatters (side stream) equals
the same step with every collective on the compute stream (to the run-to-run noise of the backward kernels' atomics); only rank 0 builds real weights (the other rank
builds on the meta device and receives its shards)."""

import os
import sys

import torch
import torch.distributed as dist

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(_HERE, "..", ".."))  # the repository root
sys.path.insert(0, os.path.join(_HERE, ".."))  # tests/: the batch builder of the CPU engine test
from test_train_engine_cpu import make_batch  # noqa: E402

from pear_b200.models.config import HybridConfig  # noqa: E402
from pear_b200.parallel.fsdp import FlatUnit  # noqa: E402
from pear_b200.train.engine import EngineConfig, TrainEngine  # noqa: E402


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    cfg = HybridConfig(vocab_size=1024, hidden_size=256, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=256, gdn_qk_heads=2,
                       gdn_v_heads=4, gdn_head_dim=128, intermediate_size=512, num_mtp_layers=0)
    results = {}
    for overlap in (True, False):
        FlatUnit.overlap = overlap
        for sp in (1, 2):
            ecfg = EngineConfig(lr=1e-3, eps=1e-3, clip_grad=1.0, param_dtype="bf16", ulysses_sequence_parallel_size=sp,
                                enable_gradient_checkpointing=True, tf32_matmul=False)
            eng = TrainEngine(cfg, ecfg, device="cuda", world_group=dist.group.WORLD, seed=5)
            # rank 1 never held the model: its parameters were created empty
            batches = [make_batch(cfg, 0), make_batch(cfg, 1, lens=(40, 33, 21))]
            mine = batches if eng.dp_size == 1 else [batches[eng.dp_rank]]
            norms = []
            for _ in range(2):  # the second step gathers the shards the first one updated
                eng.forward_backward_batch(mine)
                norms.append(eng.optimizer_step()["actor/grad_norm"])
            state = eng.full_state_dict()
            torch.cuda.synchronize()
            results[(overlap, sp)] = (norms, {k: v.clone() for k, v in state.items()})
            del eng
    for sp in (1, 2):
        (na, sa), (nb, sb) = results[(True, sp)], results[(False, sp)]
        # the backward kernels add with atomics, so two runs of the SAME schedule already differ in the last bits (measured 6e-9
        # on a norm weight): equal to 1e-6; a gather or a reduction read too early would be off by the size of an update (1e-3)
        assert all(abs(x - y) <= 1e-5 * max(1.0, abs(x)) for x, y in zip(na, nb)), (sp, na, nb)
        for k in sa:
            assert torch.allclose(sa[k], sb[k], atol=1e-6, rtol=0), (sp, k, float((sa[k] - sb[k]).abs().max()))
        assert all(torch.isfinite(v).all() for v in sa.values())
    dist.barrier()
    if rank == 0:
        print(f"PASS fsdp_overlap (grad norms sp1 {results[(True, 1)][0]}, sp2 {results[(True, 2)][0]})", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
