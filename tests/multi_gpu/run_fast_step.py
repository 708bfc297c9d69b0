"""Worker of the tensor-parallel rollout-step test (one process per GPU under ``torch.distributed.run``): the batched
GPU-resident step sharded over the ranks of a ``SymmWorld`` against the same step on one rank with the full model. Every
rank builds the same full model and the same caches, runs the single-rank step locally, then the sharded step together
with its peers; verify-row logits must agree within the bf16 rounding of the staged partial sums, and every rank must
emit the same tokens. Prints ``PASS`` lines; any exception fails the run."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from pear_b200.models.config import HybridConfig  # noqa: E402
from pear_b200.models.hybrid import HybridForCausalLM  # noqa: E402
from pear_b200.parallel.symm import SymmWorld  # noqa: E402
from pear_b200.parallel.tensor_parallel import shard_state, tp_config  # noqa: E402
from pear_b200.rollout.fast_step import FastDecoder  # noqa: E402


def build(cfg, full_state, rank, world, symm, B, n_draft, pages, seed, ar_mode="auto", topk=False):
    local = tp_config(cfg, world) if world > 1 else cfg
    model = HybridForCausalLM(local)
    model.load_state_dict(shard_state(full_state, cfg, rank, world) if world > 1 else full_state, strict=True)
    model = model.cuda().eval()
    for name, p in model.named_parameters():
        if p.dim() >= 2 and "conv1d" not in name:
            p.data = p.data.to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(seed)
    kv_heads_full = cfg.num_kv_heads

    def kv_full():
        return torch.randn(pages, 16, kv_heads_full, cfg.head_dim, device="cuda", generator=g).to(torch.bfloat16)

    def kv_local(t):  # this rank's KV heads of the full cache
        if world == 1:
            return t
        n = local.num_kv_heads
        share = max(1, world // kv_heads_full)
        h0 = (rank // share) if kv_heads_full < world else rank * n
        return t[:, :, h0:h0 + n].contiguous()

    kc = {li: kv_local(kv_full()) for li in cfg.attention_layers}
    vc = {li: kv_local(kv_full()) for li in cfg.attention_layers}
    mk, mv = [kv_local(kv_full())], [kv_local(kv_full())]
    hv = cfg.gdn_v_heads
    rs = {}
    for li in cfg.gdn_layers:
        full_rs = torch.randn(B, hv, 128, 128, device="cuda", generator=g) * 0.05
        rs[li] = full_rs[:, rank * (hv // world):(rank + 1) * (hv // world)].contiguous() if world > 1 else full_rs
    dec = FastDecoder(model, kc, vc, rs, mk, mv, num_slots=B, max_batch=B, n_draft=n_draft, max_blocks_per_seq=16, temperature=0.8, seed=77, symm=symm, ar_mode=ar_mode, topk_logprobs=topk)
    dec.debug_logits = torch.zeros_like(dec.logits)
    kd, vd = cfg.gdn_key_dim, cfg.gdn_value_dim
    for b in range(B):
        conv = {}
        for li in cfg.gdn_layers:
            c = torch.randn(3, cfg.gdn_conv_dim, device="cuda", generator=g) * 0.5
            if world > 1:  # q | k | v sections are cut separately
                c = torch.cat([c[:, o + rank * (n // world):o + (rank + 1) * (n // world)] for o, n in ((0, kd), (kd, kd), (2 * kd, vd))], dim=1)
            conv[li] = c
        dec.assign(b, b, 40 + 17 * b, list(range(1 + 16 * b, 17 + 16 * b)), 11 + b, conv)
    return dec


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    sw = SymmWorld()
    hd = max(2, world)
    cfg = HybridConfig(vocab_size=4096, hidden_size=512, num_layers=4, num_attention_heads=2 * hd, num_kv_heads=hd // 2 if world >= 4 else hd, head_dim=256,
                       gdn_qk_heads=hd, gdn_v_heads=2 * hd, gdn_head_dim=128, intermediate_size=256 * hd, num_mtp_layers=1, init_std=0.05)
    full = HybridForCausalLM(cfg).init_weights(9)
    state = {k: v.to(torch.bfloat16).float() if v.dim() >= 2 else v for k, v in full.state_dict().items()}
    B, n_draft, pages = 3, 3, 64
    Vs = cfg.vocab_size // world
    tp = None
    modes = ["one", "two"]  # one-shot pull and two-shot (reduce-scatter + all-gather) forms of the fused reduction
    if getattr(sw.alloc((64,), torch.float32), "mc_ptr", 0) and os.environ.get("PEAR_TEST_NVLS", "1") != "0":
        modes.append("nvls")  # the two-shot form with the sum and the broadcast done by the switch (multimem)
    elif rank == 0:
        print("note: no multicast address on this platform: the nvls reduction is not exercised", flush=True)
    for ar_mode in modes:
        topk = ar_mode == modes[-1]  # the last pass also produces the top-32 log-prob lists (sharded select + merge over ranks)
        one = build(cfg, state, 0, 1, None, B, n_draft, pages, seed=5, topk=topk)
        tp = build(cfg, state, rank, world, sw, B, n_draft, pages, seed=5, ar_mode=ar_mode, topk=topk)
        steps, T = 6, 1 + n_draft
        same_hist = torch.ones(B, dtype=torch.bool)  # sequences whose committed tokens agree so far
        compared = 0
        for step in range(steps):
            in1, in2 = one.tok_in.view(B, T).cpu(), tp.tok_in.view(B, T).cpu()
            one.step()
            tp.step()
            r1, r2 = one.results(), tp.results()
            one.check()
            tp.check()
            # row t of a sequence depends on its input rows 0 .. t (the drafts are the drafter's near-tie-prone argmax and may
            # differ between the two runs): compare the rows whose inputs agree; there the sharded logits are the full logits'
            # columns up to the bf16 staging of the partial sums
            want, got = one.debug_logits[:, rank * Vs:(rank + 1) * Vs], tp.debug_logits[:, :Vs]
            for b in range(B):
                for t in range(T):
                    if not same_hist[b] or not torch.equal(in1[b, :t + 1], in2[b, :t + 1]):
                        break
                    err, scale = float((got[b * T + t] - want[b * T + t]).abs().max()), float(want[b * T + t].abs().max())
                    assert err < 0.05 * max(1.0, scale), (ar_mode, step, b, t, err, scale)
                    compared += 1
                    if topk:  # the sharded lists against the single-rank ones: same log-probs up to the staging's rounding, and
                        # the same leading token unless the two best are closer than that
                        a_lp, b_lp = r1.topk_logprobs[b, t], r2.topk_logprobs[b, t]
                        assert torch.allclose(a_lp, b_lp, atol=0.05), (step, b, t, a_lp[:4], b_lp[:4])
                        assert int(r1.topk_ids[b, t, 0]) == int(r2.topk_ids[b, t, 0]) or float(a_lp[0] - a_lp[1]) < 0.05
                        assert len(set(r2.topk_ids[b, t].tolist())) == 32
            toks = r2.tokens.cuda()
            gathered = [torch.zeros_like(toks) for _ in range(world)]
            dist.all_gather(gathered, toks)
            assert all(torch.equal(gathered[0], t) for t in gathered), "ranks emitted different tokens"
            same_hist &= (r1.tokens == r2.tokens).all(dim=1)
        assert compared >= steps, compared  # at the very least the first row of one sequence at every step
        agree = bool(same_hist.all())
        if rank == 0:
            print(f"PASS tp_fast_step world {world} reduction {ar_mode} (tokens equal to the single-rank step through all {steps} steps: {agree})", flush=True)
    # timing of the sharded step under graph replay (max over ranks)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        tp.step()
    e1.record()
    torch.cuda.synchronize()
    tp.check()
    t = torch.tensor([e0.elapsed_time(e1) / 10], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"TIMING tp_fast_step world {world}: {float(t):.3f} ms per step (small model)", flush=True)
        print("PASS tp_fast_step_graph", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
