"""Worker of the multi-GPU kernel tests (one process per GPU under ``torch.distributed.run``): each fused
compute+collective kernel is compared with a plain fp32 PyTorch / NCCL reference of the same op. Prints one ``PASS`` line
per check; any exception fails the run. Timings (CUDA events, max over ranks) are printed for the bench notes."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from pear_b200.models import nvfp4  # noqa: E402
from pear_b200.parallel.symm import SymmWorld  # noqa: E402


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    sw = SymmWorld()
    g = torch.Generator(device="cuda").manual_seed(1234)  # same stream of numbers on every rank
    big = len(sys.argv) > 1 and sys.argv[1] == "big"

    # ---- all-reduce + residual add + RMSNorm
    T, H = 8, 5120
    parts = torch.randn(world, T, H, device="cuda", generator=g) * 0.5
    resid0 = torch.randn(T, H, device="cuda", generator=g)
    w = torch.randn(H, device="cuda", generator=g) * 0.1
    ws = sw.make_ar_workspace(64, H)
    for it in range(3):  # several epochs: both parities of the double buffer
        resid = resid0.clone()
        out = sw.all_reduce_add_rmsnorm(ws, parts[rank].to(torch.bfloat16), resid, w, 1e-6)
        torch.cuda.synchronize()
        sw.check()
        ref_r = resid0 + parts.to(torch.bfloat16).float().sum(0)
        ref = ref_r * torch.rsqrt(ref_r.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + w)
        assert torch.allclose(resid, ref_r, atol=1e-5, rtol=1e-5), (resid - ref_r).abs().max()
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), (out.float() - ref).abs().max()
    if rank == 0:
        print("PASS all_reduce_add_rmsnorm", flush=True)

    # ---- all-gather -> GEMM
    M, N, K = (world * 4096, 8192, 8192) if big else (world * 256, 512, 512)  # big: ~1 ms of GEMM, launch overheads negligible
    a_full = (torch.randn(M, K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    shard = sw.alloc((M // world, K), torch.bfloat16)
    shard.tensor.copy_(a_full[rank * (M // world):(rank + 1) * (M // world)])
    c = sw.ag_gemm(shard, b, torch.float32)
    torch.cuda.synchronize()
    sw.check()
    ref = a_full.float() @ b.float().t()
    err = (c - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err
    sw.ag_gemm_done()
    if rank == 0:
        print("PASS ag_gemm", flush=True)

    # ---- GEMM -> reduce-scatter
    Kl = K // world
    a_loc = a_full[:, rank * Kl:(rank + 1) * Kl].contiguous()
    b_loc = b[:, rank * Kl:(rank + 1) * Kl].contiguous()
    acc = sw.make_rs_accumulator(M // world, N)
    out = sw.gemm_rs(a_loc, b_loc, acc)
    torch.cuda.synchronize()
    sw.check()
    mine = ref[rank * (M // world):(rank + 1) * (M // world)]
    err = (out - mine).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err
    if rank == 0:
        print("PASS gemm_rs", flush=True)

    # ---- weight broadcast fused with NVFP4 requantisation (rank 0 is the trainer)
    rows, k = 384, 1024
    wsrc = (torch.randn(rows, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    staging = sw.alloc((rows, k), torch.bfloat16)
    if rank == 0:
        staging.tensor.copy_(wsrc)
    sw.device_barrier()
    packed, gs = sw.pull_quantize_nvfp4(staging, 0, rows, k)
    torch.cuda.synchronize()
    ref_packed, ref_gs = nvfp4.quantize_packed(wsrc.float())
    assert gs == ref_gs, (gs, ref_gs)
    assert torch.equal(packed.cpu(), ref_packed.cpu()), (packed.cpu() != ref_packed.cpu()).sum()
    sw.device_barrier()
    if rank == 0:
        print("PASS pull_quantize_nvfp4", flush=True)

    # ---- weight sync over NVSwitch: rank 0 stages buckets, every other rank pulls only its tensor-parallel shard
    from pear_b200.loop.weight_sync import SymmTransport, SyncConfig, WeightSync
    from pear_b200.models import hybrid as _hy
    from pear_b200.models.config import HybridConfig as _HC
    from pear_b200.parallel.tensor_parallel import shard_state as _shard_state

    wcfg = _HC(vocab_size=1024, hidden_size=512, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=256, gdn_qk_heads=2,
               gdn_v_heads=4, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=0)
    full_state = {k: v.cuda() for k, v in _hy.HybridForCausalLM(wcfg, with_mtp=False).init_weights(3).state_dict().items()}
    scfg = SyncConfig(bucket_megabytes=4, rollout_dtype=torch.bfloat16, fp32_modules=("norm",))
    for tp_world, nvfp4_mode in ((1, False), (2, False), (1, True)):
        tp_rank = 1 if tp_world == 2 else 0  # every receiver plays the same tensor-parallel rank: the check is per receiver
        tr = SymmTransport(sw, 0, wcfg, tp_rank=tp_rank, tp_world=tp_world, bucket_megabytes=4, nvfp4=nvfp4_mode)
        if rank == 0:
            stats = WeightSync(scfg, tr).sync(full_state, version=7)
            assert stats["weight_sync/buckets"] >= 2
        else:
            got, last = {}, False
            while not last:
                part, version, last = tr.receive()
                got.update(part)
            torch.cuda.synchronize()
            assert version == 7
            from pear_b200.loop.weight_sync import cast_for_rollout

            want = _shard_state({k: cast_for_rollout(k, v, scfg) for k, v in full_state.items()}, wcfg, tp_rank, tp_world)
            assert set(got) == set(want)
            quantised = 0
            for k, v in want.items():
                if isinstance(got[k], tuple):  # NVFP4 on receipt: equal to the torch quantiser on the bf16 weights
                    packed, gs = got[k]
                    ref_packed, ref_gs = nvfp4.quantize_packed(v.float())
                    assert gs == ref_gs and torch.equal(packed.cpu(), ref_packed.cpu()), k
                    quantised += 1
                else:
                    assert got[k].dtype == v.dtype and torch.equal(got[k], v), k
            assert (quantised > 0) == nvfp4_mode
            whole = sum(v.numel() * cast_for_rollout(k, v, scfg).element_size() for k, v in full_state.items())
            if tp_world == 2:  # a shard's worth of bytes crossed NVLink, not the model
                assert tr.bytes_pulled < 0.7 * whole, (tr.bytes_pulled, whole)
        sw.device_barrier()
        sw.check()
    if rank == 0:
        print("PASS weight_sync_symm", flush=True)

    # ---- the same transport in front of a real replica: WeightSync on the trainer rank, receive_all + RolloutServer on the others
    from pear_b200.loop.weight_sync import receive_all
    from pear_b200.rollout.engine import EngineConfig as _EC, SamplingParams as _SP
    from pear_b200.rollout.server import build_server, to_rollout_dtypes

    tr = SymmTransport(sw, 0, wcfg, bucket_megabytes=4)
    new_state = {k: (v * 0.5 if v.dim() >= 2 else v) for k, v in full_state.items()}
    if rank == 0:
        WeightSync(scfg, tr).sync(new_state, version=8)
    else:
        rm = _hy.HybridForCausalLM(wcfg, with_mtp=False)
        rm.load_state_dict({k: v.cpu() for k, v in full_state.items()})
        srv = build_server(to_rollout_dtypes(rm.cuda()), _EC(num_blocks=64, max_num_seqs=2), device="cuda", name=f"replica-{rank}")
        try:
            before = srv.generate(list(range(1, 12)), _SP(max_tokens=3, temperature=0.0)).output
            assert receive_all(tr, srv) == 8 and srv.engine.policy_version == 8
            got_state = srv.engine.model.state_dict()
            for k, v in new_state.items():
                assert torch.equal(got_state[k].float(), cast_for_rollout(k, v, scfg).float().to(got_state[k].dtype).float()), k
            after = srv.generate(list(range(1, 12)), _SP(max_tokens=3, temperature=0.0)).output
            assert len(before) == 3 and len(after) == 3
        finally:
            srv.close()
    sw.device_barrier()
    sw.check()
    if rank == 0:
        print("PASS weight_sync_server", flush=True)

    # ---- vocab-parallel logits all-gather by P2P stores
    Tl, Vs = 8, 4096
    shards = torch.randn(world, Tl, Vs, device="cuda", generator=g)
    full = sw.alloc((16, world * Vs), torch.float32)
    for it in range(2):
        got = sw.all_gather_logits(shards[rank] + it, full)
        torch.cuda.synchronize()
        sw.check()
        want = torch.cat([shards[r] + it for r in range(world)], dim=1)
        assert torch.equal(got, want)
        sw.device_barrier()  # nobody overwrites a buffer a peer is still reading
    if rank == 0:
        print("PASS all_gather_logits", flush=True)

    # ---- sharded argmax exchange
    xbuf = sw.make_argmax_buffer(16)
    for it in range(2):
        sh = shards + it  # [world, Tl, Vs]
        tok, val = sw.sharded_argmax(sh[rank].contiguous(), xbuf)
        torch.cuda.synchronize()
        sw.check()
        full_l = torch.cat([sh[r] for r in range(world)], dim=1)
        assert torch.equal(tok, full_l.argmax(-1)) and torch.equal(val, full_l.max(-1).values)
        sw.device_barrier()
    if rank == 0:
        print("PASS sharded_argmax", flush=True)

    # ---- timings against the unfused NCCL + cuBLAS sequence
    if big:
        gathered = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")

        def unfused_ag():
            dist.all_gather_into_tensor(gathered, shard.tensor)
            return gathered @ b.t()

        def fused_ag():
            r = sw.ag_gemm(shard, b, torch.bfloat16)
            sw.ag_gemm_done()
            return r

        t_ref, t_own = timed(unfused_ag), timed(fused_ag)
        rs_out = torch.empty(M // world, N, dtype=torch.bfloat16, device="cuda")

        def unfused_rs():
            dist.reduce_scatter_tensor(rs_out, a_loc @ b_loc.t())

        t_ref2, t_own2 = timed(unfused_rs), timed(lambda: sw.gemm_rs(a_loc, b_loc, acc))
        sw.check()
        if rank == 0:
            print(f"TIMING world {world} M {M} N {N} K {K}: ag_gemm fused {t_own:.3f} ms vs nccl+cublas {t_ref:.3f} ms; "
                  f"gemm_rs fused {t_own2:.3f} ms vs cublas+nccl {t_ref2:.3f} ms", flush=True)
    # ---- projection GEMM -> all-to-all (token-sharded rows in, head-sharded columns out)
    for (Mq, Nq, Kq) in ((256, world * 384, 512), (128, world * 512, 320)):
        a_all = (torch.randn(world, Mq, Kq, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        wq = (torch.randn(Nq, Kq, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        obuf = sw.make_a2a_buffer(Mq, Nq // world)
        for _ in range(2):
            got = sw.gemm_a2a(a_all[rank], wq, obuf)
            torch.cuda.synchronize()
            sw.check()
            grp = Nq // world
            want = (a_all.float().reshape(world * Mq, Kq) @ wq.float().t())[:, rank * grp:(rank + 1) * grp]
            assert torch.allclose(got.float(), want, atol=3e-2, rtol=2e-2), (got.float() - want).abs().max()
    if rank == 0:
        print("PASS gemm_a2a", flush=True)
    if big:
        Mq, Nq, Kq = 8192, 14336, 5120  # 8192 tokens per rank through a q / k / v projection of the 27B shape
        a_loc2 = (torch.randn(Mq, Kq, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        wq = (torch.randn(Nq, Kq, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        obuf = sw.make_a2a_buffer(Mq, Nq // world)
        recv = torch.empty(world * Mq, Nq // world, dtype=torch.bfloat16, device="cuda")

        def unfused_a2a():
            y = a_loc2 @ wq.t()
            send = y.view(Mq, world, Nq // world).transpose(0, 1).contiguous()
            dist.all_to_all_single(recv, send.view(world * Mq, Nq // world))

        t_ref4, t_own4 = timed(unfused_a2a), timed(lambda: sw.gemm_a2a(a_loc2, wq, obuf))
        sw.check()
        if rank == 0:
            print(f"TIMING world {world} M {Mq} N {Nq} K {Kq}: gemm_a2a fused {t_own4:.3f} ms vs cublas + pack + nccl all-to-all {t_ref4:.3f} ms", flush=True)
        del obuf, recv

    # ---- all-to-all -> GEMM (head-sharded columns in, token-sharded rows out)
    for (Mo, No, Ko) in ((256, 384, world * 128), (128, 640, world * 320)):
        src_all = (torch.randn(world, world * Mo, Ko // world, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        wo = (torch.randn(No, Ko, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        sbuf = sw.alloc((world * Mo, Ko // world), torch.bfloat16)
        for _ in range(2):
            sbuf.tensor.copy_(src_all[rank])
            got = sw.a2a_gemm(sbuf, wo)
            sw.a2a_gemm_done()
            torch.cuda.synchronize()
            sw.check()
            a_mine = torch.cat([src_all[p2][rank * Mo:(rank + 1) * Mo] for p2 in range(world)], dim=1).float()
            want = a_mine @ wo.float().t()
            assert torch.allclose(got, want, atol=3e-2, rtol=2e-2), (got - want).abs().max()
    if rank == 0:
        print("PASS a2a_gemm", flush=True)
    if big:
        Mo, No, Ko = 8192, 5120, 6144  # o_proj of the 27B shape over 8192 tokens per rank
        sbuf = sw.alloc((world * Mo, Ko // world), torch.bfloat16)
        sbuf.tensor.normal_(generator=g)
        wo = (torch.randn(No, Ko, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        recv2 = torch.empty(world, Mo, Ko // world, dtype=torch.bfloat16, device="cuda")

        def unfused_a2a_gemm():
            dist.all_to_all_single(recv2.view(world * Mo, Ko // world), sbuf.tensor)
            return recv2.permute(1, 0, 2).reshape(Mo, Ko) @ wo.t()

        def fused_a2a_gemm():
            r = sw.a2a_gemm(sbuf, wo, torch.bfloat16)
            sw.a2a_gemm_done()
            return r

        t_ref5, t_own5 = timed(unfused_a2a_gemm), timed(fused_a2a_gemm)
        sw.check()
        if rank == 0:
            print(f"TIMING world {world} M {Mo} N {No} K {Ko}: a2a_gemm fused {t_own5:.3f} ms vs nccl all-to-all + unpack + cublas {t_ref5:.3f} ms", flush=True)
        del sbuf, recv2

    # ---- gradient reduce-scatter + clip + sharded AdamW + parameter all-gather in two kernels
    from pear_b200.parallel.symm import FusedShardedAdamW

    n_par = 3 * 1000 * 1000 + 13
    for gdt in (torch.bfloat16, torch.float32):
        opt = FusedShardedAdamW(sw, n_par, grads_dtype=gdt, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_norm=1.0)
        p0 = torch.randn(n_par, device="cuda", generator=g)
        opt.load_parameters(p0)
        ref_p, ref_m, ref_v = p0.clone(), torch.zeros_like(p0), torch.zeros_like(p0)
        for t in (1, 2, 3):
            all_g = (torch.randn(world, n_par, device="cuda", generator=g) * (0.02 if t < 3 else 1e-5)).to(gdt)  # step 3: below the clip
            opt.grads.tensor[:n_par].copy_(all_g[rank])
            norm = opt.step(grad_scale=1.0 / world)
            torch.cuda.synchronize()
            sw.check()
            gsum = all_g.float().sum(0) / world
            ref_norm = gsum.norm()
            gc = gsum * min(1.0, 1.0 / (float(ref_norm) + 1e-6))
            ref_m = 0.9 * ref_m + 0.1 * gc
            ref_v = 0.95 * ref_v + 0.05 * gc * gc
            ref_p = ref_p * (1 - 1e-3 * 0.1) - (1e-3 / (1 - 0.9 ** t)) * ref_m / (ref_v.sqrt() / (1 - 0.95 ** t) ** 0.5 + 1e-8)
            assert abs(float(norm) - float(ref_norm)) <= 1e-4 * float(ref_norm), (float(norm), float(ref_norm))
            got = opt.params.tensor[:n_par].float()
            assert torch.equal(got, ref_p.to(torch.bfloat16).float()) or (got - ref_p).abs().max() <= 1e-2 * ref_p.abs().max(), (got - ref_p).abs().max()
            lo, hi = opt.lo, min(opt.lo + opt.shard, n_par)
            assert torch.allclose(opt.master[: hi - lo], ref_p[lo:hi], atol=1e-5, rtol=1e-5), (opt.master[: hi - lo] - ref_p[lo:hi]).abs().max()
    if rank == 0:
        print("PASS reduce_scatter_adamw", flush=True)
    if big:
        n_big = 1 << 30  # 1 Gi parameters: 2 GiB of bf16 gradients per rank
        opt = FusedShardedAdamW(sw, n_big, grads_dtype=torch.bfloat16)
        opt.grads.tensor.normal_(generator=g)
        rs_in, rs_out = opt.grads.tensor, torch.empty(n_big // world, dtype=torch.bfloat16, device="cuda")
        pm, m1, v1 = (torch.zeros(n_big // world, device="cuda") for _ in range(3))
        full = torch.empty(n_big, dtype=torch.bfloat16, device="cuda")

        def unfused_opt():
            dist.reduce_scatter_tensor(rs_out, rs_in)
            gf = rs_out.float()
            nrm = gf.pow(2).sum()
            dist.all_reduce(nrm)
            gf.mul_(torch.clamp(1.0 / (nrm.sqrt() + 1e-6), max=1.0))
            torch._foreach_lerp_([m1], [gf], 0.1)
            v1.mul_(0.999).addcmul_(gf, gf, value=0.001)
            pm.mul_(1 - 1e-8).addcdiv_(m1, v1.sqrt().add_(1e-8), value=-1e-6)
            dist.all_gather_into_tensor(full, pm.to(torch.bfloat16))

        t_ref3, t_own3 = timed(unfused_opt, iters=5), timed(lambda: opt.step(1.0 / world), iters=5)
        if rank == 0:
            print(f"TIMING world {world} optimizer step over {n_big} parameters: fused {t_own3:.3f} ms vs nccl + torch {t_ref3:.3f} ms", flush=True)
        del opt, full, pm, m1, v1, rs_out

    # ---- tensor-parallel rollout engine: every reduction of the step through the fused all-reduce + add + RMSNorm kernel
    from pear_b200.models import hybrid
    from pear_b200.models.config import HybridConfig
    from pear_b200.ops import lib as kl
    from pear_b200.parallel.tensor_parallel import shard_state, tp_config
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    hd = max(2, world)  # every sharded head count divisible by the world size
    cfg = HybridConfig(vocab_size=4096, hidden_size=512, num_layers=4, num_attention_heads=4 * hd, num_kv_heads=hd, head_dim=128, rotary_dim=64,
                       gdn_qk_heads=hd, gdn_v_heads=2 * hd, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=0)
    full = hybrid.HybridForCausalLM(cfg, with_mtp=False).init_weights(5)
    prompts = [list(range(3, 40)), list(range(100, 117)), [5, 6, 7]]
    tp = hybrid.HybridForCausalLM(tp_config(cfg, world), with_mtp=False)
    tp.load_state_dict(shard_state(full.state_dict(), cfg, rank, world), strict=True)
    outs = {}
    fused_calls = [0]
    plain_ar = sw.all_reduce_add_rmsnorm

    def counting_ar(*a, **k):
        fused_calls[0] += 1
        return plain_ar(*a, **k)

    sw.all_reduce_add_rmsnorm = counting_ar
    for mode in ("nccl", "fused"):
        hybrid.set_tensor_parallel_group(dist.group.WORLD)
        if mode == "fused":
            hybrid.set_tensor_parallel_fused(sw, 256, cfg.hidden_size)
        try:
            eng = RolloutEngine(tp, EngineConfig(num_blocks=128, max_num_seqs=4), device="cuda")
            first = []  # logits of the first step (the three prompts' prefill: the same inputs under both transports)
            plain_forward = eng.runner.forward

            def recording_forward(*a, _f=plain_forward, _first=first, **k):
                res = _f(*a, **k)
                if not _first:
                    _first.append(res[0].float().clone())
                return res

            eng.runner.forward = recording_forward
            before = kl.LAUNCH_COUNT
            outs[mode] = ([r.output for r in eng.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0))], kl.LAUNCH_COUNT - before)
            torch.cuda.synchronize()
            sw.check()
            outs[mode + "_logits"] = first[0]
        finally:
            hybrid.set_tensor_parallel_group(None)
    # the two transports differ only in the rounding of the partial sums (bf16 staging in the fused kernel): the logits of the
    # same inputs agree to a bf16-level bound; a reduction that dropped or doubled a rank's partial would be off by O(1)
    la, lb = outs["nccl_logits"], outs["fused_logits"]
    assert la.shape == lb.shape
    logit_err = float((la - lb).abs().max()) / float(la.abs().max())
    assert logit_err < 2e-2, logit_err
    same = sum(a == b for x, y in zip(outs["nccl"][0], outs["fused"][0]) for a, b in zip(x, y))
    total = sum(len(x) for x in outs["nccl"][0])
    # the fused path rounds the partial sums to bf16 before adding them, so a near-tie of a random-weight model may flip
    # and the sequence then diverges; a wrong reduction would agree on no token at all (vocabulary 4096)
    assert same >= total // 3, (same, total, outs["nccl"][0], outs["fused"][0])
    assert fused_calls[0] >= (2 * cfg.num_layers - 1) * 8, fused_calls  # every step reduced through the NVSwitch kernel
    if rank == 0:
        print(f"PASS tp_rollout_fused (first-step logits within {logit_err:.1e} of the NCCL transport's, relative to their maximum; {same}/{total} tokens equal)", flush=True)

    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
