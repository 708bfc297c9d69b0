"""Training entry point: ``python -m pear_b200.train.main <recipe> key=value ...``.

The order of upstream ``pear/trainer/main.py:12-32`` and ``runner.py:22-88``: compose the recipe, derive the run sizes
(``RunConfig.prepare``), open the transfer queue, build the trainer engine and the rollout replicas, start the
environment server pools and the agent-loop manager, ``fit``; on the way out (also on error) cancel in-flight prompt
groups, stop the servers and close the queue.

One process hosts one trainer rank. With ``WORLD_SIZE > 1`` (torchrun) the ranks form the FSDP / HSDP / sequence-parallel
groups; rank 0 drives the rollouts. With ``rollout.checkpoint_engine.replica_urls`` set (what ``launch/launch.py`` passes)
the replicas are processes of their own on their own GPUs: rank 0 reaches them over HTTP (``rollout/remote.py``) and sends
weights through a process group that holds only itself and the replica ranks (``weight_sync.StandaloneGroup``), checked by a
heartbeat before every sync. Without it rank 0 hosts the replicas in-process (the single-process recipes and the tests).
"""

from __future__ import annotations

import json
import os
import sys
import time
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..config.loader import compose
from ..loop.agent_loop import AgentLoopConfig
from ..loop.dataset import EpisodeDataset
from ..loop.manager import AgentLoopManager
from ..loop.transfer_queue import TransferQueue
from ..loop.weight_sync import BroadcastTransport, InProcessTransport, StandaloneGroup, SyncConfig, WeightSync
from ..models.config import HybridConfig
from ..models.hybrid import HybridForCausalLM
from ..models import io as model_io
from ..rollout.engine import EngineConfig as RolloutConfig
from ..rollout.server import apply_rollout_kernels, build_server
from ..utils.logging_utils import get_logger
from .checkpoint import CheckpointManager
from .engine import EngineConfig, TrainEngine
from .replay_buffer import ReplayBuffer
from .trainer import Trainer, TrainerConfig

log = get_logger("pear_b200.train")


@dataclass
class RunConfig:
    """Derived sizes (upstream ``pear/trainer/config.py:37-63``): with ``run_sizes.sessions_per_replica`` set,
    ``max_num_seqs = seqs_per_session * sessions_per_replica``, the agent workers cover those slots, and the trainer
    caps in-flight sessions at ``replicas * sessions_per_replica``."""

    cfg: object
    replicas: int = 1

    def prepare(self):
        cfg = self.cfg
        rs = cfg.run_sizes
        ro = cfg.actor_rollout_ref.rollout
        if rs.sessions_per_replica is not None:
            spr = int(rs.sessions_per_replica)
            ro.max_num_seqs = int(rs.seqs_per_session) * spr
            ro.agent.num_workers = max(1, (ro.max_num_seqs * self.replicas + int(rs.seqs_per_agent_worker) - 1) // int(rs.seqs_per_agent_worker))
            cfg.trainer.v1.sampler.max_inflight_sessions = self.replicas * spr
        validate_config(cfg)
        for k, v in cfg.get("env_vars", {}).items():
            os.environ.setdefault(str(k), str(v))
        os.makedirs(cfg.run_dir, exist_ok=True)
        return cfg


# Keys the recipes carry whose other values select algorithms or modes this framework does not implement: they are accepted at
# the implemented value only, so a recipe edited to ask for something else fails at start instead of training something else.
IMPLEMENTED_VALUES = {
    "algorithm.adv_estimator": ("grpo",),
    "algorithm.use_kl_in_reward": (False,),
    "algorithm.rollout_correction.bypass_mode": (True,),
    "algorithm.rollout_correction.loss_type": ("reinforce",),
    "actor_rollout_ref.actor.use_kl_loss": (False,),
    "actor_rollout_ref.actor.use_dynamic_bsz": (True,),
    "actor_rollout_ref.actor.policy_loss.loss_mode": ("bypass_mode",),
    "actor_rollout_ref.actor.strategy": ("fsdp2", "fsdp"),
    "actor_rollout_ref.hybrid_engine": (False,),
    "actor_rollout_ref.rollout.calculate_log_probs": (True,),
    "actor_rollout_ref.rollout.enable_chunked_prefill": (True,),
    "actor_rollout_ref.rollout.multi_turn.max_parallel_calls": (1,),
    "trainer.val_before_train": (False,),
    "trainer.test_freq": (-1, 0),
    "trainer.v1.separate_async.num_warmup_batches": (0,),
    "algorithm.filter_groups.max_num_gen_batches": (0,),
}


def validate_config(cfg) -> None:
    """The role of upstream's ``validate_config`` call (pear/trainer/main.py:12-32): refuse what would be silently ignored."""
    from ..config.loader import MISSING, ConfigError

    bad = []
    for key, allowed in IMPLEMENTED_VALUES.items():
        v = cfg.get_path(key, MISSING)
        if v != MISSING and v not in allowed:
            bad.append(f"{key}={v!r} (implemented: {', '.join(map(repr, allowed))})")
    if bad:
        raise ConfigError("settings this framework does not implement:\n  " + "\n  ".join(bad))


def _model_config(path: str) -> HybridConfig:
    if path.startswith("preset:"):
        return getattr(HybridConfig, path.split(":", 1)[1])()
    return model_io.load_config(path)


class MetricsLog:
    """Per-step metrics to the backends ``trainer.logger`` lists: ``file`` (``metrics.jsonl`` + a one-line-per-step
    ``train.log``), ``console``, ``wandb`` (one ``wandb.log(..., commit=True)`` per trainer step, so a step's metrics appear
    as one row whatever logged them: 3rdparty/verl/patches/0014; the package is imported only when the backend is listed)."""

    def __init__(self, run_dir: str, backends=("console", "file"), project: str = "pear_b200", name: Optional[str] = None):
        self.path = os.path.join(run_dir, "metrics.jsonl")
        self.train_log = os.path.join(run_dir, "train.log")
        self.backends = backends
        self.tensorboard = None
        if "tensorboard" in backends:
            from torch.utils.tensorboard import SummaryWriter  # fails loudly when the backend is asked for and the package is absent

            self.tensorboard = SummaryWriter(log_dir=os.environ.get("TENSORBOARD_DIR") or os.path.join(run_dir, "tensorboard"))
        self.wandb = None
        if "wandb" in backends:
            import wandb  # fails loudly when the backend is asked for and the package is absent

            self.wandb = wandb
            wandb.init(project=project, name=name or os.path.basename(os.path.normpath(run_dir)), dir=run_dir, resume="allow")

    def __call__(self, step: int, m: dict) -> None:
        rec = {"step": step, "time": time.time(), **{k: (float(v) if isinstance(v, (int, float)) else v) for k, v in m.items()}}
        if "file" in self.backends:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
            with open(self.train_log, "a") as f:
                f.write(f"step:{step} - " + " - ".join(f"{k}:{v:.6g}" for k, v in sorted(m.items()) if isinstance(v, (int, float))) + "\n")
        if self.tensorboard is not None:
            for k, v in rec.items():
                if isinstance(v, (int, float)) and k not in ("step", "time"):
                    self.tensorboard.add_scalar(k, v, step)
            self.tensorboard.flush()
        if self.wandb is not None:
            self.wandb.log({k: v for k, v in rec.items() if isinstance(v, (int, float)) and k != "step"}, step=step, commit=True)
        if "console" in self.backends:
            keys = ("data/reward_mean", "actor/pg_loss", "actor/grad_norm", "timing/step_s", "train/staleness_mean")
            log.info("step %d | %s", step, " | ".join(f"{k.split('/')[-1]} {m[k]:.4g}" for k in keys if k in m))


def build_stack(cfg, replicas: int = 1, device: str = "cpu", env_families: Optional[dict] = None, world_group=None):
    """Everything a single-node run needs, wired together. Returns (trainer, closers)."""
    mcfg = _model_config(str(cfg.actor_rollout_ref.model.path))
    ecfg = EngineConfig.from_config(cfg)
    init = None
    mpath = str(cfg.actor_rollout_ref.model.path)
    vcfg = cfg.actor_rollout_ref.model.get("vision", None)
    vision_cfg = None
    if vcfg is not None and bool(vcfg.enable):
        from ..models.vision import FamilyVisionConfig, VisionConfig

        preset = str(vcfg.preset)
        if preset == "checkpoint":  # the tower the model directory carries (model.visual.*, sizes from its vision_config)
            vision_cfg = model_io.load_vision_config(mpath)
            if vision_cfg is None:
                raise ValueError(f"{mpath} has no vision_config: vision.preset=checkpoint needs a multi-modal model directory")
        elif preset.startswith("family_"):
            vision_cfg = getattr(FamilyVisionConfig, preset[len("family_"):])(out_hidden=mcfg.hidden_size)
        else:
            vision_cfg = getattr(VisionConfig, preset)(out_hidden=mcfg.hidden_size)
    train_vision = vision_cfg is not None and bool(vcfg.get("train", False))
    if not mpath.startswith("preset:"):
        from_dir = train_vision and str(vcfg.preset) == "checkpoint"  # the directory's tower trains on: its tensors are part of the start
        m = HybridForCausalLM(mcfg, with_mtp=False, vision=vision_cfg if train_vision else None)
        model_io.load_model_dir(mpath, m, allow_missing=() if (from_dir or not train_vision) else ("visual.",))
        init = m.state_dict()
    if str(device).startswith("cuda"):  # sized on the host before anything is allocated: over capacity is said now, not by the allocator mid-step
        try:
            from .memory_plan import plan as memory_plan

            world = dist.get_world_size(world_group) if world_group is not None else 1
            shard = world if ecfg.fsdp_size in (-1, 0) or ecfg.fsdp_size >= world else ecfg.fsdp_size
            capacity = torch.cuda.get_device_properties(device).total_memory
            mp = memory_plan(mcfg, ecfg, int(cfg.actor_rollout_ref.actor.ppo_max_token_len_per_gpu) * ecfg.ulysses_sequence_parallel_size, shard,
                             hbm_bytes=capacity, raise_if_over=False)
            over = mp.total_device_bytes > 0.92 * capacity
            if int(os.environ.get("RANK", "0")) == 0:
                (log.warning if over else log.info)("trainer memory plan per GPU%s:\n%s", " (OVER the device's capacity)" if over else "", mp.table())
        except Exception as e:  # noqa: BLE001 - a planning note never stops a run
            log.warning("trainer memory plan skipped: %r", e)
    engine = TrainEngine(mcfg, ecfg, device=device, world_group=world_group, seed=int(cfg.trainer.seed), state_dict=init,
                         vision=vision_cfg if train_vision else None)
    rank = engine.rank
    if rank == 0:
        mcfg.save(os.path.join(str(cfg.run_dir), "model_config.json"))  # the offline merger reads it
    queue = TransferQueue(int(cfg.transfer_queue.num_data_storage_units))
    ro = cfg.actor_rollout_ref.rollout
    servers, manager = [], None
    tcfg = TrainerConfig.from_config(cfg)
    ce = ro.checkpoint_engine
    urls = [str(u) for u in (ce.get("replica_urls", None) or [])]
    transport, heartbeat = None, None
    if rank == 0:
        full = engine.full_state_dict(torch.float32)
        if urls:  # replicas are processes of their own: requests over HTTP, weights through a world shared with them only
            from ..rollout.remote import RemoteReplica

            backend = "gloo" if device == "cpu" or str(ce.backend) == "gloo" else "nccl"
            # every rank of a tensor-parallel replica receives for itself: the world is this rank plus all of theirs
            group = StandaloneGroup(str(ce.sync_master), 0, 1 + len(urls) * max(1, int(ro.tensor_model_parallel_size)), backend, device)
            transport = BroadcastTransport(group, 0, device if backend == "nccl" else "cpu")
            heartbeat = group.heartbeat(float(ce.get("heartbeat_timeout_s", 30.0)))
            servers = [RemoteReplica(u, name=f"replica-{i}") for i, u in enumerate(urls)]
            for s in servers:
                s.wait_ready(float(ce.get("ready_timeout_s", 600)))
        for i in range(0 if urls else replicas):
            mtp_cfg = cfg.actor_rollout_ref.model.mtp
            rm = HybridForCausalLM(mcfg, with_mtp=bool(mtp_cfg.enable_rollout))
            rm.load_state_dict(full, strict=False)
            if rm.mtp is not None and not mpath.startswith("preset:"):
                # the frozen drafter comes from files (the base model's directory unless `mtp.drafter_path` names another): the
                # trainer's state has none, and a drafter left at its random init would propose nothing that is accepted
                src = str(mtp_cfg.get("drafter_path", None) or mpath)
                own, seen = dict(rm.state_dict()), set()
                with torch.no_grad():
                    for key, t in model_io.iter_model_tensors(src, only=lambda k: model_io.from_hf_name(k).startswith("mtp.")):
                        name = model_io.from_hf_name(key)
                        if name in own:
                            own[name].copy_(t.to(own[name].dtype))
                            seen.add(name)
                lost = [k for k in own if k.startswith("mtp.") and k not in seen]
                if lost:
                    raise KeyError(f"{src} lacks {len(lost)} drafter tensors (first: {lost[:4]}): set actor_rollout_ref.model.mtp.drafter_path")
            rc = RolloutConfig(num_blocks=int(ro.get("num_blocks", 2048)), block_size=int(ro.block_size), max_num_seqs=int(ro.max_num_seqs),
                               max_num_batched_tokens=int(ro.max_num_batched_tokens), enable_prefix_caching=bool(ro.enable_prefix_caching),
                               num_speculative_tokens=int(cfg.actor_rollout_ref.model.mtp.num_speculative_tokens) if cfg.actor_rollout_ref.model.mtp.enable_rollout else 0,
                               host_blocks=int(ro.get("host_blocks", 0)),
                               host_bytes=int(float(ro.custom.lmcache.l1_size_gb) * (1 << 30)) if bool(ro.custom.lmcache.enable) else 0, seed=int(cfg.trainer.seed) + i)
            rc = apply_rollout_kernels(ro.get("kernels", None), rc, model=rm)  # the family's hooks check and complete the settings
            servers.append(build_server(rm, rc, device, name=f"replica-{i}", fp32_modules=tuple(ro.fp32_modules)))
        families = env_families or {"synthetic": {"env_path": "pear_b200.envs.synthetic.SyntheticEnv", "num_processes": 2,
                                                  "env_kwargs": {"hidden": mcfg.hidden_size, "tokens_per_image": 4}}}
        env_hosts = [str(u) for u in (ro.agent.get("env_hosts", None) or [])]
        if env_hosts and env_families is None:  # environment hosts are processes of their own (the launcher's env role)
            for spec in families.values():
                spec["urls"] = env_hosts
        acfg = AgentLoopConfig(token_budget=int(cfg.data.max_response_length), temperature=float(ro.temperature), top_p=float(ro.top_p), top_k=int(ro.get("top_k", -1)),
                               topk_heads=tcfg.topk_heads, max_model_len=int(ro.max_model_len), max_prompt_length=int(cfg.data.get("max_prompt_length", 0) or 0), log_dir=os.environ.get("PEAR_LOG_DIR"),
                               synthetic_turns=int(ro.multi_turn.synthetic_turns), turn_max_tokens=int(ro.multi_turn.turn_max_tokens),
                               synthetic_reward=ro.multi_turn.synthetic_reward, tool_parser=str(ro.multi_turn.get("format", "fenced_json")),
                               picture_positions=str(ro.get("picture_positions", "sequential")))
        from ..utils.tokenizer import load_tokenizer

        vision = None
        if vision_cfg is not None:
            from ..loop.vision_encoder import VisionEncoder
            from ..models.vision import FamilyVisionConfig, FamilyVisionTower, VisionTower

            family = isinstance(vision_cfg, FamilyVisionConfig)
            tower = (FamilyVisionTower if family else VisionTower)(vision_cfg).init_weights(int(cfg.trainer.seed))
            if family and not mpath.startswith("preset:") and not train_vision:  # the checkpoint's own tower weights
                own = dict(tower.state_dict())
                with torch.no_grad():
                    for key, t in model_io.iter_model_tensors(mpath, only=lambda k: model_io.from_hf_name(k).startswith("visual.")):
                        name = model_io.from_hf_name(key)[len("visual."):]
                        if name in own:
                            own[name].copy_(t.to(own[name].dtype))
            if train_vision:  # the agent loop's copy starts from (and then follows) the trainer's tower
                tower.load_state_dict({k[len("visual."):]: v for k, v in full.items() if k.startswith("visual.")})
            pixel_dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[str(cfg.data.get("pixel_dtype", "fp32"))]
            vision = VisionEncoder(tower, str(vcfg.device), pixel_dtype=pixel_dtype)
        manager = AgentLoopManager(servers, mcfg.hidden_size, families, acfg, queue, num_workers=int(ro.agent.num_workers),
                                   tokenizer=load_tokenizer(mpath), vision=vision)
    else:
        full = engine.full_state_dict(torch.float32)  # collective: every rank takes part
    sam = cfg.trainer.v1.sampler
    replay = ReplayBuffer(queue, tcfg.n, int(sam.max_off_policy_threshold), str(sam.max_off_policy_strategy),
                          bool(cfg.algorithm.filter_groups.enable), sam.max_inflight_sessions)
    files = cfg.data.train_files
    dataset = EpisodeDataset(files if files is not None else {"family": "synthetic", "args": {"task": ["reach"], "seed": list(range(64))}},
                             seed=int(cfg.trainer.seed))
    sync = WeightSync(SyncConfig(int(ce.update_weights_bucket_megabytes), getattr(torch, str(ro.dtype)), tuple(ro.fp32_modules)),
                      transport or InProcessTransport(servers), servers, heartbeat=heartbeat,
                      listeners=[manager.loop.vision.follow] if (manager is not None and manager.loop.vision is not None and train_vision) else None) if rank == 0 else None
    if sync is not None and urls:  # replica processes built their own weights: start them from the trainer's policy
        sync.sync(full, engine.policy_version)
    ckpt = CheckpointManager(str(cfg.run_dir), rank, engine.world, cfg.trainer.max_actor_ckpt_to_keep,
                             barrier=(lambda: dist.barrier(world_group)) if engine.world > 1 else None)
    trainer = Trainer(tcfg, engine, dataset, manager, replay, queue, sync, ckpt, MetricsLog(str(cfg.run_dir), tuple(cfg.trainer.logger)))

    def close():
        if manager is not None:
            manager.close()
        for s in servers:
            s.close()
        queue.close()

    return trainer, close


def main(argv: Optional[list[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    from ..utils.process import dump_stacks_on_signal

    dump_stacks_on_signal()
    recipe = argv.pop(0) if argv and "=" not in argv[0] else "training"
    cfg = RunConfig(compose(recipe, argv)).prepare()
    world_group = None
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
        world_group = dist.group.WORLD
    device = f"cuda:{os.environ.get('LOCAL_RANK', 0)}" if torch.cuda.is_available() else "cpu"
    trainer, close = build_stack(cfg, device=device, world_group=world_group)
    try:
        trainer.fit()
    finally:
        close()
        if world_group is not None:
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
