"""Per-GPU memory of a trainer configuration, from the model's sizes and the engine's switches, before anything is allocated.

What the engine keeps on one GPU (``train/engine.py``, ``parallel/fsdp.py``, ``train/checkpointing.py``):

* the fp32 master shard of every flat unit, and AdamW's two fp32 moments of it (on the host with ``streamed_adamw``);
* the fp32 gradient shard of every unit once its reduce-scatter ran;
* up to two layers gathered in the compute dtype at a time (the running one and the prefetched one), the root unit (embedding,
  head, final norm) gathered for the whole step, one unit's full fp32 gradient while it is flattened for the reduce-scatter;
* with gradient checkpointing one fp32 residual row per token and layer (on the host with activation offload, where two
  layers' worth stay on the device in flight), otherwise every layer's intermediates;
* the intermediates of ONE layer during its recompute + backward, and the head's chunk of logits.

The token count is the rank's slice: ``tokens_per_micro_batch / sequence_parallel_size``. Upstream sizes the same
configuration by hand in its recipe (examples/models/qwen3_8_27b_pear/train/run_stage1.sh:15-45: 64 sequences of 16k tokens,
SP 8, offload); here the recipe can be checked against the GPU's capacity on a CPU.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..models.config import HybridConfig
from .engine import EngineConfig

GIB = float(1 << 30)


@dataclass
class TrainMemoryPlan:
    master_bytes: int
    optimizer_bytes: int
    optimizer_on_host: bool
    grad_shard_bytes: int
    gathered_bytes: int
    flat_grad_bytes: int
    checkpoint_bytes: int
    checkpoints_on_host: bool
    layer_peak_bytes: int
    head_bytes: int
    total_device_bytes: int
    host_bytes: int

    def table(self) -> str:
        rows = [("fp32 master shards", self.master_bytes), ("AdamW moments" + (" (host)" if self.optimizer_on_host else ""), self.optimizer_bytes),
                ("fp32 gradient shards", self.grad_shard_bytes), ("gathered units (2 layers + root)", self.gathered_bytes),
                ("one unit's flat fp32 gradient", self.flat_grad_bytes),
                ("checkpointed residuals" + (" (host, 2 layers in flight)" if self.checkpoints_on_host else ""), self.checkpoint_bytes),
                ("one layer's recompute + backward", self.layer_peak_bytes), ("head chunk", self.head_bytes)]
        lines = [f"{name:48s} {b / GIB:9.2f} GiB" for name, b in rows]
        lines.append(f"{'device total':48s} {self.total_device_bytes / GIB:9.2f} GiB   (host: {self.host_bytes / GIB:.2f} GiB)")
        return "\n".join(lines)


def layer_parameters(cfg: HybridConfig) -> tuple[int, int]:
    """(largest decoder layer, root unit) in parameters."""
    h = cfg.hidden_size
    mlp = 3 * h * cfg.intermediate_size + 2 * h
    attn = h * ((2 if cfg.attn_output_gate else 1) * cfg.q_size) + 2 * h * cfg.kv_size + cfg.q_size * h + 2 * cfg.head_dim
    gdn = (h * cfg.gdn_conv_dim + h * cfg.gdn_value_dim + 2 * h * cfg.gdn_v_heads + cfg.gdn_conv_dim * cfg.conv_kernel + 2 * cfg.gdn_v_heads
           + cfg.gdn_head_dim + cfg.gdn_value_dim * h)
    kinds = set(cfg.layer_types)
    layer = mlp + max(attn if "full_attention" in kinds else 0, gdn if "linear_attention" in kinds else 0)
    return layer, 2 * cfg.vocab_size * h + h


def plan(cfg: HybridConfig, ecfg: EngineConfig, tokens_per_micro_batch: int, shard_world: int, hbm_bytes: int = 180 << 30,
         utilization: float = 0.92, raise_if_over: bool = True) -> TrainMemoryPlan:
    params = cfg.num_parameters()
    layer, root = layer_parameters(cfg)
    cbytes = {"bf16": 2, "fp16": 2, "fp32": 4}[ecfg.param_dtype]
    t = -(-tokens_per_micro_batch // max(1, ecfg.ulysses_sequence_parallel_size))  # this rank's tokens
    h, sp = cfg.hidden_size, max(1, ecfg.ulysses_sequence_parallel_size)
    master = 4 * params // shard_world
    opt = 8 * params // shard_world
    grads = 4 * params // shard_world
    gathered = cbytes * (2 * layer + root)
    flat_grad = 4 * max(layer, root)
    ckpt_all = 4 * t * h * cfg.num_layers
    if ecfg.enable_gradient_checkpointing:
        on_host = bool(ecfg.enable_activation_offload)
        ckpt_dev = 4 * t * h * 2 if on_host else ckpt_all
    else:
        on_host, ckpt_dev = False, 0
    # one layer's live tensors in the recompute + backward (fp32 activations, as the reference statement keeps them, plus their
    # gradients): residual, normed input, the mixer's projections, the MLP's gate / up / product, and the attention's q, k, v
    # for the WHOLE sequence of the heads this rank owns after the all-to-all (heads / sp of t * sp tokens = the same count)
    attn_act = t * (2 * cfg.q_size + 2 * cfg.kv_size + cfg.q_size)
    gdn_act = t * (cfg.gdn_conv_dim * 2 + 2 * cfg.gdn_value_dim + 4 * cfg.gdn_v_heads)
    mlp_act = t * (3 * cfg.intermediate_size + 2 * h)
    layer_peak = 2 * 4 * (2 * t * h + max(attn_act, gdn_act) + mlp_act)
    if not ecfg.enable_gradient_checkpointing:
        layer_peak *= cfg.num_layers  # every layer's intermediates stay for the backward
    k = 1 + max(0, int(ecfg.topk_log_probs))
    head = 4 * min(t, int(ecfg.head_chunk)) * cfg.vocab_size * 2 + 4 * t * (h + 2 * k)  # a chunk of logits and its gradient
    total = master + (0 if ecfg.streamed_adamw else opt) + grads + gathered + flat_grad + ckpt_dev + layer_peak + head
    host = (opt if ecfg.streamed_adamw else 0) + (ckpt_all if on_host else 0)
    p = TrainMemoryPlan(master, opt, bool(ecfg.streamed_adamw), grads, gathered, flat_grad, ckpt_dev if on_host else (ckpt_all if ecfg.enable_gradient_checkpointing else 0),
                        on_host, layer_peak, head, total, host)
    if raise_if_over and total > hbm_bytes * utilization:
        raise MemoryError(f"the trainer plan needs {total / GIB:.1f} GiB per GPU of {hbm_bytes * utilization / GIB:.1f} GiB:\n{p.table()}\n"
                          "shard over more ranks, raise the sequence-parallel size, stream the optimizer state or offload the checkpoints")
    return p


def main(argv=None) -> int:
    """``python -m pear_b200.train.memory_plan <recipe> [--gpus N] [--tokens T] key=value ...``: the plan of a composed recipe."""
    import argparse

    from ..config.loader import compose
    from .main import _model_config

    ap = argparse.ArgumentParser()
    ap.add_argument("recipe", nargs="?", default="training")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=None, help="tokens of one micro-batch (default: actor.ppo_max_token_len_per_gpu x SP)")
    args, overrides = ap.parse_known_args(argv)
    cfg = compose(args.recipe, [o for o in overrides if "=" in o], check_missing=False)
    ecfg = EngineConfig.from_config(cfg)
    mcfg = _model_config(str(cfg.actor_rollout_ref.model.path))
    tokens = args.tokens or int(cfg.actor_rollout_ref.actor.ppo_max_token_len_per_gpu) * ecfg.ulysses_sequence_parallel_size
    shard = args.gpus if ecfg.fsdp_size in (-1, 0) or ecfg.fsdp_size >= args.gpus else ecfg.fsdp_size
    p = plan(mcfg, ecfg, tokens, shard, raise_if_over=False)
    print(f"{mcfg.num_parameters() / 1e9:.2f} B parameters, {tokens} tokens per micro-batch, SP {ecfg.ulysses_sequence_parallel_size}, sharded over {shard} of {args.gpus} GPUs")
    print(p.table())
    return 0 if p.total_device_bytes <= (180 << 30) * 0.92 else 1


if __name__ == "__main__":
    raise SystemExit(main())
