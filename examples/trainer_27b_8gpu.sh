#!/bin/bash
# 27B-shape GRPO update on 8 GPUs: bf16 FSDP over all ranks, Ulysses sequence parallelism 8, gradient checkpointing,
# activation offload to pinned host memory, fused sharded AdamW. 64 sequences of 16k tokens per step.
set -e
RUN=${RUN:-runs/trainer_27b}
python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 --master-port ${PORT:-29512} \
  -m pear_b200.train.main training run_dir=$RUN actor_rollout_ref.model.path=${MODEL:-preset:qwen3_8_27b} \
  trainer.total_training_steps=${STEPS:-1} data.train_batch_size=8 actor_rollout_ref.rollout.n=8 data.max_prompt_length=4096 \
  data.max_response_length=12288 actor_rollout_ref.actor.fsdp_config.ulysses_sequence_parallel_size=8 \
  actor_rollout_ref.model.enable_gradient_checkpointing=true actor_rollout_ref.model.enable_activation_offload=true "$@"
