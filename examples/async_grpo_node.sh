#!/bin/bash
# One node split into roles that run as separate processes: trainer ranks (FSDP + Ulysses SP) on the first TRAIN GPUs,
# rollout replicas of TP GPUs each on the rest, an environment host and the monitor. The trainer's exit ends the run.
#   GPUS=8 TRAIN=4 TP=4 RUN=runs/async ./examples/async_grpo_node.sh  (add --dry-run to print the plan)
set -e
RUN=${RUN:-runs/async_node}
python -m pear_b200.launch.launch training --gpus ${GPUS:-8} --trainer-gpus ${TRAIN:-4} --rollout-tp ${TP:-4} \
  run_dir=$RUN actor_rollout_ref.model.path=${MODEL:-preset:qwen3_8_27b} trainer.v1.trainer_mode=separate_async \
  data.train_batch_size=64 actor_rollout_ref.rollout.n=8 data.max_response_length=3072 \
  actor_rollout_ref.rollout.multi_turn.synthetic_turns=6 actor_rollout_ref.rollout.multi_turn.turn_max_tokens=512 \
  actor_rollout_ref.rollout.multi_turn.synthetic_reward=bernoulli:0.3 "$@"
