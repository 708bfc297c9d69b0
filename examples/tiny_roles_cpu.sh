#!/bin/bash
# The roles of a node as separate processes, on CPU / gloo (plumbing, no GPU): two trainer ranks (FSDP + Ulysses SP 2), one
# rollout replica of two tensor-parallel ranks running in lock-step behind one HTTP endpoint, an environment host and the
# monitor. The trainer reaches the replica over HTTP and syncs weights through a process group of its own; its exit ends
# the run and takes the other roles with it.
set -e
RUN=${RUN:-runs/tiny_roles_cpu}
CUDA_VISIBLE_DEVICES="" python -m pear_b200.launch.launch training --gpus 4 --trainer-gpus 2 --rollout-tp 2 \
  --replica-master-port ${REPLICA_PORT:-0} --master-port ${PORT:-29521} --rollout-port ${ROLLOUT_PORT:-8121} --env-port ${ENV_PORT:-8221} --sync-port ${SYNC_PORT:-29621} \
  run_dir=$RUN actor_rollout_ref.model.path=preset:tiny trainer.total_training_steps=${STEPS:-2} data.train_batch_size=4 \
  actor_rollout_ref.rollout.n=4 data.max_response_length=48 \
  actor_rollout_ref.actor.fsdp_config.ulysses_sequence_parallel_size=2 \
  actor_rollout_ref.rollout.multi_turn.synthetic_turns=1 actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash \
  actor_rollout_ref.rollout.max_model_len=2048 actor_rollout_ref.rollout.max_num_seqs=16 actor_rollout_ref.actor.ppo_max_token_len_per_gpu=8192 \
  trainer.logger=[file,console] "$@"
