#!/bin/bash
# Tiny hybrid decoder GRPO step on CPU / gloo, world size 2 (plumbing, no GPU): 4 layers (3 GDN + 1 gated attention),
# hidden 256, vocab 1024, 8 prompts x group 4, 64 sampled tokens, seeded hash reward, score centering.
set -e
RUN=${RUN:-runs/tiny_cpu}
python -m torch.distributed.run --nnodes=1 --nproc-per-node=2 --master-addr 127.0.0.1 --master-port ${PORT:-29511} \
  -m pear_b200.train.main training run_dir=$RUN actor_rollout_ref.model.path=preset:tiny \
  trainer.total_training_steps=${STEPS:-1} data.train_batch_size=8 actor_rollout_ref.rollout.n=4 \
  data.max_response_length=64 actor_rollout_ref.actor.fsdp_config.ulysses_sequence_parallel_size=2 \
  actor_rollout_ref.rollout.multi_turn.synthetic_turns=1 actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash \
  actor_rollout_ref.rollout.max_model_len=2048 actor_rollout_ref.rollout.max_num_seqs=32 actor_rollout_ref.actor.ppo_max_token_len_per_gpu=8192 \
  trainer.logger=[file,console] "$@"
