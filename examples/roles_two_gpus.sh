#!/bin/bash
# The roles as processes with the rollout replica on GPUs: one replica of two tensor-parallel ranks (GPUs 0 and 1) in lock-step
# behind one HTTP endpoint, decoding through the batched GPU-resident step with its reductions over NVLink peer memory; a trainer
# process WITHOUT a GPU drives it over HTTP and syncs weights (gloo) after each step. NVLS / multicast stay off: the ranks of a
# replica must be able to end without the others' memory being bound to a multicast object.
set -e
RUN=${RUN:-runs/roles_two_gpus}
NCCL_NVLS_ENABLE=0 TORCH_SYMM_MEM_DISABLE_MULTICAST=1 PYTORCH_CUDA_ALLOC_CONF=expandable_segments:False \
python -m pear_b200.launch.launch training --gpus 2 --trainer-gpus 0 --rollout-tp 2 \
  --replica-master-port ${REPLICA_PORT:-0} --master-port ${PORT:-29531} --rollout-port ${ROLLOUT_PORT:-8131} --env-port ${ENV_PORT:-8231} --sync-port ${SYNC_PORT:-29631} \
  run_dir=$RUN actor_rollout_ref.model.path=preset:tiny_gpu trainer.total_training_steps=${STEPS:-1} trainer.save_freq=0 \
  data.train_batch_size=2 actor_rollout_ref.rollout.n=4 data.max_response_length=32 \
  actor_rollout_ref.rollout.multi_turn.synthetic_turns=1 actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash \
  actor_rollout_ref.rollout.max_model_len=2048 actor_rollout_ref.rollout.max_num_seqs=16 \
  actor_rollout_ref.rollout.checkpoint_engine.backend=gloo actor_rollout_ref.actor.ppo_max_token_len_per_gpu=8192 \
  trainer.logger=[file,console] "$@"
