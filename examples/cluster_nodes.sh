#!/bin/bash
# A job over several nodes: run this same script on every node with its own NODE_RANK. The first TRAIN_NODES nodes train with all
# their GPUs (one torch.distributed.run world, rendezvous on node 0), every other node serves rollout replicas of TP GPUs; node 0
# also runs the environment host and the monitor. The trainer reaches the replicas by their nodes' addresses and sends weights
# through the weight-sync world (rendezvous on node 0); a rollout node ends by itself when the trainer is gone.
#   NODES=10.0.0.1,10.0.0.2,10.0.0.3 NODE_RANK=0 TRAIN_NODES=1 TP=4 ./examples/cluster_nodes.sh     (add --dry-run to print this node's plan)
set -e
RUN=${RUN:-runs/cluster}
python -m pear_b200.launch.launch training --node-addrs ${NODES:?comma-separated addresses of all nodes} --node-rank ${NODE_RANK:?position of this node in NODES} \
  --trainer-nodes ${TRAIN_NODES:-1} --gpus ${GPUS:-8} --rollout-tp ${TP:-4} \
  run_dir=$RUN actor_rollout_ref.model.path=${MODEL:-preset:qwen3_8_27b} trainer.v1.trainer_mode=separate_async \
  data.train_batch_size=64 actor_rollout_ref.rollout.n=8 data.max_response_length=3072 \
  actor_rollout_ref.actor.fsdp_config.ulysses_sequence_parallel_size=${SP:-8} \
  actor_rollout_ref.rollout.multi_turn.synthetic_turns=6 actor_rollout_ref.rollout.multi_turn.turn_max_tokens=512 \
  actor_rollout_ref.rollout.multi_turn.synthetic_reward=bernoulli:0.3 "$@"
