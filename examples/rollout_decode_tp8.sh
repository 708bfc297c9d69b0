#!/bin/bash
# Rollout decode of the 27B-shape bf16 model, tensor-parallel over N GPUs (default 8): 32 sequences per GPU, 6k-token shared
# prefix + 2k-token suffix, 16-token KV pages, temperature 1.0, 3 MTP draft tokens; prints one JSON line.
set -e
N=${N:-8}
if [ "$N" = 1 ]; then
  python bench.py --gpus 1 --steps ${STEPS:-64} --warmup 4 "$@"
else
  python -m torch.distributed.run --nnodes=1 --nproc-per-node=$N --master-addr 127.0.0.1 --master-port ${PORT:-29513} \
    bench.py --gpus $N --steps ${STEPS:-64} --warmup 4 "$@"
fi
