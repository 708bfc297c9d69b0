#!/bin/bash
# Single-GPU NVFP4 batch-1 decode of the 27B-shape model on the persistent decode megakernel.
#   SERVE=1: start the one-session deploy server (OpenAI-style completions on 127.0.0.1:8000)
#   default: the benchmark (4k-token prompt, 3-token speculative verify), as the `nvfp4_bs1` key of bench.py's line
set -e
if [ "${SERVE:-0}" = 1 ]; then
  python -m pear_b200.deploy.server server model=${MODEL:-preset:qwen3_8_27b} "$@"
else
  python bench.py --gpus 1 --steps ${STEPS:-16} --warmup 3 --mk-steps ${MK_STEPS:-256} "$@"
fi
