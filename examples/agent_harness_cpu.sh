#!/bin/bash
# The deployment chain on CPU, every part a process of its own: a tiny rollout replica (its Messages routes, a small vision tower for the camera pictures), the agent harness
# in front of it (session service + proxy, the scripted agent as the agent process), and a station session on the simulated
# arm that asks its turns of the harness. The tiny model's weights are random, so its answers hold no action and every turn
# ends "rejected": the run shows the plumbing (sessions, rewriting, sizing, records), not a policy.
set -e
RUN=${RUN:-runs/agent_harness_cpu}
MODEL_PORT=${MODEL_PORT:-8131}
HARNESS_PORT=${HARNESS_PORT:-8132}
mkdir -p $RUN
CUDA_VISIBLE_DEVICES="" python -m pear_b200.rollout.server --model preset:tiny --name tiny --vision tiny --port $MODEL_PORT --num-blocks 256 --max-num-seqs 4 > $RUN/model_server.log 2>&1 &
MODEL_PID=$!
python -m pear_b200.deploy.harness.service upstream=http://127.0.0.1:$MODEL_PORT model=tiny port=$HARNESS_PORT audit_dir=$RUN/audit require_summary_end=false "$@" > $RUN/harness.log 2>&1 &
HARNESS_PID=$!
trap 'kill $HARNESS_PID $MODEL_PID 2>/dev/null || true' EXIT
for i in $(seq 1 240); do
  if python -c "import requests,sys; sys.exit(0 if requests.get('http://127.0.0.1:$HARNESS_PORT/health', timeout=2).json().get('status') == 'ok' else 1)" 2>/dev/null; then break; fi
  sleep 0.5
done
SCRIPTED_AGENT_MAX_TOKENS=16 python -m pear_b200.deploy.station.cli --client harness --url http://127.0.0.1:$HARNESS_PORT --model tiny --steps ${STEPS:-3} --directory $RUN/station
