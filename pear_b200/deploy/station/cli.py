"""Run a task on the simulated arm against a model: ``python -m pear_b200.deploy.station.cli --task "..." --client harness
--url http://127.0.0.1:8100 --model <id> --steps 10 --directory runs/station``. ``--client messages`` asks a model server's
``/v1/messages`` directly (``rollout/server.py`` or ``deploy/server.py``); ``--client harness`` goes through the session service
of ``deploy/harness``. Upstream's station CLI (pear/deploy/station/cli.py) opens real arms and a GUI; neither is here."""

from __future__ import annotations

import argparse
import json
import threading

from .agent_loop import StationAgentLoop, system_prompt
from .clients import ContextLimit, HarnessClient, MessagesClient, SessionLost
from .records import TaskRecords
from .robot import CARTESIAN, SimulatedArm


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--task", default="Move the gripper over the green target.")
    ap.add_argument("--client", choices=("harness", "messages"), default="messages")
    ap.add_argument("--url", required=True)
    ap.add_argument("--model", required=True)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--timeout-s", type=float, default=120.0)
    ap.add_argument("--directory", default="runs/station")
    args = ap.parse_args(argv)
    arm = SimulatedArm()
    prompt = system_prompt(args.task, CARTESIAN)
    client = HarnessClient(args.url, args.model, prompt) if args.client == "harness" else MessagesClient(args.url, args.model, prompt)
    health = client.check()
    if health.get("status") != "ok":
        raise SystemExit(f"the model is not available: {health}")
    loop = StationAgentLoop(arm, client, CARTESIAN, args.timeout_s, args.directory, reference_images=(arm.observe().cameras["top"],))
    never, records = threading.Event(), TaskRecords(args.directory)
    try:
        for i in range(args.steps):
            try:
                result = loop.step(never, records.on_event)
            except (ContextLimit, SessionLost) as e:
                print(json.dumps({"turn": i + 1, "blocked": str(e)}))
                break
            print(json.dumps({"turn": i + 1, **result.to_record(), "distance": round(arm.distance(), 4)}))
            if arm.distance() < 0.02:
                break
    finally:
        loop.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
