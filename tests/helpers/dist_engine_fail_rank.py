"""A 2-stage CPU pipeline whose second rank leaves between steps (host-side failure injection):
rank 1 serves a few plans and then exits without a goodbye; rank 0 must notice through the
heartbeat and raise instead of waiting forever."""

import json
import os
import sys
import time

import torch

from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.parallel import launcher


def main() -> None:
    spec = json.loads(sys.argv[1])
    out_path = sys.argv[2]
    torch.set_num_threads(2)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    launcher.init_process_group(rank, world, int(os.environ["MASTER_PORT"]), "cpu")
    eng = launcher.build_dist_engine(spec)
    if rank == 1:
        for _ in range(spec["plans_before_exit"]):
            eng.serve_one()
        eng.finish_sends()
        os._exit(0)          # between steps, nothing of this rank in flight
    eng.liveness_timeout_s = 2.0
    eng.step_timeout_s = 60.0
    reqs = [Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=50, temperature=0.0, ignore_eos=True),
                    max_total_length=256) for p in spec["prompts"]]
    for r in reqs:
        eng.add_request(r)
    t0 = time.time()
    result = {"error": None, "steps": 0}
    try:
        while eng.has_work():
            eng.step()
            result["steps"] += 1
    except Exception as exc:
        result["error"] = f"{type(exc).__name__}: {exc}"
    result["seconds"] = time.time() - t0
    with open(out_path, "w") as f:
        json.dump(result, f)
    os._exit(0)              # the peer is gone: skip collective teardown


if __name__ == "__main__":
    main()
