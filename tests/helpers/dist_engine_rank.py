"""One rank of a CPU (gloo) DistEngine group, started by tests/test_dist_engine_cpu.py."""

import json
import os
import sys

import torch

from parallax_b200.engine.request import SamplingParams
from parallax_b200.parallel import launcher


def _nodes(root):
    stack = list(root.children.values())
    while stack:
        n = stack.pop()
        stack.extend(n.children.values())
        yield n


def main() -> None:
    spec = json.loads(sys.argv[1])
    out_path = sys.argv[2]
    torch.manual_seed(0)
    torch.set_num_threads(2)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    launcher.init_process_group(rank, world, int(os.environ["MASTER_PORT"]), "cpu")
    eng = launcher.build_dist_engine(spec)
    if rank == 0:
        prompts = spec["prompts"]
        eng.mark()
        sp = SamplingParams(max_new_tokens=spec["max_new"], temperature=0.0, ignore_eos=True)
        if spec.get("schema_of"):
            # per prompt a JSON schema (or None): constrained decoding on the rank that samples
            from parallax_b200.engine.request import Request

            reqs = []
            for p, sch in zip(prompts, spec["schema_of"]):
                d = dict(sp.to_dict(), max_new_tokens=spec["max_new"] if sch is None else 120)
                if sch is not None:
                    d.update(json_schema=json.dumps(sch), ignore_eos=False)
                reqs.append(Request(input_ids=list(p), sampling_params=SamplingParams.from_dict(d)))
            for r in reqs:
                eng.add_request(r)
            while eng.has_work():
                eng.step()
            outs = [r.output_ids for r in reqs]
        elif spec.get("lora_of"):
            from parallax_b200.engine.request import Request

            reqs = [Request(input_ids=list(p), sampling_params=SamplingParams.from_dict(sp.to_dict()), lora_path=a)
                    for p, a in zip(prompts, spec["lora_of"])]
            for r in reqs:
                eng.add_request(r)
            while eng.has_work():
                eng.step()
            outs = [r.output_ids for r in reqs]
        else:
            outs = eng.generate(prompts, sp)
        eng.mark()
        probe = eng.elapsed()
        pc = eng.cache.prefix_cache if eng.n_plans == 1 else None
        hits = None if pc is None else pc.hits
        snapshots = None if pc is None else sum(1 for n in _nodes(pc.root) if n.linear_slot is not None)
        eng.shutdown()
        with open(out_path, "w") as f:
            json.dump({"outputs": outs, "steps": eng.steps, "probe": probe, "prefix_hits": hits,
                       "state_snapshots": snapshots}, f)
    else:
        eng.serve_forever()
    import torch.distributed as dist

    dist.destroy_process_group()


if __name__ == "__main__":
    main()
