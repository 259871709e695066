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
        if spec.get("stress_seed") is not None:
            # a random mix: staggered arrivals, shared prefixes, sampling, penalties, client aborts, a small KV pool
            import random

            from parallax_b200.engine.request import Request

            rnd = random.Random(spec["stress_seed"])
            vocab = eng.cfg.vocab_size
            shared = [rnd.randrange(vocab) for _ in range(48)]
            plan = []
            for i in range(spec.get("stress_requests", 14)):
                n = rnd.randint(1, 90)
                ids = (shared[:min(n, 48)] + [rnd.randrange(vocab) for _ in range(max(n - 48, 0))]) if rnd.random() < 0.4 \
                    else [rnd.randrange(vocab) for _ in range(n)]
                d = dict(max_new_tokens=rnd.randint(1, 7), temperature=rnd.choice([0.0, 0.0, 0.8]), ignore_eos=True)
                if rnd.random() < 0.25:
                    d.update(repetition_penalty=1.3, presence_penalty=0.5)
                if d["temperature"] > 0:
                    d.update(top_k=rnd.choice([-1, 5]), top_p=rnd.choice([1.0, 0.9]))
                adapter = None
                feats = spec.get("stress_features") or []
                if "schema" in feats and rnd.random() < 0.3:
                    d.update(json_schema=json.dumps(spec["stress_schema"]), max_new_tokens=60, ignore_eos=False)
                    ids = [t % 250 for t in ids]
                elif "lora" in feats and rnd.random() < 0.5:
                    adapter = rnd.choice(sorted(spec["lora"]["paths"]))
                plan.append((rnd.randint(0, 25), Request(input_ids=ids, sampling_params=SamplingParams.from_dict(d),
                                                         lora_path=adapter, return_probs=rnd.random() < 0.4),
                             rnd.random() < 0.15))
            reqs = [r for _a, r, _k in plan]
            step, aborted = 0, set()
            while plan or eng.has_work():
                for a, r, _k in [x for x in plan if x[0] <= step]:
                    eng.add_request(r)
                plan = [x for x in plan if x[0] > step]
                eng.step()
                step += 1
                if step % 7 == 3:       # a client goes away now and then
                    live = [r for r in reqs if not r.is_finished and r.output_ids and r.request_id not in aborted]
                    if live and rnd.random() < 0.5:
                        victim = rnd.choice(live)
                        aborted.add(victim.request_id)
                        eng.abort_request(victim.request_id)
                assert step < 3000, "the engine does not drain"
            outs = [r.output_ids for r in reqs]
            spec["_stress"] = {"status": [r.status.name for r in reqs], "want": [r.sampling_params.max_new_tokens for r in reqs],
                               "aborted": [r.request_id in aborted for r in reqs],
                               "live_requests": sum(len(pl.cache.reqs) for pl in eng.planners),
                               "free_blocks": [pl.cache.num_free_blocks() for pl in eng.planners],
                               "tree_blocks": [0 if pl.cache.prefix_cache is None else pl.cache.prefix_cache.num_nodes
                                               for pl in eng.planners],
                               "num_blocks": eng.num_blocks, "steps": step,
                               "schema": [bool(r.sampling_params.json_schema) for r in reqs],
                               "probs_ok": [(not r.return_probs) or (len(r.output_probs) == len(r.output_ids)
                                                                     and all(0.0 <= p <= 1.0 + 1e-6 for p in r.output_probs))
                                            for r in reqs],
                               "lora_pins": None if eng.lora is None else sum(eng.lora.pins.values()),
                               "grammars_known": len(eng._grammar_known)}
        elif spec.get("schema_of"):
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
                       "state_snapshots": snapshots, "stress": spec.get("_stress")}, f)
    else:
        eng.serve_forever()
    import torch.distributed as dist

    dist.destroy_process_group()


if __name__ == "__main__":
    main()
