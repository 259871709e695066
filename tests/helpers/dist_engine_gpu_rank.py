"""One rank of a 2-GPU DistEngine check (started with torchrun by tests/test_tp_gpu.py).

mode "tp": pp=1, tp=2 with the fused kernels; rank 0 compares the logits of one mixed step and
the generated tokens with a single-GPU engine built on its own GPU.
mode "ep": like "tp" on a two-layer Qwen3-30B-A3B-shaped MoE model: attention tensor-parallel,
experts expert-parallel through the dispatch / combine kernels.
mode "pp": pp=2, tp=1; the generated tokens must equal the single-GPU engine's exactly (same
kernels in the same order, only the hand-off differs).
"""

import json
import os
import sys

import torch
import torch.distributed as dist

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config
from parallax_b200.ops import cuda as cu
from parallax_b200.parallel import launcher
from parallax_b200.parallel.dist_engine import DistEngine


def main() -> None:
    import faulthandler

    faulthandler.dump_traceback_later(120, exit=True)   # a stuck rank shows where and ends itself
    mode, out_path = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    launcher.init_process_group(rank, world, int(os.environ["MASTER_PORT"]), "cuda")
    dev = torch.device("cuda", rank)
    cfg = named_config("qwen3-0.6b")
    if mode == "ep":        # Qwen3-30B-A3B layer shapes (128 experts, top-8), two layers
        cfg = named_config("qwen3-30b-a3b")
        cfg.num_hidden_layers = 2
    pp, tp = (2, 1) if mode == "pp" else (1, 2)
    kw = dict(page_size=16, num_blocks=512, max_batch_size=8, max_num_tokens_per_batch=2048, chunked_prefill_size=512,
              max_total_length=2048, seed=0)
    eng = DistEngine(cfg, pp, tp, dev, torch.bfloat16, **kw)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (37, 300, 5, 129, 64, 700)]
    sp = SamplingParams(max_new_tokens=8, temperature=0.0, ignore_eos=True)
    if rank != 0:
        eng.serve_forever()
    else:
        eng.keep_logits = True
        reqs = [Request(input_ids=p, sampling_params=SamplingParams.from_dict(sp.to_dict()), max_total_length=2048)
                for p in prompts]
        for r in reqs:
            eng.add_request(r)
        eng.step()
        first_logits = None if eng.last_logits is None else eng.last_logits.float().clone()
        while eng.has_work():
            eng.step()
        eng.shutdown()
        cu.check_status(dev)
        outs = [r.output_ids for r in reqs]
        ref = Engine(cfg, device=dev, dtype=torch.bfloat16, **kw)
        ref.keep_logits = True
        rreqs = [Request(input_ids=p, sampling_params=SamplingParams.from_dict(sp.to_dict()), max_total_length=2048)
                 for p in prompts]
        for r in rreqs:
            ref.add_request(r)
        ref.step()
        ref_logits = ref.last_logits.float().clone()
        while ref.has_work():
            ref.step()
        routs = [r.output_ids for r in rreqs]
        res = {"mode": mode, "outs": outs, "ref_outs": routs}
        if first_logits is not None and first_logits.shape == ref_logits.shape:
            res["logit_rel_err"] = float((first_logits - ref_logits).norm() / ref_logits.norm())
            res["logit_shape"] = list(ref_logits.shape)
        agree = sum(int(a == b) for x, y in zip(outs, routs) for a, b in zip(x, y))
        res["token_agreement"] = agree / sum(len(x) for x in routs)
        with open(out_path, "w") as f:
            json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
