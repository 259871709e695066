"""One rank of a multi-GPU DistEngine check (started with torchrun by tests/test_tp_gpu.py).

The layout comes as a string: ``pp<P>``, ``tp<T>`` (fused tensor-parallel kernels for the GQA decoder; heads split over library collectives
for ``@small-mla`` / ``@small-dsa`` / ``@small-hybrid`` / ``@small-msa``), ``dpep<E>`` (expert
parallelism with data-parallel attention) and combinations such as ``pp2tp2`` or ``pp2dpep2``; ``ep2``
is attention tensor-parallel with the experts sharded over the same two ranks. ``#fp8kv`` stores K/V pages as
e4m3, ``%lora`` gives four of the six requests one of two LoRA adapters. Rank 0 runs the same
prompts through a single-GPU engine on its own GPU afterwards and compares:

* the generated tokens, margin-aware: a request is compared up to (not including) its first step at
  which the single-GPU logits' gap between best and second-best token is smaller than the noise that
  a different summation order can cause in bf16; all compared tokens must be equal;
* for layouts where rank 0's first step sees the same rows as the single GPU, the logits of that step.
"""

import json
import os
import re
import sys

import torch
import torch.distributed as dist

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config
from parallax_b200.ops import cuda as cu
from parallax_b200.parallel import launcher
from parallax_b200.parallel.dist_engine import DistEngine


def parse_layout(mode: str):
    legacy = {"tp": "tp2", "pp": "pp2", "ep": "ep2"}
    mode = legacy.get(mode, mode)
    pp = int(m.group(1)) if (m := re.search(r"pp(\d+)", mode)) else 1
    tp = int(m.group(1)) if (m := re.search(r"tp(\d+)", mode)) else 1
    dpep = int(m.group(1)) if (m := re.search(r"dpep(\d+)", mode)) else 1
    moe = "ep" in mode
    if dpep == 1 and (m := re.fullmatch(r"ep(\d+)", mode)):
        tp = int(m.group(1))          # attention tensor-parallel, experts over the same ranks
    return pp, tp, dpep, moe


def _write_adapters(cfg, adir: str) -> None:
    """Two PEFT-format adapters (rank 4 and 8) on q/k/v/o/down of every layer, small enough not to swamp the model."""
    from safetensors.torch import save_file

    D, Hq, Hkv, H, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.hidden_size, cfg.intermediate_size
    dims = {"self_attn.q_proj": (H, Hq * D), "self_attn.k_proj": (H, Hkv * D), "self_attn.v_proj": (H, Hkv * D),
            "self_attn.o_proj": (Hq * D, H)}
    if not cfg.is_moe:
        dims["mlp.down_proj"] = (I, H)
    for seed, (name, r) in enumerate((("x", 4), ("y", 8))):
        g = torch.Generator().manual_seed(100 + seed)
        t = {}
        for li in range(cfg.num_hidden_layers):
            for mod, (n_in, n_out) in dims.items():
                base = f"base_model.model.model.layers.{li}.{mod}"
                t[base + ".lora_A.weight"] = torch.randn(r, n_in, generator=g) * 0.03
                t[base + ".lora_B.weight"] = torch.randn(n_out, r, generator=g) * 0.03
        os.makedirs(os.path.join(adir, name), exist_ok=True)
        save_file(t, os.path.join(adir, name, "adapter_model.safetensors"))
        with open(os.path.join(adir, name, "adapter_config.json"), "w") as f:
            json.dump({"r": r, "lora_alpha": 2 * r}, f)


def main() -> None:
    import faulthandler

    faulthandler.dump_traceback_later(150, exit=True)   # a stuck rank shows where and ends itself
    mode, out_path = sys.argv[1], sys.argv[2]
    # "<layout>@<named config>" picks another model family, "<layout>#fp8kv" an e4m3 KV cache (on both engines)
    # "<layout>%lora": two of the requests use a LoRA adapter each (on both engines)
    mode, _, lora_flag = mode.partition("%")
    mode, _, kv_flag = mode.partition("#")
    mode, _, model = mode.partition("@")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    launcher.init_process_group(rank, world, int(os.environ["MASTER_PORT"]), "cuda")
    dev = torch.device("cuda", rank)
    pp, tp, dpep, moe = parse_layout(mode)
    assert pp * tp * dpep == world, (mode, world)
    cfg = named_config("qwen3-0.6b")
    if moe:        # Qwen3-30B-A3B layer shapes (128 experts, top-8), a few layers
        cfg = named_config("qwen3-30b-a3b")
        cfg.num_hidden_layers = max(2, pp)
    if model:
        cfg = named_config(model)
    kw = dict(page_size=16, num_blocks=512, max_batch_size=8, max_num_tokens_per_batch=2048, chunked_prefill_size=512,
              max_total_length=2048, seed=0)
    if kv_flag == "fp8kv":
        kw["kv_cache_dtype"] = "fp8_e4m3"
    lora_of = [None] * 6
    if lora_flag == "lora":
        adir = os.path.join(os.path.dirname(out_path), "adapters")
        kw["lora"] = {"max_loaded": 2, "max_rank": 8, "paths": {"x": os.path.join(adir, "x"), "y": os.path.join(adir, "y")}}
        lora_of = ["x", None, "y", "x", None, "y"]
        if rank == 0:
            _write_adapters(cfg, adir)       # the other ranks read them when the load arrives with a step plan
    eng = DistEngine(cfg, pp, tp, dev, torch.bfloat16, ep=dpep, **kw)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (37, 300, 5, 129, 64, 700)]
    sp = SamplingParams(max_new_tokens=8, temperature=0.0, ignore_eos=True)
    if rank != 0:
        eng.serve_forever()
    else:
        eng.keep_logits = True
        reqs = [Request(input_ids=p, sampling_params=SamplingParams.from_dict(sp.to_dict()), max_total_length=2048,
                        lora_path=a) for p, a in zip(prompts, lora_of)]
        for r in reqs:
            eng.add_request(r)
        eng.step()
        first_logits = None if eng.last_logits is None else eng.last_logits.float().clone()
        while eng.has_work():
            eng.step()
        eng.shutdown()
        cu.check_status(dev)
        outs = [r.output_ids for r in reqs]
        # step by step, so that the logits of a step and the tokens it returns belong together
        ref = Engine(cfg, device=dev, dtype=torch.bfloat16, async_scheduling=False, **kw)
        ref.keep_logits = True
        rreqs = [Request(input_ids=p, sampling_params=SamplingParams.from_dict(sp.to_dict()), max_total_length=2048,
                         lora_path=a) for p, a in zip(prompts, lora_of)]
        for r in rreqs:
            ref.add_request(r)
        gaps = {r.request_id: [] for r in rreqs}       # per request: top-2 logit gap of every generated token
        ref_logits = None
        noise = 0.0
        while ref.has_work():
            results = ref.step()
            lg = ref.last_logits.float()
            if ref_logits is None:
                ref_logits = lg.clone()
            produced = [rq for rq, tok in results if tok is not None]
            if len(produced) == lg.shape[0]:
                top2 = lg.topk(2, dim=-1).values
                # bf16 summation order moves a logit by a few per cent of the spread; with e4m3 pages a
                # last-bit difference in a key or value can cross a rounding boundary of the 3-bit mantissa,
                # which moves it several times further
                noise = max(noise, (0.2 if kv_flag == "fp8kv" else 0.04) * float(lg.std()))
                for rq, gap in zip(produced, (top2[:, 0] - top2[:, 1]).tolist()):
                    gaps[rq.request_id].append(gap)
        routs = [r.output_ids for r in rreqs]
        res = {"mode": mode}
        if first_logits is not None and ref_logits is not None and first_logits.shape == ref_logits.shape and dpep == 1:
            res["logit_rel_err"] = float((first_logits - ref_logits).norm() / ref_logits.norm())
            res["logit_abs_err"] = float((first_logits - ref_logits).abs().max())
            res["logit_shape"] = list(ref_logits.shape)
            # the two engines run different tile shapes (other row counts per step): a margin counts as clear
            # when it is twice the largest difference that this alone produced on any logit of the first step
            noise = max(noise, 2.0 * res["logit_abs_err"])
        compared = equal = 0
        mismatches = []
        for ri, (r, x, y) in enumerate(zip(rreqs, outs, routs)):
            for i, (a, b) in enumerate(zip(x, y)):
                gp = gaps[r.request_id]
                if i >= len(gp) or gp[i] < noise:
                    break
                compared += 1
                equal += int(a == b)
                if a != b:
                    mismatches.append([ri, i, round(gp[i], 4), a, b])
        res.update({"compared": compared, "equal": equal, "noise": round(noise, 4), "mismatches": mismatches,
                    "outs": outs, "ref_outs": routs})
        agree = sum(int(a == b) for x, y in zip(outs, routs) for a, b in zip(x, y))
        res["token_agreement"] = agree / sum(len(x) for x in routs)
        with open(out_path, "w") as f:
            json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback

        with open(f"{sys.argv[2]}.rank{os.environ.get('RANK', '0')}.err", "w") as f:
            traceback.print_exc(file=f)
        raise
