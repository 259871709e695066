"""Per-op device time inside one steady-state step of the headline workload.

    python benchmarks/step_breakdown.py [--steps 4]

Builds the same closed-loop state as ``bench.py`` (Qwen3-8B, 512 concurrent, 1024 in / 256 out) on one
GPU, switches the stage to the per-layer Python loop and brackets every op with CUDA events (with a
synchronisation after each, so the total is the serialised sum, a little above the real step time).
"""
import sys, os, collections
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
steps = int(sys.argv[sys.argv.index('--steps') + 1]) if '--steps' in sys.argv else 4
import torch
import bench
from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config
from parallax_b200.ops import cuda as cu

cfg = named_config("qwen3-8b")
conc = 512
dev = torch.device("cuda", 0)
eng = Engine(cfg, device=dev, page_size=16, kv_fraction=0.88, max_batch_size=conc, max_num_tokens_per_batch=8192 + conc,
             chunked_prefill_size=4096, enable_prefix_cache=True, max_total_length=1024 + 256 + 64, request_timeout_s=None)
new_prompt = bench.make_workload(0, cfg.vocab_size)
greedy = dict(temperature=0.0, ignore_eos=True)
def admit(n_out, length=1024):
    eng.add_request(Request(input_ids=new_prompt(length), sampling_params=SamplingParams(max_new_tokens=n_out, **greedy), max_total_length=1344))
initial = []
for i in range(conc):
    g = (i * 256) // conc
    r = Request(input_ids=new_prompt(1024 + g), sampling_params=SamplingParams(max_new_tokens=256 - g, **greedy), max_total_length=1344)
    initial.append(r); eng.add_request(r)
def one():
    for req, tok in eng.step():
        if req.is_finished: admit(256)
while any(r.is_prefill for r in initial): one()
for _ in range(3): one()
torch.cuda.synchronize()
eng.stages[0].model._native = False
times = collections.defaultdict(float); counts = collections.Counter()
def wrap(name):
    fn = getattr(cu, name)
    def w(*a, **k):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); r = fn(*a, **k); e.record(); e.synchronize()
        key = name
        if name == "linear":
            key = f"linear M={a[0].shape[0]} N={a[1].shape[0]} K={a[1].shape[1]}"
        times[key] += s.elapsed_time(e); counts[key] += 1
        return r
    setattr(cu, name, w)
for n in ["linear", "rmsnorm", "qk_norm_rope_cache", "attn_decode", "attn_prefill", "gather_rows", "argmax"]:
    wrap(n)
for _ in range(steps): one()
tot = sum(times.values())
print("stats", eng.last_step_stats)
for k, v in sorted(times.items(), key=lambda kv: -kv[1]):
    print(f"{v/steps:8.3f} ms/step  {100*v/tot:5.1f}%  x{counts[k]//steps:4d}  {k}")
print(f"total {tot/steps:.2f} ms/step (serialised)")
