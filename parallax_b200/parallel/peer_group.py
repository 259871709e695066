"""A pipeline peer whose layers run tensor-parallel over the GPUs of its node.

In the reference every pipeline peer may itself be tensor-parallel: the launcher starts one executor process per
rank and rank 0 hands the batch to the others (``src/parallax/launch.py:171-183``,
``src/parallax/server/executor/sglang_executor.py:560-571``); the scheduler tells a joining node to use all of
its GPUs that way (``src/backend/server/rpc_connection_handler.py:181``). Here the node process is rank 0: it owns
the peer executor (scheduler, KV bookkeeping, packets) and this group; ranks 1..T-1 are follower processes that run
the same stage forward on the plans rank 0 publishes through the in-box control channel. Incoming activations are
broadcast to the ranks, each takes its row shard (the residual stream is sharded by rows inside the stage), and
the stage output is gathered back on every rank - rank 0 alone uses it.

Followers are started with ``python -m parallax_b200.parallel.peer_group '<spec json>'``.
"""

from __future__ import annotations

import json
import logging
import os
import subprocess
import sys
import uuid
from typing import Optional

import torch
import torch.distributed as dist

from parallax_b200.engine.batch import BatchBuilder
from parallax_b200.engine.worker import StageWorker
from parallax_b200.models.config import ModelConfig
from parallax_b200.parallel.ctrl_channel import CtrlChannel

logger = logging.getLogger(__name__)

_ARRAYS = ("ids", "pos", "slots", "p_q", "p_ctx", "p_tables", "d_ctx", "d_tables", "logit_rows", "seq_rows")


class TPStageGroup:
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None, page_size: int = 16,
                 num_blocks: Optional[int] = None, kv_fraction: float = 0.8, max_batch_size: int = 8,
                 max_num_tokens_per_batch: int = 16384, max_total_length: int = 32768, seed: int = 0,
                 weights: Optional[dict] = None, kv_cache_dtype: Optional[str] = None, fused: Optional[bool] = None,
                 lora: Optional[dict] = None):
        assert dist.is_initialized(), "init the node's process group first (one rank per GPU of the node)"
        from parallax_b200.models.registry import family_of
        from parallax_b200.parallel.tp_comm import CollectiveTPComm, FusedTPComm

        self.cfg = cfg
        self.device = torch.device(device)
        self.rank, self.tp = dist.get_rank(), dist.get_world_size()
        on_gpu = self.device.type == "cuda"
        self.ctrl = dist.new_group(list(range(self.tp)), backend="gloo")
        self.tp_group = dist.new_group(list(range(self.tp)), backend="nccl" if on_gpu else "gloo")
        family = family_of(cfg.architecture)
        if cfg.is_moe and family != "decoder":
            raise ValueError("a tensor-parallel cluster node serves the GQA decoder families and dense MLA / hybrid "
                             "stages; MoE stages of the other families run under `serve --tp-size`")
        if (on_gpu if fused is None else fused) and family == "decoder":
            comm = FusedTPComm(self.tp_group, self.tp, self.rank, self.device, max_num_tokens_per_batch, cfg.hidden_size,
                               max_n=cfg.hidden_size,
                               max_k=max(cfg.hidden_size, cfg.intermediate_size // self.tp, cfg.q_size // self.tp))
        else:
            comm = CollectiveTPComm(self.tp_group, self.tp, self.rank, align=128 if on_gpu else 1)
        self.comm = comm
        box = [f"pxl_peer_{os.getpid()}_{uuid.uuid4().hex[:8]}" if self.rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=self.ctrl)
        max_blocks = (max_total_length + page_size - 1) // page_size + 1
        slot_bytes = 16 * (max_num_tokens_per_batch + max_batch_size) + 4 * max_batch_size * (max_blocks + 8) + (64 << 10)
        slot_bytes = max(1 << 18, (slot_bytes + 4095) // 4096 * 4096)
        if self.rank == 0:
            self.chan = CtrlChannel(box[0], create=True, n_readers=self.tp - 1, slots=8, slot_bytes=slot_bytes)
        dist.barrier(group=self.ctrl)
        if self.rank != 0:
            self.chan = CtrlChannel(box[0], create=False, n_readers=self.tp - 1, reader_index=self.rank - 1, slots=8,
                                    slot_bytes=slot_bytes)
        self.worker = StageWorker(cfg, start_layer, end_layer, self.device, dtype, page_size, num_blocks=num_blocks,
                                  kv_fraction=kv_fraction, seed=seed, weights=weights,
                                  max_positions=max_total_length + 8, tp_rank=self.rank, tp_size=self.tp,
                                  tp_group=self.tp_group, comm=comm, kv_cache_dtype=kv_cache_dtype,
                                  num_linear_slots=max(max_batch_size * 2, 16) if cfg.has_linear_layers else 0)
        nb = torch.tensor([self.worker.num_blocks], dtype=torch.int64)
        dist.all_reduce(nb, op=dist.ReduceOp.MIN, group=self.ctrl)      # every rank must agree on the KV blocks
        self.worker.num_blocks = self.num_blocks = int(nb)
        self.builder = BatchBuilder(self.device, max_num_tokens_per_batch + max_batch_size, max_batch_size, max_blocks)
        self.on_command = None          # followers: callable(name, payload) for commands other than a forward
        if lora:
            # per-request adapters: every rank keeps its slice of each resident adapter (see TPLoRAStack); rank 0
            # decides which adapter lives in which slot and sends the loads as commands
            from parallax_b200.loader.lora import TPLoRAStack

            if not hasattr(self.worker.model, "lora") or family != "decoder":
                raise ValueError("per-request LoRA on a tensor-parallel node needs a GQA decoder family")
            self.worker.model.lora = TPLoRAStack(self.worker.model, int(lora.get("max_loaded") or 4),
                                                 int(lora.get("max_rank") or 64))
        import threading

        self._lock = threading.Lock()   # rank 0: forwards and commands are published (and run here) one at a time

    # ------------------------------------------------------------------ one forward on every rank
    def forward(self, arrays: dict, hidden: Optional[torch.Tensor], want_logits: bool, lora_ids=None):
        """Rank 0: run the stage on a planned batch. ``hidden`` ``[T, H]`` (later peers) or None (first peer);
        ``lora_ids``: adapter slot of every token row (int32, -1 = none) when some request uses an adapter.
        Returns ``(stage output [T, H] or None on the last peer, logits or None)``."""
        plan = {"cmd": "fwd", "arrays": {k: arrays[k] for k in _ARRAYS}, "rows": int(arrays["pos"].shape[0]),
                "has_hidden": hidden is not None, "want_logits": bool(want_logits), "lora_ids": lora_ids}
        with self._lock:
            self.chan.publish(plan)
            return self._execute(plan, hidden)

    def _execute(self, plan: dict, hidden: Optional[torch.Tensor]):
        a, T = plan["arrays"], plan["rows"]
        model = self.worker.model
        rows_lora = plan.get("lora_ids")
        fb = self.builder.build(a["ids"] if model.is_first else None, a["pos"], a["slots"], a["p_q"], a["p_ctx"],
                                a["p_tables"], a["d_ctx"], a["d_tables"], a["logit_rows"], a.get("seq_rows"),
                                extra={"lora_ids": rows_lora} if rows_lora is not None else None)
        if rows_lora is not None:
            fb.extras["lora_ids_host"] = rows_lora
        rp = self.comm.rows_per_rank(T)
        with torch.inference_mode():
            if plan["has_hidden"]:
                buf = torch.zeros((self.tp * rp, self.cfg.hidden_size), dtype=self.worker.dtype, device=self.device)
                if self.rank == 0:
                    buf[:T].copy_(hidden)
                dist.broadcast(buf, src=0, group=self.tp_group)
                h = buf[self.rank * rp:(self.rank + 1) * rp].contiguous()
            else:
                h = model._embed_shard(fb, rp)
            h = model.forward_layers_tp(h, fb)
            if model.is_last:
                return None, (model.logits_tp(h, fb) if plan["want_logits"] else None)
            return self.comm.all_gather_rows(h)[:T], None

    def command(self, name: str, payload=None, local=None):
        """Rank 0: have every follower run ``on_command(name, payload)`` (e.g. a weight refit) in plan order;
        ``local()`` is this rank's share, run at the same place in that order. Returns what ``local`` returns."""
        with self._lock:
            self.chan.publish({"cmd": name, "payload": payload})
            return local() if local is not None else None

    # ------------------------------------------------------------------ followers
    def serve_forever(self) -> None:
        parent = os.getppid()
        while True:
            try:
                plan = self.chan.receive(timeout_s=5.0)
            except TimeoutError:
                if os.getppid() != parent:      # the node process is gone: nothing will ever arrive
                    return
                continue
            if plan["cmd"] == "stop":
                return
            if plan["cmd"] == "fwd":
                self._execute(plan, None)
            elif self.on_command is not None:
                self.on_command(plan["cmd"], plan.get("payload"))

    def shutdown(self) -> None:
        if self.rank == 0:
            try:
                self.chan.publish({"cmd": "stop"}, timeout_s=5.0)
            except Exception:
                pass
        self.chan.close()


# ---------------------------------------------------------------------- process plumbing
def build_group(spec: dict) -> TPStageGroup:
    """The same construction on every rank of the node (``spec`` as written by :func:`launch_followers`)."""
    from parallax_b200.models.config import config_from_hf, named_config

    rank = dist.get_rank()
    if spec.get("model_path"):
        with open(os.path.join(spec["model_path"], "config.json")) as f:
            cfg = config_from_hf(json.load(f))
    else:
        cfg = named_config(spec["model_name"])
    on_gpu = spec.get("device_type", "cuda") == "cuda"
    device = torch.device("cuda", rank % torch.cuda.device_count()) if on_gpu else torch.device("cpu")
    dtype = getattr(torch, spec.get("dtype", "bfloat16")) if on_gpu else torch.float32
    weights = None
    if spec.get("model_path"):
        from parallax_b200.loader.shard_loader import ShardLoader

        weights = ShardLoader(spec["model_path"], spec["start_layer"], spec["end_layer"]).load_weights("cpu", None)
    keys = ("page_size", "num_blocks", "kv_fraction", "max_batch_size", "max_num_tokens_per_batch", "max_total_length",
            "seed", "kv_cache_dtype", "lora")
    return TPStageGroup(cfg, spec["start_layer"], spec["end_layer"], device, dtype, weights=weights,
                        **{k: spec[k] for k in keys if spec.get(k) is not None})


def launch_followers(spec: dict, tp: int) -> tuple[TPStageGroup, list]:
    """Rank 0 (the node process): start ranks 1..tp-1, form the process group, build the stage everywhere."""
    from parallax_b200.parallel.launcher import free_port, init_process_group

    port = free_port()
    procs = []
    for r in range(1, tp):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(tp), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-m", "parallax_b200.parallel.peer_group", json.dumps(spec)], env=env))
    os.environ.update(RANK="0", WORLD_SIZE=str(tp), LOCAL_RANK="0")
    init_process_group(0, tp, port, spec.get("device_type", "cuda"))
    return build_group(spec), procs


def stop_followers(group: TPStageGroup, procs: list, timeout_s: float = 20.0) -> None:
    group.shutdown()
    for p in procs:
        try:
            p.wait(timeout_s)
        except subprocess.TimeoutExpired:
            p.terminate()
    if dist.is_initialized():
        dist.destroy_process_group()


def follower_main() -> None:
    from parallax_b200.parallel.launcher import init_process_group

    spec = json.loads(sys.argv[1])
    logging.basicConfig(level=spec.get("log_level", "INFO"))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    init_process_group(rank, world, int(os.environ["MASTER_PORT"]), spec.get("device_type", "cuda"))
    group = build_group(spec)

    def on_command(name: str, payload) -> None:
        if name == "refit":
            from parallax_b200.utils.weight_refit import apply_refit_to_stage

            apply_refit_to_stage(group.worker, cfg=group.cfg, refit=payload)
        elif name == "lora_load":
            from parallax_b200.loader.lora import LoRAAdapter

            slot, adapter, path = payload
            group.worker.model.lora.load(int(slot), LoRAAdapter.load(path, adapter))

    group.on_command = on_command
    try:
        group.serve_forever()
    finally:
        group.chan.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    follower_main()
