"""Adapter preparation: bring a LoRA adapter directory into one normal form that this framework, PEFT and the
reference's own (MLX) backend can all read.

The reference ships a converter that completes a PEFT ``adapter_config.json`` with the fields its MLX loader wants
(``fine_tune_type``, ``num_layers``, ``lora_parameters = {rank, scale, dropout}``) and gathers the weights into a
single fp16 file (``src/parallax_utils/prepare_adapter.py:13-83,151-164``). Here the same preparation is a function
and a small command:

    python -m parallax_b200.utils.prepare_adapter <adapter dir> [--base <model dir>] [--out <dir>] [--layout peft|mlx]

It reads either layout (PEFT ``adapter_model.safetensors`` with ``lora_A [r, in]`` / ``lora_B [out, r]``, or the
single-file ``adapters.safetensors`` with ``lora_a [in, r]`` / ``lora_b [r, out]``) and writes the requested one
together with a config that carries both sets of fields, so the result loads everywhere.
"""

from __future__ import annotations

import argparse
import json
import re
from pathlib import Path
from typing import Optional

_PEFT = re.compile(r"^(?P<prefix>(?:base_model\.model\.)?)(?P<mod>.*)\.lora_(?P<ab>[AB])(?:\.default)?\.weight$")
_MLX = re.compile(r"^(?P<mod>.*)\.lora_(?P<ab>[ab])$")


def complete_adapter_config(cfg: dict, num_layers: Optional[int] = None) -> dict:
    """The config with the fields of both layouts filled in from whichever are present."""
    out = dict(cfg)
    lp = dict(out.get("lora_parameters") or {})
    rank = int(out.get("r") or lp.get("rank") or 8)
    if "lora_alpha" in out:
        alpha = float(out["lora_alpha"])
    elif "scale" in lp:
        alpha = float(lp["scale"]) * rank
    else:
        alpha = float(rank)
    out.setdefault("peft_type", "LORA")
    out.setdefault("fine_tune_type", str(out["peft_type"]).lower())
    out["r"] = rank
    out["lora_alpha"] = alpha
    if num_layers is not None:
        out.setdefault("num_layers", int(num_layers))
    lp.setdefault("rank", rank)
    lp.setdefault("scale", alpha / rank)          # the multiplier itself, which is how this layout applies it
    lp.setdefault("dropout", float(out.get("lora_dropout", 0.0)))
    out["lora_parameters"] = lp
    return out


def read_adapter_tensors(src: Path) -> tuple[dict, str]:
    """``({module path: {"A": [r, in], "B": [out, r]}}, layout found)``."""
    from safetensors.torch import load_file

    peft, mlx = src / "adapter_model.safetensors", src / "adapters.safetensors"
    mods: dict = {}
    if peft.exists():
        for k, v in load_file(str(peft)).items():
            m = _PEFT.match(k)
            if m:
                mods.setdefault(m.group("mod"), {})[m.group("ab")] = v
        return mods, "peft"
    if mlx.exists():
        for k, v in load_file(str(mlx)).items():
            m = _MLX.match(k)
            if m:
                mods.setdefault(m.group("mod"), {})[m.group("ab").upper()] = v.t().contiguous()
        return mods, "mlx"
    raise FileNotFoundError(f"{src}: neither adapter_model.safetensors nor adapters.safetensors")


def prepare_adapter(src: str, out: Optional[str] = None, base: Optional[str] = None, layout: str = "peft",
                    dtype: str = "float16") -> Path:
    """Write the adapter at ``src`` to ``out`` (default: in place) in ``layout`` with a completed config.
    ``base``: the base model's directory, for ``num_layers`` (read from its ``config.json``)."""
    import torch
    from safetensors.torch import save_file

    src_p = Path(src)
    out_p = Path(out) if out else src_p
    out_p.mkdir(parents=True, exist_ok=True)
    cfg_file = src_p / "adapter_config.json"
    if not cfg_file.exists():
        raise FileNotFoundError(f"adapter_config.json not found at: {cfg_file}")
    cfg = json.loads(cfg_file.read_text())
    num_layers = cfg.get("num_layers")
    if num_layers is None and base:
        mc = json.loads((Path(base) / "config.json").read_text())
        mc = mc.get("text_config", mc)
        if "num_hidden_layers" not in mc:
            raise ValueError("config.json is missing the 'num_hidden_layers' field")
        num_layers = mc["num_hidden_layers"]
    mods, found = read_adapter_tensors(src_p)
    if num_layers is None:
        layers = [int(m.group(1)) for k in mods if (m := re.search(r"layers\.(\d+)\.", k))]
        num_layers = max(layers) + 1 if layers else None
    cfg = complete_adapter_config(cfg, num_layers)
    td = getattr(torch, dtype)
    tensors = {}
    for mod, ab in mods.items():
        if "A" not in ab or "B" not in ab:
            continue
        if layout == "mlx":
            name = mod[len("model."):] if mod.startswith("model.model.") else mod
            tensors[f"{name}.lora_a"] = ab["A"].t().contiguous().to(td)
            tensors[f"{name}.lora_b"] = ab["B"].t().contiguous().to(td)
        else:
            tensors[f"base_model.model.{mod}.lora_A.weight"] = ab["A"].contiguous().to(td)
            tensors[f"base_model.model.{mod}.lora_B.weight"] = ab["B"].contiguous().to(td)
    name = "adapters.safetensors" if layout == "mlx" else "adapter_model.safetensors"
    save_file(tensors, str(out_p / name), metadata={"format": "mlx" if layout == "mlx" else "pt"})
    (out_p / "adapter_config.json").write_text(json.dumps(cfg, indent=2))
    return out_p


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="Normalise a LoRA adapter directory")
    ap.add_argument("adapter")
    ap.add_argument("--base", default=None, help="base model directory (for num_layers)")
    ap.add_argument("--out", default=None)
    ap.add_argument("--layout", choices=["peft", "mlx"], default="peft")
    ap.add_argument("--dtype", default="float16")
    a = ap.parse_args(argv)
    print(f"adapter written to {prepare_adapter(a.adapter, a.out, a.base, a.layout, a.dtype)}")


if __name__ == "__main__":
    main()
