"""Start-up banners of ``parallax run`` and ``parallax join``.

The reference plays a coloured ASCII animation from JSON frame files when the scheduler starts and when a node has
joined with its model (``src/parallax_utils/ascii_anime.py:130-227``). Here it is one drawn frame: a stage diagram
that says what the process is (scheduler, or a node serving a layer range of a model), printed only to a terminal
and never into logs or pipes.
"""

from __future__ import annotations

import os
import sys
from typing import Optional

_C = {"dim": "\033[2m", "b": "\033[1m", "g": "\033[38;5;114m", "y": "\033[38;5;221m", "c": "\033[38;5;80m", "x": "\033[0m"}


def _paint(text: str, colour: bool) -> str:
    for k, v in _C.items():
        text = text.replace("{" + k + "}", v if colour else "")
    return text


def _stages(n: int, hot: Optional[int] = None) -> str:
    cells = []
    for i in range(n):
        cells.append(("{y}[#]{x}" if i == hot else "{c}[ ]{x}"))
    return "{dim}--{x}".join(cells)


def render_run(colour: bool = False) -> str:
    lines = ["{b}{g}parallax_b200{x}  scheduler + API gateway",
             "  requests {dim}->{x} " + _stages(4) + " {dim}->{x} tokens",
             "  {dim}nodes join with `parallax join -s <this host>:<port>` and are given a layer range{x}"]
    return _paint("\n".join(lines), colour)


def render_join(model_name: str, start_layer: Optional[int] = None, end_layer: Optional[int] = None,
                num_layers: Optional[int] = None, colour: bool = False) -> str:
    where = ""
    hot = None
    if start_layer is not None and end_layer is not None:
        where = f"  layers [{start_layer}, {end_layer})" + (f" of {num_layers}" if num_layers else "")
        if num_layers:
            hot = min(3, (start_layer * 4) // max(num_layers, 1))
    lines = ["{b}{g}parallax_b200{x}  node serving {b}" + str(model_name) + "{x}" + where,
             "  requests {dim}->{x} " + _stages(4, hot) + " {dim}->{x} tokens"]
    return _paint("\n".join(lines), colour)


def _tty() -> bool:
    return sys.stdout.isatty() and not os.environ.get("NO_COLOR") and os.environ.get("TERM", "") != "dumb"


def display_parallax_run() -> None:
    if sys.stdout.isatty():
        print(render_run(_tty()))


def display_parallax_join(model_name: str, start_layer: Optional[int] = None, end_layer: Optional[int] = None,
                          num_layers: Optional[int] = None) -> None:
    if sys.stdout.isatty():
        print(render_join(model_name, start_layer, end_layer, num_layers, _tty()))
