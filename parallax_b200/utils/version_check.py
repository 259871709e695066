"""Installed version and the "a newer release exists" notice.

The reference asks the project's release feed once at start-up of ``run`` and ``join`` and prints an update hint when
the newest tag differs from the installed version; any network problem is silent
(``src/parallax_utils/version_check.py:6-42``). Same behaviour here, with the feed URL taken from
``PARALLAX_RELEASE_FEED`` (unset or empty: no request is made, which is the right default for air-gapped GPU boxes)
and a short timeout.
"""

from __future__ import annotations

import json
import os
import urllib.request
from typing import Callable, Optional


def get_current_version() -> str:
    try:
        import importlib.metadata

        return importlib.metadata.version("parallax_b200")
    except Exception:
        try:
            import parallax_b200

            return getattr(parallax_b200, "__version__", "unknown")
        except Exception:
            return "unknown"


def _as_tuple(v: str):
    parts = []
    for p in v.lstrip("vV").split("."):
        digits = "".join(ch for ch in p if ch.isdigit())
        parts.append(int(digits) if digits else 0)
    return tuple(parts)


def check_latest_release(feed_url: Optional[str] = None, timeout_s: float = 4.0,
                         out: Callable[[str], None] = print) -> Optional[str]:
    """Returns the newer version's tag (after printing the notice) or None. Never raises."""
    url = feed_url if feed_url is not None else os.environ.get("PARALLAX_RELEASE_FEED", "")
    if not url:
        return None
    try:
        with urllib.request.urlopen(url, timeout=timeout_s) as resp:
            data = json.loads(resp.read())
        latest = str(data.get("tag_name") or data.get("name") or "").lstrip("vV")
        current = get_current_version().lstrip("vV")
        if latest and current != "unknown" and _as_tuple(latest) > _as_tuple(current):
            out(f"\033[93m[parallax_b200] new version available: {latest} (installed: {current}); "
                f"update the checkout and rebuild the kernels (`python -c 'import __graft_entry__ as g; g.build()'`)\033[0m")
            return latest
    except Exception:
        pass
    return None
