"""Per-request serving metrics derived from the final SSE chunk (the one carrying ``usage``)."""

from __future__ import annotations

import json


def get_request_metrics(chunk, start_time, first_token_time, last_token_time):
    """(tokens/s, TTFT ms, prompt tokens, completion tokens) or four Nones if unavailable."""
    try:
        if isinstance(chunk, bytes):
            chunk = chunk.decode("utf-8")
        if isinstance(chunk, str):
            # a network chunk may hold several SSE events: take the last data line with usage
            payloads = [l[5:].strip() for l in chunk.splitlines() if l.startswith("data:")]
            payloads = [p for p in payloads if p and p != "[DONE]"]
            chunk = json.loads(payloads[-1] if payloads else chunk)
        usage = chunk["usage"]
        n_in, n_out = usage["prompt_tokens"], usage["completion_tokens"]
        span = last_token_time - first_token_time
        tps = n_out / span if span > 0 else float(n_out)
        return tps, int((first_token_time - start_time) * 1000), n_in, n_out
    except Exception:
        return None, None, None, None
