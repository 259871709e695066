"""Small utilities: version notice, start-up banners."""

import io
import json

from parallax_b200.utils import banner, version_check


class _Resp(io.BytesIO):
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def test_version_notice(monkeypatch):
    said = []
    monkeypatch.setattr(version_check, "get_current_version", lambda: "0.1.0")
    monkeypatch.setattr(version_check.urllib.request, "urlopen",
                        lambda url, timeout=0: _Resp(json.dumps({"tag_name": "v0.2.0"}).encode()))
    assert version_check.check_latest_release("http://feed", out=said.append) == "0.2.0"
    assert "0.2.0" in said[0] and "0.1.0" in said[0]
    monkeypatch.setattr(version_check.urllib.request, "urlopen",
                        lambda url, timeout=0: _Resp(json.dumps({"tag_name": "v0.1.0"}).encode()))
    assert version_check.check_latest_release("http://feed", out=said.append) is None and len(said) == 1

    def boom(url, timeout=0):
        raise OSError("no network")

    monkeypatch.setattr(version_check.urllib.request, "urlopen", boom)
    assert version_check.check_latest_release("http://feed", out=said.append) is None      # silent
    monkeypatch.delenv("PARALLAX_RELEASE_FEED", raising=False)
    assert version_check.check_latest_release(out=said.append) is None                       # no feed: no request
    assert version_check._as_tuple("v1.10.2") > version_check._as_tuple("1.9.9")
    assert version_check.get_current_version() == "0.1.0"


def test_banners_are_plain_text_off_a_terminal(capsys):
    txt = banner.render_join("Qwen/Qwen3-8B", 18, 36, 36)
    assert "Qwen/Qwen3-8B" in txt and "[18, 36) of 36" in txt and "\033" not in txt and txt.count("[#]") == 1
    assert "\033[" in banner.render_run(colour=True) and "scheduler" in banner.render_run()
    banner.display_parallax_run()                # stdout is captured, not a terminal: nothing is printed
    banner.display_parallax_join("m")
    assert capsys.readouterr().out == ""


def test_nvtx_ranges_are_a_no_op_when_off(monkeypatch):
    from parallax_b200.utils import trace

    monkeypatch.setattr(trace, "_NVTX", None)
    monkeypatch.delenv("PXL_NVTX", raising=False)
    assert not trace.nvtx_enabled()
    with trace.nvtx_range("x") as r:
        assert r is trace._NO_RANGE
    monkeypatch.setattr(trace, "_NVTX", None)
    monkeypatch.setenv("PXL_NVTX", "1")
    import torch

    assert trace.nvtx_enabled() == torch.cuda.is_available()
    monkeypatch.setattr(trace, "_NVTX", None)


def test_offline_generation_reports_prefill_and_decode_steps():
    from parallax_b200.generate import percentile, run

    lines = []
    res = run("tiny", "Hello there", max_tokens=5, random_init=True, device="cpu", out=lines.append)
    assert res["generated_tokens"] == 5 and len(res["decode_ms"]) == 4 and res["prompt_tps"] > 0
    assert any(l.startswith("Prefill:") for l in lines) and any(l.startswith("Decode step time (ms): min=") for l in lines)
    assert percentile([1, 2, 3, 4], 50) == 2.5 and percentile([5], 99) == 5
