"""``parallax`` command line: ``serve``, ``run``, ``join``, ``chat``.

Same sub-commands and flags as the reference CLI (``src/parallax/cli.py:372-470``): unknown
flags are passed through to the launched module, and the child runs in its own process group
so that Ctrl-C can escalate SIGINT -> SIGTERM -> SIGKILL over the whole tree (``:93-163``).
The reference's version-telemetry upload is not implemented; ``-u/--skip-upload`` is accepted
and has no effect.

  parallax serve -m Qwen/Qwen3-8B                 standalone server on this box
  parallax run -m Qwen/Qwen3-8B -n 2              cluster scheduler + REST backend (port 3001)
  parallax join -s 10.0.0.5:3001                  join a cluster as a worker node
  parallax chat -s 10.0.0.5:3001                  local chat endpoint that forwards to a cluster
"""

from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
from typing import Optional, Sequence

DEFAULT_SCHEDULER_PORT = 3001


def _flag_present(args: Sequence[str], names: Sequence[str]) -> bool:
    return any(a == n or a.startswith(n + "=") for a in args for n in names)


def _signal_group(proc: subprocess.Popen, sig: int) -> None:
    try:
        os.killpg(proc.pid, sig)
    except Exception:
        try:
            proc.send_signal(sig)
        except Exception:
            pass


def _execute_with_graceful_shutdown(cmd: list[str], env: Optional[dict] = None) -> None:
    proc = None
    try:
        proc = subprocess.Popen(cmd, env=env, start_new_session=True)
        rc = proc.wait()
        if rc != 0:
            sys.exit(rc)
    except KeyboardInterrupt:
        if proc is None:
            sys.exit(0)

        def force(_signum, _frame):
            _signal_group(proc, signal.SIGKILL)
            os._exit(130)

        try:
            signal.signal(signal.SIGINT, force)  # a second Ctrl-C kills immediately
        except Exception:
            pass
        for sig in (signal.SIGINT, signal.SIGTERM):
            _signal_group(proc, sig)
            try:
                proc.wait(timeout=5)
                break
            except subprocess.TimeoutExpired:
                continue
        else:
            _signal_group(proc, signal.SIGKILL)
            proc.wait()
        sys.exit(0)


def _module_cmd(module: str) -> list[str]:
    return [sys.executable, "-m", module]


def _normalise_scheduler_addr(addr: str) -> str:
    if addr == "auto":
        return f"127.0.0.1:{DEFAULT_SCHEDULER_PORT}"
    return addr


def serve_command(args, passthrough: Optional[list[str]] = None) -> None:
    cmd = _module_cmd("parallax_b200.launch") + ["--model-path", args.model_path] + list(passthrough or [])
    _execute_with_graceful_shutdown(cmd, env=os.environ.copy())


def run_command(args, passthrough: Optional[list[str]] = None) -> None:
    passthrough = list(passthrough or [])
    cmd = _module_cmd("parallax_b200.backend.app")
    if not _flag_present(passthrough, ["--port"]):
        cmd += ["--port", str(DEFAULT_SCHEDULER_PORT)]
    if args.model_name:
        cmd += ["--model-name", args.model_name]
    if args.init_nodes_num:
        cmd += ["--init-nodes-num", str(args.init_nodes_num)]
    if args.use_relay:
        print("note: relay servers are not needed for in-rack clusters; --use-relay is ignored", file=sys.stderr)
    _execute_with_graceful_shutdown(cmd + passthrough)


def join_command(args, passthrough: Optional[list[str]] = None) -> None:
    cmd = _module_cmd("parallax_b200.launch") + ["--scheduler-addr", _normalise_scheduler_addr(args.scheduler_addr)]
    _execute_with_graceful_shutdown(cmd + list(passthrough or []), env=os.environ.copy())


def chat_command(args, passthrough: Optional[list[str]] = None) -> None:
    cmd = _module_cmd("parallax_b200.launch_chat") + ["--scheduler-addr", _normalise_scheduler_addr(args.scheduler_addr)]
    _execute_with_graceful_shutdown(cmd + list(passthrough or []))


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="parallax", description="parallax_b200 - pipeline-parallel LLM serving on B200",
                                formatter_class=argparse.RawDescriptionHelpFormatter, epilog=__doc__)
    sub = p.add_subparsers(dest="command", help="Available commands")
    s = sub.add_parser("serve", help="Start a standalone server by launching the model locally")
    s.add_argument("-m", "--model-path", required=True, type=str, help="Path to the model repository or model name")
    s.add_argument("-u", "--skip-upload", action="store_true", help="Accepted for compatibility")
    r = sub.add_parser("run", help="Start the cluster scheduler and its REST backend")
    r.add_argument("-n", "--init-nodes-num", type=int, help="Number of initial nodes")
    r.add_argument("-m", "--model-name", type=str, help="Model name")
    r.add_argument("-r", "--use-relay", action="store_true", help="Accepted for compatibility")
    r.add_argument("-u", "--skip-upload", action="store_true", help="Accepted for compatibility")
    j = sub.add_parser("join", help="Join a cluster as a worker node")
    j.add_argument("-s", "--scheduler-addr", default="auto", type=str, help="Scheduler address host:port")
    j.add_argument("-r", "--use-relay", action="store_true", help="Accepted for compatibility")
    j.add_argument("-u", "--skip-upload", action="store_true", help="Accepted for compatibility")
    c = sub.add_parser("chat", help="Start a local chat endpoint that forwards to a cluster")
    c.add_argument("-s", "--scheduler-addr", default="auto", type=str, help="Scheduler address host:port")
    c.add_argument("-r", "--use-relay", action="store_true", help="Accepted for compatibility")
    return p


def main(argv: Optional[Sequence[str]] = None) -> None:
    parser = build_parser()
    args, passthrough = parser.parse_known_args(argv)
    handlers = {"run": run_command, "serve": serve_command, "join": join_command, "chat": chat_command}
    if args.command not in handlers:
        parser.print_help()
        sys.exit(1)
    handlers[args.command](args, passthrough)


if __name__ == "__main__":
    main()
