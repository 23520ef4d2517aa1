#!/usr/bin/env python
"""One-command launcher for a training run on one multi-GPU box.

    python -m dawn_srw_b200.tools.launch --config configs/dawn_v4_0_1_400M.yaml
        [--gpus N] [--from-scratch] [--detach] [--log FILE] [--master-port P]
        [--stop] [--status] [--dry-run] [-- <extra arguments for tools.train>]

What it does, in order (the reference does the equivalent for a TPU pod with
two shell scripts that ssh into every worker, install the dependencies, sync
the repository and start ``train_jax.py`` in a tmux session:
scripts/launch_tpu_pod.sh:1-123, scripts/setup_and_run_tpu_pod.sh:33-87):

1. checks the box: counts the visible GPUs, builds / loads the CUDA extension
   once in this process so that the ranks do not race on the build;
2. refuses to start while the run recorded in the PID file is still alive
   (``--stop`` ends that run: SIGTERM to its process group, which the trainer
   turns into a cooperative emergency checkpoint);
3. starts one rank per GPU with ``torch.distributed.run`` on 127.0.0.1 and hands
   ``--config`` / ``--from-scratch`` and everything after ``--`` to
   ``dawn_srw_b200.tools.train`` (which resumes from the newest checkpoint unless
   told otherwise);
4. with ``--detach`` the job runs in its own session, detached from this
   terminal (it survives a closed ssh connection like the reference's tmux
   session), output goes to ``--log`` and the PID to ``<log>.pid``.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
from typing import List, Optional


def visible_gpus() -> int:
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def build_command(config: str, gpus: int, master_port: int, from_scratch: bool,
                  extra: List[str]) -> List[str]:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={max(gpus, 1)}", "--master-addr", "127.0.0.1",
           "--master-port", str(master_port), "-m", "dawn_srw_b200.tools.train",
           "--config", config]
    if from_scratch:
        cmd.append("--from-scratch")
    return cmd + list(extra)


def _read_pid(pid_file: str) -> Optional[int]:
    try:
        return int(open(pid_file).read().split()[0])
    except Exception:
        return None


def _alive(pid: Optional[int]) -> bool:
    if not pid:
        return False
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    # a zombie child of this very process still answers signal 0
    try:
        done, _ = os.waitpid(pid, os.WNOHANG)
        return done == 0
    except ChildProcessError:
        return True


def stop_run(pid_file: str, grace_s: float = 60.0) -> bool:
    """SIGTERM to the recorded run's process group (the trainer reacts with an
    emergency checkpoint), SIGKILL after ``grace_s``.  Only the PID written by
    this launcher is touched."""
    pid = _read_pid(pid_file)
    if not _alive(pid):
        return False
    try:
        os.killpg(pid, signal.SIGTERM)
    except ProcessLookupError:
        return False
    t0 = time.time()
    while time.time() - t0 < grace_s:
        if not _alive(pid):
            return True
        time.sleep(0.5)
    try:
        os.killpg(pid, signal.SIGKILL)
    except ProcessLookupError:
        pass
    return True


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    extra: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, extra = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config")
    ap.add_argument("--gpus", type=int, default=0, help="ranks to start (default: every visible GPU)")
    ap.add_argument("--from-scratch", action="store_true", help="ignore existing checkpoints")
    ap.add_argument("--detach", action="store_true", help="run in the background, detached from this terminal")
    ap.add_argument("--log", default="train.log")
    ap.add_argument("--master-port", type=int, default=29500)
    ap.add_argument("--stop", action="store_true", help="end the run recorded in <log>.pid")
    ap.add_argument("--status", action="store_true", help="say whether that run is alive")
    ap.add_argument("--dry-run", action="store_true", help="print the command and exit")
    ap.add_argument("--no-build", action="store_true", help="skip the extension build / load check")
    args = ap.parse_args(argv)
    pid_file = args.log + ".pid"

    if args.status:
        pid = _read_pid(pid_file)
        print(json.dumps({"pid": pid, "alive": _alive(pid), "log": args.log}))
        return 0
    if args.stop:
        print(json.dumps({"stopped": stop_run(pid_file)}))
        return 0
    if not args.config:
        ap.error("--config is required")
    if not os.path.exists(args.config) and "://" not in args.config:
        ap.error(f"config {args.config} does not exist")

    n_vis = visible_gpus()
    gpus = args.gpus or n_vis or 1
    if n_vis and gpus > n_vis:
        ap.error(f"--gpus {gpus} but only {n_vis} GPUs are visible")
    cmd = build_command(args.config, gpus, args.master_port, args.from_scratch, extra)
    if args.dry_run:
        print(" ".join(cmd))
        return 0
    if _alive(_read_pid(pid_file)):
        print(f"a run started from here is still alive (PID {_read_pid(pid_file)}, {pid_file}); "
              "use --stop first", file=sys.stderr)
        return 2
    if n_vis and not args.no_build:
        from ..ops import build as B
        B.build()
        B.load()
    print("============================================")
    print("Launching DAWN-SRW training")
    print(f"  GPUs:    {gpus} (visible: {n_vis})")
    print(f"  Config:  {args.config}")
    print(f"  Args:    {'--from-scratch ' if args.from_scratch else ''}{' '.join(extra)}")
    print(f"  Log:     {args.log if args.detach else '(this terminal)'}")
    print("============================================", flush=True)
    env = dict(os.environ)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    if not args.detach:
        proc = subprocess.Popen(cmd, env=env, start_new_session=True)
        open(pid_file, "w").write(f"{proc.pid}\n")
        try:
            rc = proc.wait()
        except KeyboardInterrupt:
            os.killpg(proc.pid, signal.SIGTERM)      # cooperative emergency checkpoint
            rc = proc.wait()
        finally:
            try:
                os.remove(pid_file)
            except OSError:
                pass
        return rc
    logf = open(args.log, "ab")
    proc = subprocess.Popen(cmd, env=env, stdout=logf, stderr=subprocess.STDOUT,
                            stdin=subprocess.DEVNULL, start_new_session=True)
    open(pid_file, "w").write(f"{proc.pid}\n")
    print(f"  started PID {proc.pid} (its own session); follow it with: tail -f {args.log}")
    print(f"  stop it with: python -m dawn_srw_b200.tools.launch --log {args.log} --stop")
    return 0


if __name__ == "__main__":
    sys.exit(main())
