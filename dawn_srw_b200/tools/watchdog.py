#!/usr/bin/env python
"""Liveness check of a training run from its per-rank heartbeat files.

    python -m dawn_srw_b200.tools.watchdog RUN_DIR [--max-age 300] [--watch SECONDS]

Exit code 0: every rank refreshed its heartbeat within ``--max-age`` seconds;
3: at least one rank is stale or missing (a hung collective, a crashed
process).  With ``--watch`` it polls at that period until that happens.  Meant
for a supervisor that restarts the job from the newest checkpoint (training
resumes automatically from the newest run folder).
"""
from __future__ import annotations

import argparse
import json
import sys
import time

from ..train.logging import stale_ranks


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("run_dir")
    ap.add_argument("--max-age", type=float, default=300.0)
    ap.add_argument("--watch", type=float, default=0.0)
    args = ap.parse_args(argv)
    while True:
        rep = stale_ranks(args.run_dir, args.max_age)
        bad = bool(rep["stale"] or rep["missing"] or rep["world"] == 0)
        if bad or args.watch <= 0:
            print(json.dumps(rep))
            return 3 if bad else 0
        time.sleep(args.watch)


if __name__ == "__main__":
    sys.exit(main())
