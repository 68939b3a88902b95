"""Run a scheduler + workers job and restart it from its last checkpoint when a process fails.

The reference has no recovery at all (no re-registration, no rank replacement; its
scheduler waits forever, necklace/trainer/tndsnc.py:464-477).  Here the services already turn
any failure into a job-wide abort with non-zero exit codes (``trainer/service.py``); this
supervisor is the other half: it starts the processes, and if one ends with an error it
stops exactly the processes it started, and starts the job again with ``resume_args``
appended (the scripts then continue from ``trainer.resume``'s newest common checkpoint).

    python -m necklace_b200.utils.supervise --restarts 2 --resume-arg=--resume \\
        -- python train.py -r scheduler ... ++ python train.py -r worker -k 0 ... ++ ...
"""
from __future__ import annotations

import argparse
import subprocess
import sys
import time


def _stop(procs, grace=5.0):
    for p in procs:
        if p.poll() is None:
            p.terminate()
    t_end = time.time() + grace
    for p in procs:
        try:
            p.wait(timeout=max(0.1, t_end - time.time()))
        except subprocess.TimeoutExpired:
            p.kill()
            p.wait()


def run_job(cmds, max_restarts=1, resume_args=("--resume",), timeout=None, poll=0.2,
            popen_kwargs=None, log=None):
    """``cmds``: one argv list per process.  Returns ``(exit_codes, restarts)`` of the last
    attempt; all zero means the job finished."""
    log = log or (lambda *a: None)
    attempt, extra = 0, []
    while True:
        kw = popen_kwargs(attempt) if callable(popen_kwargs) else (popen_kwargs or {})
        procs = [subprocess.Popen(list(c) + extra, **(kw[i] if isinstance(kw, list) else kw))
                 for i, c in enumerate(cmds)]
        t0, failed = time.time(), False
        while True:
            codes = [p.poll() for p in procs]
            if any(c not in (None, 0) for c in codes):
                failed = True
                break
            if all(c == 0 for c in codes):
                break
            if timeout is not None and time.time() - t0 > timeout:
                failed = True
                log(f"attempt {attempt}: timed out after {timeout}s")
                break
            time.sleep(poll)
        if not failed:
            return [p.returncode for p in procs], attempt
        # the services abort everyone once one process failed; give them a moment, then stop
        # what is left (only the processes started above)
        t_end = time.time() + 10.0
        while time.time() < t_end and any(p.poll() is None for p in procs):
            time.sleep(poll)
        _stop(procs)
        codes = [p.returncode for p in procs]
        log(f"attempt {attempt}: exit codes {codes}")
        if attempt >= max_restarts:
            return codes, attempt
        attempt += 1
        extra = list(resume_args)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--restarts", type=int, default=1)
    ap.add_argument("--resume-arg", action="append", default=None)
    ap.add_argument("--timeout", type=float, default=None)
    ap.add_argument("cmds", nargs=argparse.REMAINDER,
                    help="-- cmd args ++ cmd args ++ ... (one process per ++-separated part)")
    args = ap.parse_args(argv)
    words = args.cmds[1:] if args.cmds[:1] == ["--"] else args.cmds
    cmds, cur = [], []
    for w in words:
        if w == "++":
            cmds.append(cur)
            cur = []
        else:
            cur.append(w)
    if cur:
        cmds.append(cur)
    if not cmds:
        ap.error("no commands")
    codes, restarts = run_job(cmds, args.restarts, tuple(args.resume_arg or ["--resume"]),
                              args.timeout, log=lambda *a: print("[supervise]", *a, flush=True))
    print(f"[supervise] exit codes {codes} after {restarts} restart(s)", flush=True)
    return 0 if all(c == 0 for c in codes) else 1


if __name__ == "__main__":
    sys.exit(main())
