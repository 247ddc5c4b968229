"""`python -m xllm_b200.launch_server --model <dir> --nproc N [server flags]` — start one server rank
per GPU of this node.

Counterpart of the reference's launcher (xllm/launch_server.py:35-80: one `xllm` process per rank with
`--nnodes/--node_rank/--master_node_addr`, per-rank log files, the job goes down as a whole).  Here
every rank is `python -m xllm_b200.serve`; rank 0 hosts the HTTP port and mirrors requests to the
others.  With `--pd` the ranks are split into a prefill instance and a decode instance
(`--pd-prefill-ranks K`: the first K ranks prefill, the rest decode); the two are linked through the
servers' `/link_p2p` route once both answer `/health`.

The launcher owns the children: a rank that exits takes the job down (the others get SIGTERM, then
SIGKILL after a grace period), SIGINT / SIGTERM are forwarded, the exit code is that of the first rank
that failed.
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time
from dataclasses import dataclass
from typing import List, Optional, TextIO


@dataclass
class RankProcess:
    rank: int
    proc: subprocess.Popen
    log: Optional[TextIO]


def build_commands(nproc: int, server_args: List[str], master_addr: str, master_port: int, python: str = sys.executable):
    """[(rank, argv, env additions)] of the `nproc` server ranks."""
    out = []
    for r in range(nproc):
        argv = [python, "-m", "xllm_b200.serve", *server_args]
        if nproc > 1:
            argv += [f"--nnodes={nproc}", f"--node_rank={r}", f"--master_node_addr={master_addr}:{master_port}"]
        env = {"RANK": str(r), "LOCAL_RANK": str(r), "WORLD_SIZE": str(nproc), "MASTER_ADDR": master_addr,
               "MASTER_PORT": str(master_port)}
        out.append((r, argv, env))
    return out


def launch(nproc: int, server_args: List[str], master_addr="127.0.0.1", master_port=19888, log_dir: str = "",
           grace_seconds: float = 10.0, poll_seconds: float = 0.2, env=None) -> int:
    procs: List[RankProcess] = []
    base_env = dict(os.environ if env is None else env)
    for r, argv, extra in build_commands(nproc, server_args, master_addr, master_port):
        log = open(os.path.join(log_dir, f"rank{r}.log"), "w") if log_dir else None
        p = subprocess.Popen(argv, env=dict(base_env, **extra), stdout=log or None, stderr=subprocess.STDOUT if log else None)
        procs.append(RankProcess(r, p, log))
    stopping = {"sig": None}

    def forward(signum, _frame):
        stopping["sig"] = signum
        for rp in procs:
            if rp.proc.poll() is None:
                try:
                    rp.proc.send_signal(signum)
                except OSError:
                    pass

    old = {s: signal.signal(s, forward) for s in (signal.SIGINT, signal.SIGTERM)}
    code = 0
    try:
        while True:
            done = [rp for rp in procs if rp.proc.poll() is not None]
            if done:
                first = done[0]
                code = first.proc.returncode if stopping["sig"] is None else 0
                break
            time.sleep(poll_seconds)
        # one rank is gone: the job cannot go on without it
        for rp in procs:
            if rp.proc.poll() is None:
                rp.proc.terminate()
        deadline = time.time() + grace_seconds
        for rp in procs:
            try:
                rp.proc.wait(timeout=max(0.0, deadline - time.time()))
            except subprocess.TimeoutExpired:
                rp.proc.kill()                      # this exact child, nothing else
                rp.proc.wait()
    finally:
        for s, h in old.items():
            signal.signal(s, h)
        for rp in procs:
            if rp.log:
                rp.log.close()
    return code if code is not None else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="start one xllm_b200 server rank per GPU", allow_abbrev=False)
    ap.add_argument("--nproc", type=int, default=0, help="ranks to start (default: the visible GPUs, at least 1)")
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=19888)
    ap.add_argument("--log-dir", default="", help="write rank<N>.log files here instead of sharing the terminal")
    args, server_args = ap.parse_known_args(argv)
    n = args.nproc
    if n <= 0:
        try:
            import torch
            n = max(1, torch.cuda.device_count())
        except Exception:
            n = 1
    if args.log_dir:
        os.makedirs(args.log_dir, exist_ok=True)
    return launch(n, server_args, args.master_addr, args.master_port, args.log_dir)


if __name__ == "__main__":
    sys.exit(main())
