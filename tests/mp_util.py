"""Launch ``world`` child processes that each run one function of tests/mp_worker.py as a rank of a
torch.distributed world (rendezvous on 127.0.0.1).  Raises with the children's output on failure."""

import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def run_workers(fn, world, backend='gloo', timeout=180, env=None, args=()):
    """Run the workers; a failed attempt is repeated, up to twice, on a fresh port after a short pause (a rendezvous
    on a shared host can lose its port between the probe and the bind), and only a third failure fails the test."""
    import time
    failures = []
    for attempt in range(3):
        try:
            return _run_workers_once(fn, world, backend, timeout, env, args)
        except AssertionError as exc:
            failures.append(str(exc))
            time.sleep(1.0 + attempt)
    raise AssertionError('\n==== earlier attempt ====\n'.join(reversed(failures)))


def _run_workers_once(fn, world, backend, timeout, env, args):
    port = _free_port()
    procs = []
    for rank in range(world):
        e = dict(os.environ)
        e.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR='127.0.0.1',
                 MASTER_PORT=str(port), MP_BACKEND=backend, OMP_NUM_THREADS='2')
        e.setdefault('PLANMOE_WAIT_BUDGET_MS', '5000')
        if env:
            e.update({k: str(v) for k, v in env.items()})
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, 'mp_worker.py'), fn] + [str(a) for a in args],
                                      env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs, bad = [], False
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            bad = True
        outs.append(out)
        bad = bad or p.returncode != 0
    if bad:
        raise AssertionError('worker `%s` failed:\n%s' % (fn, '\n----\n'.join(o[-3000:] for o in outs)))
    return outs
