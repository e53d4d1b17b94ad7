#!/usr/bin/env python3
"""Launch ``LOCAL_SIZE`` ranks per host under mpiexec (or a single host without it).

    mpiexec -x LOCAL_SIZE=8 -host a,b python -m planmoe_b200.launcher.run -m planmoe_b200.examples.pre_test

Each mpiexec task (one per host) replaces itself with ``torch.distributed.run`` for that host's
GPUs; every rank is then wrapped by ``planmoe_b200.launcher.execl`` (NUMA binding, optional one-GPU
sandbox).  Counterpart of ``PlanMoE/launcher/run.py:6-38``.
"""

import os
import sys


def build_command(argv, env):
    host_size = int(env.get('OMPI_COMM_WORLD_SIZE', 1))
    host_rank = int(env.get('OMPI_COMM_WORLD_RANK', 0))
    local_size = int(env.get('LOCAL_SIZE', 1))
    master_addr = env.get('MASTER_ADDR', '127.0.0.1') if host_size > 1 else '127.0.0.1'
    master_port = int(env.get('MASTER_PORT', 23232))
    new_env = dict(env)
    if host_size * local_size >= 512 and 'TUTEL_ALLTOALL_ALGO' not in env:
        new_env['TUTEL_ALLTOALL_ALGO'] = '2D'
    new_env.setdefault('OMP_NUM_THREADS', str(max(1, (os.cpu_count() or 1) // max(local_size, 1))))
    new_env['LOCAL_SIZE'] = str(local_size)
    skip = 1 if (argv and argv[0] == '-m') else 0
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nproc_per_node=%d' % local_size,
           '--nnodes=%d' % host_size, '--node_rank=%d' % host_rank, '--master_addr=%s' % master_addr,
           '--master_port=%d' % master_port, '-m', 'planmoe_b200.launcher.execl']
    if not skip:
        cmd.append(sys.executable)
    else:
        cmd += [sys.executable, '-m']
    return cmd + list(argv[skip:]), new_env


def main():
    cmd, env = build_command(sys.argv[1:], os.environ)
    os.execve(cmd[0], cmd, env)


if __name__ == '__main__':
    main()
