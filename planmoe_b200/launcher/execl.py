#!/usr/bin/env python3
"""Per-rank wrapper: optional one-GPU sandbox and NUMA binding, then exec the real command.

``TUTEL_CUDA_SANDBOX=2`` exposes only this rank's GPU (``CUDA_VISIBLE_DEVICES=LOCAL_RANK``, and
``LOCAL_RANK`` then becomes 0 for the program).  When ``numactl`` exists the rank is bound to the
NUMA node ``LOCAL_RANK * nodes / LOCAL_SIZE``.  Counterpart of ``PlanMoE/launcher/execl.py:8-45``.
"""

import os
import re
import shutil
import sys


def numa_nodes(root='/sys/devices/system/node'):
    try:
        return sorted(int(d[4:]) for d in os.listdir(root) if re.match(r'node[0-9]+$', d))
    except OSError:
        return []


def build_command(argv, env):
    env = dict(env)
    local_rank = int(env.get('LOCAL_RANK', 0))
    local_size = int(env.get('LOCAL_SIZE', env.get('LOCAL_WORLD_SIZE', 1)))
    if int(env.get('TUTEL_CUDA_SANDBOX', 0)) == 2:
        env['CUDA_VISIBLE_DEVICES'] = str(local_rank)
        env['TUTEL_CUDA_SANDBOX'] = '1'
    env.setdefault('OMP_NUM_THREADS', '8')
    cmd = list(argv)
    nodes = numa_nodes()
    numactl = shutil.which('numactl')
    if numactl and len(nodes) > 1 and int(env.get('NUMA_TYPE', 1)) > 0:
        node = nodes[(local_rank * len(nodes)) // max(local_size, 1) % len(nodes)]
        cmd = [numactl, '--cpunodebind=%d' % node, '--preferred=%d' % node] + cmd
    return cmd, env


def main():
    if len(sys.argv) < 2:
        raise SystemExit('usage: python -m planmoe_b200.launcher.execl <command> [args...]')
    cmd, env = build_command(sys.argv[1:], os.environ)
    exe = shutil.which(cmd[0]) or cmd[0]
    os.execve(exe, cmd, env)


if __name__ == '__main__':
    main()
