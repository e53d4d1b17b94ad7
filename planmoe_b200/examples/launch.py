#!/usr/bin/env python3
"""Map an OpenMPI task to torch.distributed rank variables and exec the given command
(one MPI task per GPU; counterpart of ``PlanMoE/examples/launch.py:5-25``)."""

import os
import sys


def main():
    env = dict(os.environ)
    env['RANK'] = env.get('OMPI_COMM_WORLD_RANK', env.get('RANK', '0'))
    env['WORLD_SIZE'] = env.get('OMPI_COMM_WORLD_SIZE', env.get('WORLD_SIZE', '1'))
    env['LOCAL_RANK'] = env.get('OMPI_COMM_WORLD_LOCAL_RANK', env.get('LOCAL_RANK', '0'))
    env.setdefault('LOCAL_SIZE', env.get('OMPI_COMM_WORLD_LOCAL_SIZE', '1'))
    env.setdefault('MASTER_ADDR', '127.0.0.1')
    env.setdefault('MASTER_PORT', '23232')
    if len(sys.argv) < 2:
        raise SystemExit('usage: launch.py <command> [args...]')
    os.execvpe(sys.argv[1], sys.argv[1:], env)


if __name__ == '__main__':
    main()
