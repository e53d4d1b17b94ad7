"""Facade: process-level helpers (reference ``PlanMoE/system.py:8-78``): NUMA affinity,
data/model-parallel session set-up, a process-wide cache and a synchronising timer."""

import atexit
import logging
import os
import re
import sys
import time

TUTEL_CUDA_SANDBOX = int(os.environ.get('TUTEL_CUDA_SANDBOX', 0))


def _numa_cpu_sets(root='/sys/devices/system/node'):
    nodes = sorted(int(d[4:]) for d in os.listdir(root) if re.match(r'node[0-9]+$', d))
    return [sorted(int(c[3:]) for c in os.listdir('%s/node%d' % (root, n))
                   if re.match(r'cpu[0-9]+$', c)) for n in nodes]


def init_affinity_at_program_beginning():
    """Pin this process to the NUMA node chosen by LOCAL_RANK // NUMA_TYPE (NUMA_TYPE <= 0 or
    TUTEL_CUDA_SANDBOX disables it)."""
    if TUTEL_CUDA_SANDBOX:
        return
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    try:
        numa_type = int(os.environ.get('NUMA_TYPE', '1'))
        if numa_type <= 0:
            return
        cpus = [c for c in _numa_cpu_sets() if c]
        node = (local_rank // numa_type) % len(cpus)
        os.sched_setaffinity(0, cpus[node])
        logging.info('LOCAL_RANK %d is to set NUMA node: %d (total NUMA nodes = %d)' % (
            local_rank, node, len(cpus)))
    except Exception as ex:
        if local_rank == 0:
            logging.warning('Failed to set NUMA status: %s' % ex)


def init_data_model_parallel(group_count=1, backend='nccl'):
    from . import net as C
    result = C.create_groups_from_world(group_count=group_count, include_init=backend)
    result.is_cuda = (result.local_device is not None and result.local_device.type == 'cuda')
    logging.critical('Registering device global rank %d: data_rank = %d, model_rank = %d' % (
        result.global_rank, result.data_rank, result.model_rank))
    init_data_model_parallel.default_env = result

    def on_quit():
        sys.stdout.flush()
        sys.stderr.flush()

    atexit.register(on_quit)
    return result


class LocalCache:
    _CACHE = dict()

    @staticmethod
    def reset():
        LocalCache._CACHE = dict()

    @staticmethod
    def set(key, val):
        LocalCache._CACHE[key] = val

    @staticmethod
    def get(key=None):
        if key not in LocalCache._CACHE:
            return list(LocalCache._CACHE.values())
        return LocalCache._CACHE[key]


def cache():
    return LocalCache


def get_local_session():
    if not hasattr(init_data_model_parallel, 'default_env'):
        raise Exception("Current session is not initialized with: system.init_data_model_parallel(). "
                        "Please try with: system.record_time(is_cuda=False)")
    return init_data_model_parallel.default_env


def record_time(is_cuda=None):
    is_cuda = is_cuda if is_cuda is not None else get_local_session().is_cuda
    if is_cuda:
        import torch
        torch.cuda.synchronize()
    return time.time()
