"""Multi-process CPU (Gloo) tests: expert-parallel layer against the dense oracle for every comm
algorithm, collectives of ``net``, the ZeRO optimizer wrapper, sharded experts, and host-side
failure detection."""

import pytest

from mp_util import run_workers


@pytest.mark.parametrize("comm,world,local", [('naive', 2, 0), ('pipe', 4, 2), ('dd', 4, 2), ('hetu', 4, 2)])
def test_ep_layer_matches_oracle(comm, world, local):
    run_workers('cpu_layer', world, env={'LOCAL_SIZE': local} if local else None, args=(comm, 'no', 1))


def test_ep_layer_chunked_and_int8():
    run_workers('cpu_layer', 2, args=('naive', 'no', 2))
    run_workers('cpu_layer', 2, args=('naive', 'int8', 1))


@pytest.mark.parametrize("compress", ['lz', 'zfp'])
def test_ep_layer_two_ranks_lz_and_zfp(compress):
    # every rank's data compresses to a different size: the exchange must still agree on one shape
    run_workers('cpu_layer', 2, args=('naive', compress, 1))
    run_workers('cpu_layer', 2, args=('naive', compress, 2))


def test_net_collectives():
    run_workers('cpu_collectives', 4)


def test_async_a2a_functions():
    run_workers('cpu_async_a2a_functions', 2)


def test_checkpoint_gather_and_reload():
    run_workers('cpu_checkpoint_gather_and_reload', 2)


def test_zero_optimizer():
    run_workers('cpu_zero_optimizer', 2)


@pytest.mark.parametrize("mode", ['model', 'data'])
def test_sharded_experts(mode):
    run_workers('cpu_sharded_experts', 2, args=(mode,))


def test_missing_rank_is_detected_on_the_host():
    outs = run_workers('cpu_rank_never_joins', 3, timeout=120)
    assert any('caught' in o for o in outs)
