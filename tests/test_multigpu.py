"""Multi-GPU tests (one process per GPU, NCCL control plane): the fused expert-parallel layer and
the generic codec/comm pipeline against the dense oracle, and every all-to-all algorithm of the
symmetric-heap transport against ``all_to_all_single``."""

import pytest
import torch

from mp_util import run_workers

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
need2 = pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
need4 = pytest.mark.skipif(NGPU < 4, reason="needs 4 GPUs")
ENV = {'NCCL_NVLS_ENABLE': '0'}


@need2
@pytest.mark.parametrize("degree", [1, 2])
def test_fused_layer_two_ranks(degree):
    run_workers('gpu_layer', 2, backend='nccl', env=ENV, args=('naive', 'no', degree, 1))


@need2
def test_generic_layer_two_ranks_int8_pipe():
    run_workers('gpu_layer', 2, backend='nccl', env=ENV, args=('naive', 'int8', 2, 0))


@need2
@pytest.mark.parametrize("algo", ['flat', 'pipe', 'dd', 'hetu'])
def test_a2a_two_ranks(algo):
    run_workers('gpu_a2a', 2, backend='nccl', env=dict(ENV, LOCAL_SIZE=1 if algo == 'pipe' else 2), args=(algo,))


@need4
@pytest.mark.parametrize("algo", ['flat', 'pipe', 'dd', 'hetu'])
def test_a2a_four_ranks_two_groups(algo):
    run_workers('gpu_a2a', 4, backend='nccl', env=dict(ENV, LOCAL_SIZE=2), args=(algo,))


@need4
def test_fused_layer_four_ranks():
    run_workers('gpu_layer', 4, backend='nccl', env=ENV, args=('naive', 'no', 2, 1))


@need2
def test_codec_comm_pipeline():
    run_workers('gpu_codec_comm_pipeline', 2, backend='nccl', env=ENV, args=('naive', 'int8'))
