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
need8 = pytest.mark.skipif(NGPU < 8, reason="needs 8 GPUs")
ENV = {'NCCL_NVLS_ENABLE': '0'}


@need2
@pytest.mark.parametrize("degree", [1, 2])
def test_fused_layer_two_ranks(degree):
    run_workers('gpu_layer', 2, backend='nccl', env=ENV, args=('naive', 'no', degree, 1))


@need2
def test_fused_layer_two_ranks_int8():
    # int8 rows on the wire inside the fused kernels (quantised by the sender, de-quantised in front of the GEMM)
    run_workers('gpu_layer', 2, backend='nccl', env=ENV, args=('naive', 'int8', 2, 1))


@need2
def test_generic_layer_two_ranks_int8():
    run_workers('gpu_layer', 2, backend='nccl', env=ENV, args=('naive', 'int8', 2, 0))


@need2
@pytest.mark.parametrize("comm", ['pipe', 'dd', 'hetu'])
def test_generic_layer_two_ranks_comm(comm):
    # LOCAL_SIZE=1: two logical groups of one rank, so the grouped algorithms take their multi-group branches
    run_workers('gpu_layer', 2, backend='nccl', env=dict(ENV, LOCAL_SIZE=1), args=(comm, 'no', 2, 0))


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
@pytest.mark.parametrize("compress", ['int8', 'zfp', 'lz'])
def test_codec_comm_pipeline(compress):
    run_workers('gpu_codec_comm_pipeline', 2, backend='nccl', env=ENV, args=('naive', compress))


@need2
def test_codec_comm_pipeline_pipe_int8():
    run_workers('gpu_codec_comm_pipeline', 2, backend='nccl', env=dict(ENV, LOCAL_SIZE=1), args=('pipe', 'int8'))


# ---- 8 ranks: two logical groups of four (LOCAL_SIZE=4), short wait budget: a wait that runs out returns an error
@need8
@pytest.mark.parametrize("algo", ['flat', 'pipe', 'dd', 'hetu'])
def test_a2a_eight_ranks_two_groups(algo):
    run_workers('gpu_a2a', 8, backend='nccl', env=dict(ENV, LOCAL_SIZE=4, PLANMOE_WAIT_BUDGET_MS=3000), args=(algo,),
                timeout=300)


@need8
def test_a2a_eight_ranks_codec_wires():
    # int8 / lz wires: several tensors of unequal size through the same channel, buffers reused
    run_workers('gpu_codec_comm_pipeline', 8, backend='nccl', env=dict(ENV, LOCAL_SIZE=4, PLANMOE_WAIT_BUDGET_MS=3000),
                args=('pipe', 'int8'), timeout=300)
    run_workers('gpu_codec_comm_pipeline', 8, backend='nccl', env=dict(ENV, LOCAL_SIZE=4, PLANMOE_WAIT_BUDGET_MS=3000),
                args=('hetu', 'lz'), timeout=300)


@need8
@pytest.mark.parametrize("compress", ['no', 'int8'])
def test_fused_layer_eight_ranks(compress):
    run_workers('gpu_layer', 8, backend='nccl', env=dict(ENV, PLANMOE_WAIT_BUDGET_MS=3000), args=('naive', compress, 2, 1),
                timeout=300)
