"""The C++ comm extension point, used the way a user would: an all-to-all algorithm in a source file outside
the library (tests/user_comm/reverse_flat_comm.cpp) is compiled against the library's headers, loaded next to
``_C.so``, found by name through the registry and used as ``comm_name`` of a MoE layer."""

import ctypes
import os
import subprocess
import sys
import sysconfig

import pytest
import torch

from mp_util import run_workers

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def build_user_comm(out_dir):
    from planmoe_b200.ops import native
    native.lib()
    pkg = os.path.join(ROOT, 'planmoe_b200')
    cuda = os.environ.get('CUDA_HOME', '/usr/local/cuda')
    so = os.path.join(str(out_dir), 'libuser_reverse_comm.so')
    cmd = ['g++', '-shared', '-fPIC', '-O2', '-std=c++17', '-I' + os.path.join(pkg, 'csrc'), '-I' + os.path.join(cuda, 'include'),
           os.path.join(HERE, 'user_comm', 'reverse_flat_comm.cpp'), '-o', so, '-L' + pkg, '-l:_C.so',
           '-L' + os.path.join(cuda, 'lib64'), '-lcudart', '-Wl,-rpath,' + pkg]
    subprocess.run(cmd, check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return so


def test_user_comm_registers_and_is_the_identity_for_one_rank(tmp_path):
    so = build_user_comm(tmp_path)
    from planmoe_b200.ops import native
    from planmoe_b200.parallel import comms
    lib = native.lib()
    ctypes.CDLL(so, mode=ctypes.RTLD_GLOBAL)
    assert 'user_reverse' in lib.native_comm_names()
    c = comms.get_comm('user_reverse')
    assert isinstance(c, comms.NativeComm)
    x = torch.arange(64.)
    assert torch.equal(c.all_to_all(x), x)
    # and a whole layer on CPU with it
    from planmoe_b200 import moe
    layer = moe.moe_layer({'type': 'top', 'k': 2}, 32, experts={'type': 'ffn', 'count_per_node': 2,
                                                            'hidden_size_per_expert': 32}, comm_name='user_reverse')
    y = layer(torch.randn(16, 32))
    assert y.shape == (16, 32) and torch.isfinite(y).all()


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("comm", ['user_reverse', 'native_flat', 'native_pipe'])
def test_layer_with_cpp_comm_two_ranks(tmp_path, comm):
    so = build_user_comm(tmp_path)
    env = {'NCCL_NVLS_ENABLE': '0', 'PLANMOE_USER_COMM_SO': so, 'LOCAL_SIZE': 1}
    run_workers('gpu_layer', 2, backend='nccl', env=env, args=(comm, 'no', 2, 0))
    run_workers('gpu_native_comm_a2a', 2, backend='nccl', env=env, args=(comm,))
