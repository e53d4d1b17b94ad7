"""Numerics of every sm_100a kernel against plain PyTorch fp32 references of the same op.
The tiny GEMM runs first: it validates the tcgen05 descriptors on one tile before anything
larger is launched."""

import os

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
os.environ.setdefault('PLANMOE_WAIT_BUDGET_MS', '3000')


def _lib():
    from planmoe_b200.ops import native
    return native.lib()


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device='cuda') * scale).to(torch.bfloat16)


def _ref_gemm(A, a_mn, B, b_mn):
    a = A.float().transpose(-1, -2) if a_mn else A.float()          # [G, M, K]
    b = B.float() if b_mn else B.float().transpose(-1, -2)          # [G, K, N]
    return a @ b


def _check(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, (err, scale)


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (False, False), (True, True), (True, False)])
def test_gemm_single_tile(a_mn, b_mn):
    from planmoe_b200.ops import gemm
    M, N, K = 128, 256, 64
    A = _rand(1, K, M) if a_mn else _rand(1, M, K)
    B = _rand(1, K, N) if b_mn else _rand(1, N, K)
    out = gemm.grouped_gemm(A, a_mn, B, b_mn)
    gemm.check_status()
    _check(out, _ref_gemm(A, a_mn, B, b_mn))


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (False, False), (True, True), (True, False)])
def test_gemm_single_pair_tile(a_mn, b_mn):
    """One 256 x 256 tile on a two-CTA cluster (tcgen05 cta_group::2), two K steps."""
    from planmoe_b200.ops import gemm
    M, N, K = 256, 256, 128
    A = _rand(1, K, M) if a_mn else _rand(1, M, K)
    B = _rand(1, K, N) if b_mn else _rand(1, N, K)
    out = gemm.grouped_gemm(A, a_mn, B, b_mn, cta_group=2)
    gemm.check_status()
    _check(out, _ref_gemm(A, a_mn, B, b_mn))


@pytest.mark.parametrize("cg", [1, 2])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (False, False), (True, True)])
@pytest.mark.parametrize("G,M,N,K", [(2, 256, 512, 256), (3, 200, 320, 96), (2, 1024, 768, 1024), (1, 64, 64, 2048)])
def test_gemm_shapes(a_mn, b_mn, G, M, N, K, cg):
    from planmoe_b200.ops import gemm
    A = _rand(G, K, M) if a_mn else _rand(G, M, K)
    B = _rand(G, K, N) if b_mn else _rand(G, N, K)
    out = gemm.grouped_gemm(A, a_mn, B, b_mn, cta_group=cg)
    gemm.check_status()
    assert out.shape == (G, M, N)
    _check(out, _ref_gemm(A, a_mn, B, b_mn))


@pytest.mark.parametrize("cg", [1, 2])
def test_gemm_many_tiles_persistent(cg):
    """More tiles than SMs: exercises the ring / accumulator phase wrap-around."""
    from planmoe_b200.ops import gemm
    G, M, N, K = 2, 4096, 2048, 512
    A, B = _rand(G, M, K), _rand(G, K, N)
    out = gemm.grouped_gemm(A, False, B, True, cta_group=cg)
    gemm.check_status()
    _check(out, _ref_gemm(A, False, B, True))
    out2 = gemm.grouped_gemm(A, False, B, True, cta_group=cg)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("cg", [1, 2])
@pytest.mark.parametrize("act", ['relu', 'gelu', 'silu', 'identity'])
def test_gemm_epilogues(act, cg, monkeypatch):
    from planmoe_b200.ops import gemm
    monkeypatch.setattr(gemm, 'DEFAULT_CTA_GROUP', cg)
    G, M, N, K = 2, 384, 512, 256
    A, B = _rand(G, M, K), _rand(G, K, N, scale=0.1)
    bias = _rand(G, N)
    code = gemm.ACT_CODES[act]
    fn = {'relu': F.relu, 'gelu': F.gelu, 'silu': F.silu, 'identity': lambda v: v}[act]
    dact = torch.empty(G, M, N, device='cuda', dtype=torch.bfloat16)
    h = gemm.grouped_gemm(A, False, B, True, gemm.EPI_BIAS_ACT, code, bias=bias, aux=dact)
    gemm.check_status()
    ref_pre = (_ref_gemm(A, False, B, True) + bias.float()[:, None, :]).requires_grad_(True)
    ref_h = fn(ref_pre)
    ref_h.sum().backward()
    _check(h, ref_h.detach())
    _check(dact, ref_pre.grad)                    # the epilogue saves act'(A.B + bias)
    # activation backward: D = (A.B) * aux
    d = gemm.grouped_gemm(A, False, B, True, gemm.EPI_DACT, code, aux=dact)
    gemm.check_status()
    _check(d, _ref_gemm(A, False, B, True) * dact.float())


@pytest.mark.parametrize("cg", [1, 2])
def test_gemm_split_k_chunks(cg):
    from planmoe_b200.ops import gemm
    d, G, R, M, N = 3, 2, 192, 256, 320
    A, B = _rand(d, G, R, M), _rand(d, G, R, N)
    out = gemm.grouped_gemm(A, True, B, True, cta_group=cg)
    gemm.check_status()
    ref = torch.einsum('dgrm,dgrn->gmn', A.float(), B.float())
    _check(out, ref)


def test_colsum():
    x = _rand(3, 1000, 256)
    out = _lib().colsum(x)
    assert torch.allclose(out, x.float().sum(1), atol=1e-2, rtol=1e-3)
    # fold: chunk blocks of groups are added together; bf16 output comes from the same kernel
    x = _rand(6, 517, 328)
    ref = x.float().sum(1).view(3, 2, 328).sum(0)
    out = _lib().colsum(x, 3)
    assert out.shape == (2, 328) and torch.allclose(out, ref, atol=2e-2, rtol=1e-3)
    ob = _lib().colsum(x, 3, True)
    assert ob.dtype == torch.bfloat16 and torch.equal(ob, out.to(torch.bfloat16))
    assert torch.equal(_lib().colsum(x, 3), out)            # fixed summation order
    # two tensors of different shapes in one launch give what two launches give
    xa, xb = _rand(4, 700, 264), _rand(4, 300, 520)
    oa, ob2 = _lib().colsum2(xa, xb, 2)
    assert torch.equal(oa, _lib().colsum(xa, 2)) and torch.equal(ob2, _lib().colsum(xb, 2))
    assert torch.allclose(ob2, xb.float().sum(1).view(2, 2, 520).sum(0), atol=2e-2, rtol=1e-3)
    ha, hb = _lib().colsum2(xa, xb, 2, True)
    assert torch.equal(ha, oa.to(torch.bfloat16)) and torch.equal(hb, ob2.to(torch.bfloat16))


def test_expert_ffn_forward_backward():
    from planmoe_b200.ops import gemm
    G, R, M, H = 2, 512, 256, 384
    x = _rand(G, R, M).requires_grad_(True)
    w1 = _rand(G, M, H, scale=0.05).requires_grad_(True)
    b1 = _rand(G, H, scale=0.1).requires_grad_(True)
    w2 = _rand(G, H, M, scale=0.05).requires_grad_(True)
    b2 = _rand(G, M, scale=0.1).requires_grad_(True)
    y = gemm.expert_ffn(x, w1, b1, w2, b2, 'gelu')
    dy = _rand(G, R, M)
    y.backward(dy)
    gemm.check_status()
    ref_in = [t.detach().float().requires_grad_(True) for t in (x, w1, b1, w2, b2)]
    xr, w1r, b1r, w2r, b2r = ref_in
    yr = F.gelu(xr @ w1r + b1r[:, None]) @ w2r + b2r[:, None]
    yr.backward(dy.float())
    _check(y, yr)
    for t, r in zip((x, w1, b1, w2, b2), ref_in):
        _check(t.grad, r.grad, tol=3e-2)


# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("S,E,K", [(1000, 16, 2), (4096, 8, 1), (777, 64, 4), (8192, 2, 2)])
def test_fused_gate_matches_reference_routing(S, E, K):
    from planmoe_b200.impls.fast_dispatch import extract_critical
    torch.manual_seed(0)
    logits = torch.randn(S, E, device='cuda')
    cap = K * ((S + E - 1) // E)
    idx, loc, gates, smap, top1, laux = _lib().gate_forward(logits, K, cap, True)
    scores = F.softmax(logits, dim=1)
    crit, l_ref = extract_critical(scores, K, capacity_factor=1.0)
    for k in range(K):
        assert torch.equal(idx[k], crit[1][k])
        assert torch.equal(loc[k], crit[2][k])
        assert torch.allclose(gates[k], crit[3][k], atol=1e-6, rtol=1e-5)
    assert crit[4] == cap
    assert torch.allclose(laux[0], l_ref, rtol=1e-5, atol=1e-7)
    ref_map = _lib().build_slot_map(idx, loc, E, cap)
    assert torch.equal(smap, ref_map)
    # run-to-run reproducibility
    again = _lib().gate_forward(logits, K, cap, True)
    assert all(torch.equal(a, b) for a, b in zip((idx, loc, gates, smap, top1, laux), again))


@pytest.mark.parametrize("normalize", [True, False])
def test_fused_gate_backward(normalize):
    from planmoe_b200.ops.fused_moe import fused_gate
    from planmoe_b200.impls.fast_dispatch import extract_critical
    S, E, K = 512, 16, 2
    logits = torch.randn(S, E, device='cuda', requires_grad=True)
    wg = torch.randn(K, S, device='cuda')
    gates, l_aux, idx, loc, smap = fused_gate(logits, K, 64, normalize)
    ((gates * wg).sum() + 3.0 * l_aux).backward()
    ref = logits.detach().clone().requires_grad_(True)
    crit, l_ref = extract_critical(F.softmax(ref, dim=1), K, normalize_gate=normalize)
    ((torch.stack(crit[3]) * wg).sum() + 3.0 * l_ref).backward()
    assert torch.allclose(logits.grad, ref.grad, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_dispatch_kernels(dtype):
    from planmoe_b200.ops import dispatch as D
    S, E, K, M, C = 600, 8, 2, 256, 100
    torch.manual_seed(1)
    idx = torch.stack([torch.randperm(E, device='cuda')[:K] for _ in range(S)]).t().contiguous().int()
    loc = torch.zeros(K, S, dtype=torch.int32, device='cuda')
    cnt = torch.zeros(E, dtype=torch.int64)
    for k in range(K):
        for t in range(S):
            e = int(idx[k, t]); loc[k, t] = int(cnt[e]); cnt[e] += 1
    plan = D.SlotPlan(idx, loc, E, C)
    x = torch.randn(S, M, device='cuda').to(dtype).requires_grad_(True)
    gates = torch.rand(K, S, device='cuda', requires_grad=True)
    y = D.scatter(x, plan, None)
    yr = D.scatter_torch(x.detach().float(), plan, None)
    assert torch.equal(y.float(), yr)
    z = D.gather(y, plan, gates)
    (z.float() * torch.linspace(0, 1, M, device='cuda')).sum().backward()
    xr = x.detach().float().requires_grad_(True)
    gr = gates.detach().clone().requires_grad_(True)
    zr = D.gather_torch(D.scatter_torch(xr, plan, None), plan, gr)
    (zr * torch.linspace(0, 1, M, device='cuda')).sum().backward()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(z.float(), zr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol, rtol=tol)
    assert torch.allclose(gates.grad, gr.grad, atol=tol * 50, rtol=tol)


def test_int8_codec_roundtrip():
    x = F.relu(torch.randn(512, 4096, device='cuda')).to(torch.bfloat16)
    x[7] = 3.0                                          # constant row
    q, scale, bias = _lib().int8_encode(x)
    y = _lib().int8_decode(q, scale, bias, torch.bfloat16)
    f = x.float()
    lo, hi = f.min(1).values, f.max(1).values
    assert torch.allclose(scale, hi - lo) and torch.allclose(bias, lo)
    err = (y.float() - f).abs().max(1).values
    assert (err <= (hi - lo) / 255 * 0.51 + 0.02 * f.abs().max(1).values + 1e-6).all()
    assert torch.equal(y[7], x[7])


def test_cumsum_sub_one():
    from planmoe_b200.jit_kernels.gating import fast_cumsum_sub_one
    m = (torch.rand(1337, 24, device='cuda') > 0.7).int()
    assert torch.equal(fast_cumsum_sub_one(m), torch.cumsum(m, 0).int() - 1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_zfp_cuda_stream_is_bit_identical_to_cpu_oracle(dtype):
    torch.manual_seed(0)
    x = F.relu(torch.randn(4, 130, 256)).to(dtype)
    for rate in (4, 8, 16):
        s_cpu = _lib().zfp_encode(x, rate)
        s_gpu = _lib().zfp_encode(x.cuda(), rate)
        assert torch.equal(s_gpu.cpu(), s_cpu)
        y_cpu = _lib().zfp_decode(s_cpu, 4, 130, 256, rate, dtype)
        y_gpu = _lib().zfp_decode(s_gpu, 4, 130, 256, rate, dtype)
        assert torch.equal(y_gpu.cpu(), y_cpu)


@pytest.mark.parametrize("sym", [2, 4])
def test_lz_cuda_matches_cpu_oracle_and_roundtrips(sym):
    torch.manual_seed(0)
    x = F.relu(torch.randn(4, 8192)).to(torch.bfloat16 if sym == 2 else torch.float32)
    raw = x.view(torch.uint8).reshape(4, -1).contiguous()
    p_cpu, n_cpu = _lib().lz_encode(raw, sym)
    p_gpu, n_gpu = _lib().lz_encode(raw.cuda(), sym)
    assert torch.equal(n_gpu.cpu(), n_cpu)
    for s in range(4):
        n = int(n_cpu[s])
        assert torch.equal(p_gpu[s, :n].cpu(), p_cpu[s, :n])
    back = _lib().lz_decode(p_gpu, n_gpu, raw.size(1), sym)
    assert torch.equal(back.cpu(), raw)
    assert int(n_cpu.max()) < raw.size(1)


def test_codec_objects_on_cuda():
    from planmoe_b200.parallel import codecs
    x = F.relu(torch.randn(4, 64, 256, device='cuda')).to(torch.bfloat16)
    for name, tol in (('no', 0.0), ('lz', 0.0), ('int8', 0.02), ('zfp', 0.08)):
        c = codecs.get_compressor(name)
        y = c.decompress(c.compress(x, world_size=4))
        err = ((y.float() - x.float()).abs().max() / x.float().abs().max()).item()
        assert err <= tol, (name, err)


def test_bounded_flag_wait_reports_timeout_instead_of_hanging():
    """A wait on a flag that nothing sets gives up after its budget and records a status code."""
    lib = _lib()
    st = lib.StatusWord()
    flags = torch.zeros(4, dtype=torch.int64, device='cuda')
    lib.wait_flags(flags.data_ptr(), 4, 1, 50, st.device_ptr())          # 50 ms budget
    torch.cuda.synchronize()
    code = st.read()
    assert code[0] == 1 and code[2] == 1 and code[3] == 0
    st.clear()
    flags.fill_(5)
    lib.wait_flags(flags.data_ptr(), 4, 1, 50, st.device_ptr())
    torch.cuda.synchronize()
    assert st.read()[0] == 0


def test_gemm_flag_gate_times_out_cleanly_and_context_survives():
    """Flag-gated GEMM whose flags never arrive: the kernel aborts through the status word, frees its
    TMEM and returns; a normal GEMM afterwards still works."""
    from planmoe_b200.ops import gemm
    lib = _lib()
    st = lib.StatusWord()
    flags = torch.zeros(8, dtype=torch.int64, device='cuda')
    A, B = _rand(1, 256, 128), _rand(1, 128, 256)
    gemm.grouped_gemm(A, False, B, True, gate_flags_ptr=flags.data_ptr(), gate_rows=128, gate_want=1,
                      budget_ms=100, status_ptr=st.device_ptr())
    torch.cuda.synchronize()
    assert st.read()[0] in (1, 2)
    out = gemm.grouped_gemm(A, False, B, True)
    gemm.check_status()
    _check(out, _ref_gemm(A, False, B, True))


def test_user_jit_kernel_runs_on_current_stream():
    from planmoe_b200 import jit
    fn = jit.create_cuda_kernel('''
      __global__ void scale_add(float* x, float* y, int n, int k) {
        // [thread_extent] blockIdx.x = 4
        // [thread_extent] threadIdx.x = 256
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) y[i] = x[i] * @factor@ + k;
      }''', {'factor': 3})
    x = torch.arange(5000, dtype=torch.float32, device='cuda')
    y = torch.zeros_like(x)
    fn(x, y, extra=[5000, 7])
    torch.cuda.synchronize()
    assert torch.equal(y, x * 3 + 7)
