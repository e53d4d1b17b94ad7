"""CPU oracles of the codecs: ZFP fixed-rate 2-D (error bounds, fixed stream size, zero blocks), LZ
(bit-exact round trip incl. -0.0 / NaN payloads, real size reduction on sparse data), int8."""

import pytest
import torch
import torch.nn.functional as F

from planmoe_b200.ops import native
from planmoe_b200.parallel import codecs


def test_zfp_roundtrip_error_and_stream_size():
    lib = native.lib()
    torch.manual_seed(0)
    x = torch.randn(3, 10, 32)                       # rows not a multiple of 4: padded blocks
    for rate, bound in ((16, 2e-4), (8, 6e-2), (4, 0.6)):
        s = lib.zfp_encode(x, rate)
        assert s.shape == (3, 3 * 8 * 2 * rate) and s.dtype == torch.uint8
        y = lib.zfp_decode(s, 3, 10, 32, rate, torch.float32)
        rel = ((y - x).abs().max() / x.abs().max()).item()
        assert rel < bound, (rate, rel)
    z = torch.zeros(1, 4, 8)
    s = lib.zfp_encode(z, 8)
    assert int(s.sum()) == 0 and torch.equal(lib.zfp_decode(s, 1, 4, 8, 8, torch.float32), z)
    smooth = torch.linspace(0, 1, 64).view(1, 8, 8).contiguous()
    y = lib.zfp_decode(lib.zfp_encode(smooth, 8), 1, 8, 8, 8, torch.float32)
    assert (y - smooth).abs().max() < 1e-3           # smooth data compresses far better than noise


def test_zfp_bf16_and_codec_object_split_is_even():
    c = codecs.get_compressor('zfp')
    x = F.relu(torch.randn(4, 8, 64)).to(torch.bfloat16)
    p = c.compress(x, world_size=4)
    assert p.wires[0].shape[0] == 4 and p.wires[0].numel() == x.numel()      # 8 bits per value
    y = c.decompress(p)
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    assert ((y.float() - x.float()).abs().max() / x.float().abs().max()).item() < 8e-2
    # slice independence: decoding one leading slice alone gives the same values
    lib = native.lib()
    one = lib.zfp_decode(p.wires[0][2:3].contiguous(), 1, 8, 64, 8, torch.bfloat16)
    assert torch.equal(one[0], y[2])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_lz_lossless_and_smaller_on_sparse_activations(dtype):
    c = codecs.get_compressor('lz')
    torch.manual_seed(0)
    x = F.relu(torch.randn(4, 64, 256)).to(dtype)
    x[0, 0, :4] = torch.tensor([-0.0, float('nan'), float('inf'), 1.0]).to(dtype)
    p = c.compress(x, world_size=4)
    y = c.decompress(p)
    assert torch.equal(y.view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       x.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    raw = x.numel() * x.element_size()
    assert p.wire_bytes() < 0.95 * raw, (p.wire_bytes(), raw)
    dense = torch.randn(2, 16, 256).to(dtype)
    q = c.compress(dense, world_size=2)
    assert torch.equal(c.decompress(q), dense)


def test_lz_long_runs_and_tail_block():
    lib = native.lib()
    raw = torch.zeros(2, 2048 + 512, dtype=torch.uint8)
    raw[1, ::7] = 3
    payload, sizes = lib.lz_encode(raw, 2)
    assert int(sizes[0]) < 400
    back = lib.lz_decode(payload, sizes, raw.size(1), 2)
    assert torch.equal(back, raw)


def test_int8_cpu_matches_formula_and_guards_constant_rows():
    c = codecs.get_compressor('int8')
    x = torch.randn(6, 5, 32)
    x[1, 2] = 0.25
    p = c.compress(x)
    y = c.decompress(p)
    rng = x.amax(-1) - x.amin(-1)
    assert ((y - x).abs().amax(-1) <= rng / 255 * 0.5 + 1e-6).all()
    assert torch.equal(y[1, 2], x[1, 2])
    assert p.wires[0].dtype == torch.uint8 and p.wires[1].shape == (6, 5)
