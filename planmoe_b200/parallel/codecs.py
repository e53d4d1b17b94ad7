"""Payload codecs applied around every MoE all-to-all (forward activations and gradients).

Python face of the ``AbstractCompressor`` extension point (reference:
``PlanMoE/custom/compressor/abstract.h:11-22``; codecs ``no.cpp``, ``int8.cpp``, ``zfpc.cpp``,
``lz.cpp``).  A codec turns one tensor whose leading dimension is split evenly over the
destination ranks into a ``Packed`` record: a list of wire tensors, each also evenly split on
dim 0 over the ranks, so any all-to-all algorithm can move them without knowing the codec.

Names: ``no`` | ``int8`` | ``zfp`` | ``lz``; unknown names fall back to ``no`` as the
reference's factory does (``custom_kernel.cpp:194-207``).  ``register_compressor`` adds more.

Defects of the reference that are deliberately not reproduced: int8 guards a zero value range
and rounds to nearest instead of truncating; zfp accepts bf16/fp16 (widened) and any shape
whose last dim is a multiple of 4 (rows are padded to a multiple of 4); lz works on 16-bit or
32-bit symbols and really shrinks the wire volume (sizes travel first, data is packed).
"""

import torch

from ..ops import native


class Packed:
    """Wire form of one tensor: ``wires`` are moved by the all-to-all; ``meta`` stays local.

    ``var_len`` (optional) marks wire 0 as ``[W, cap]`` bytes of self-describing slices: ``(len_off,
    len_base)`` as understood by ``AbstractComm.all_to_all_var``."""
    __slots__ = ('wires', 'meta', 'var_len')

    def __init__(self, wires, meta, var_len=None):
        self.wires, self.meta, self.var_len = wires, meta, var_len

    def wire_bytes(self):
        """Bytes that cross the link (a statistic: for a variable-length wire it reads the slice headers, which
        synchronises with the device)."""
        total = sum(w.numel() * w.element_size() for w in self.wires[1 if self.var_len else 0:])
        if self.var_len:
            off, base = self.var_len
            w0 = self.wires[0]
            sizes = w0[:, off:off + 4].contiguous().view(torch.int32).to(torch.int64) + base
            total += int(((sizes + 15) // 16 * 16).sum().item())
        return total


class AbstractCompressor:
    name = 'abstract'
    lossless = False

    def compress(self, t, world_size=1):
        raise NotImplementedError

    def decompress(self, packed):
        raise NotImplementedError


class NoCompressor(AbstractCompressor):
    name, lossless = 'no', True

    def compress(self, t, world_size=1):
        return Packed([t.contiguous()], None)

    def decompress(self, packed):
        return packed.wires[0]


class Int8Compressor(AbstractCompressor):
    """Per-row (last dim) affine 8-bit quantisation: q = round((x - min) / (max - min) * 255).

    Wire: uint8 payload ``[..., M]`` plus fp32 ``scale`` and ``bias`` per row.  A constant row
    (max == min) gets scale 0 and decodes exactly.
    """
    name = 'int8'

    def compress(self, t, world_size=1):
        t = t.contiguous()
        rows = t.reshape(-1, t.size(-1))
        if t.is_cuda:
            q, scale, bias = native.lib().int8_encode(rows)
        else:
            f = rows.float()
            lo, hi = f.min(dim=1).values, f.max(dim=1).values
            scale = hi - lo
            inv = torch.where(scale > 0, 255.0 / scale, torch.zeros_like(scale))
            q = torch.clamp(torch.round((f - lo[:, None]) * inv[:, None]), 0, 255).to(torch.uint8)
            bias = lo
        lead = list(t.shape[:-1])
        return Packed([q.view(t.shape), scale.view(lead), bias.view(lead)], (t.dtype,))

    def decompress(self, packed):
        q, scale, bias = packed.wires
        (dtype,) = packed.meta
        rows = q.reshape(-1, q.size(-1))
        if q.is_cuda:
            out = native.lib().int8_decode(rows, scale.reshape(-1).contiguous(),
                                           bias.reshape(-1).contiguous(), dtype)
        else:
            out = (rows.float() * (scale.reshape(-1, 1) / 255.0) + bias.reshape(-1, 1)).to(dtype)
        return out.view(q.shape)


class ZfpCompressor(AbstractCompressor):
    """ZFP-style fixed-rate 2-D codec: 4x4 blocks, ``rate`` bits per value (default 8, i.e.
    128 bits per block) — block-floating point, integer lifting transform, sequency order,
    negabinary, embedded bit-plane coding under a fixed budget.

    The tensor is viewed as ``[rows, M]`` with rows = product of the leading dims; rows of each
    leading-dim slice are padded to a multiple of 4, so an even split of the leading dim is an
    even split of the stream.
    """
    name = 'zfp'

    def __init__(self, rate=8.0):
        self.rate = float(rate)

    def set_compress_rate(self, rate):
        self.rate = float(rate)

    def compress(self, t, world_size=1):
        t = t.contiguous()
        assert t.size(-1) % 4 == 0, "zfp codec needs the last dim to be a multiple of 4"
        lead = int(t.shape[0])
        inner = t.reshape(lead, -1, t.size(-1))
        stream = native.lib().zfp_encode(inner, int(self.rate))      # uint8 [lead, bytes]
        return Packed([stream], (t.dtype, tuple(t.shape)))

    def decompress(self, packed):
        dtype, shape = packed.meta
        lead = shape[0]
        rows = 1
        for s in shape[1:-1]:
            rows *= s
        out = native.lib().zfp_decode(packed.wires[0], lead, rows, shape[-1], int(self.rate), dtype)
        return out.view(shape)


class LzCompressor(AbstractCompressor):
    """Lossless LZ (sliding-window 32, 2 KiB blocks) on raw 16-/32-bit symbols.

    Each destination slice is compressed on its own into a self-describing record: a header (block count,
    block offsets, total code bytes) followed by the packed code.  The wire is ONE byte tensor ``[W, cap]``
    with ``cap`` the worst-case slice size; it is marked variable-length, so a transport that can read the
    header on the device (the symmetric-heap all-to-all kernels) moves only ``header + code`` bytes per slice
    and the host never reads a size.  Every rank therefore offers the same shape to the exchange whatever
    its data compresses to.
    """
    name, lossless = 'lz', True

    @staticmethod
    def _layout(raw_bytes, cuda):
        lib = native.lib()
        return lib.lz_layout(int(raw_bytes))          # (cap, len_off, header_bytes)

    def compress(self, t, world_size=1):
        t = t.contiguous()
        W = max(int(world_size), 1)
        assert t.size(0) % W == 0
        sym = t.element_size()
        assert sym in (2, 4), "lz codec works on 16- or 32-bit element types"
        raw = t.view(torch.uint8).reshape(W, -1)
        payload, _sizes = native.lib().lz_encode(raw, sym)    # uint8 [W, cap]; sizes also sit in the headers
        _cap, len_off, header = self._layout(raw.size(1), t.is_cuda)
        return Packed([payload], (t.dtype, tuple(t.shape), sym), var_len=(len_off, header))

    def decompress(self, packed):
        dtype, shape, sym = packed.meta
        payload = packed.wires[0]
        W = payload.size(0)
        numel = 1
        for s in shape:
            numel *= s
        raw_bytes = numel * sym // W
        sizes = torch.empty(0, dtype=torch.int32, device=payload.device)
        out = native.lib().lz_decode(payload.contiguous(), sizes, raw_bytes, sym)   # uint8 [W, raw]
        return out.view(dtype).view(shape)


_REGISTRY = {}


def register_compressor(name, factory):
    """Register ``factory() -> AbstractCompressor`` under ``name`` (overrides built-ins)."""
    _REGISTRY[name] = factory


class NativeCompressor(AbstractCompressor):
    """Bridge to a codec registered in C++ (``planmoe::register_compressor``)."""

    def __init__(self, name):
        self.name = name

    def compress(self, t, world_size=1):
        wire = native.lib().native_codec_run(self.name, t.contiguous(), max(int(world_size), 1), False, 0)
        return Packed([wire.view(max(int(world_size), 1), -1)], (t.dtype, tuple(t.shape)))

    def decompress(self, packed):
        dtype, shape = packed.meta
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        raw = native.lib().native_codec_run(self.name, packed.wires[0].contiguous().view(-1), 1, True, nbytes)
        return raw.view(dtype).view(shape)


def get_compressor(name):
    factory = _REGISTRY.get(name)
    if factory is not None:
        return factory()
    lib = native.maybe_lib()
    if lib is not None and name in lib.native_compressor_names():
        return NativeCompressor(name)
    return NoCompressor()


register_compressor('no', NoCompressor)
register_compressor('int8', Int8Compressor)
register_compressor('zfp', ZfpCompressor)
register_compressor('lz', LzCompressor)
