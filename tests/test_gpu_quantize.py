"""Stage 1 parity: int4 codes, packed bytes and scales bit-exact against the oracle."""
import pytest
import torch

from kv_cache_b200 import ops
from oracle import oracle
from tests.gpu_util import cpu, make_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("C", [16, 32, 64, 128, 34, 6])
@pytest.mark.parametrize("T", [1, 15, 16, 17, 257, 1000])
def test_quantize_bit_exact(cuda_device, C, T):
    w, q, key, _ = make_case(cuda_device, context=T, channels=C)
    hist = key[:, :, :T]
    ch = ops.choose_channels(hist, C)
    packed, scale = ops.quantize(hist, ch)
    codes_o, packed_o, scale_o = oracle.quantize_pack(*cpu(hist, ch))
    assert torch.equal(packed.cpu(), packed_o)
    assert torch.equal(scale.cpu().view(torch.int32), scale_o.view(torch.int32))
    assert torch.equal(ops.unpack_codes(packed).cpu(), codes_o)


def test_quantize_strided_view_and_append(cuda_device):
    """A sliced key (the HF cache hands out [:, :, :T] views) and the one-row append."""
    w, q, key, _ = make_case(cuda_device, context=300, channels=64)
    T = 300
    ch = ops.choose_channels(key[:, :, :T], 64)
    packed, scale = ops.alloc_side_cache(w.batch, w.kv_heads, T + 1, 64, cuda_device)
    packed.fill_(0xAB)
    scale.fill_(-1.0)
    ops.quantize(key[:, :, :T], ch, out=(packed, scale))          # non-contiguous batch/head strides
    ops.quantize_append(key[:, :, T:T + 1], ch, packed, scale, T)
    _, packed_o, scale_o = oracle.quantize_pack(key.cpu(), ch.cpu())
    assert torch.equal(packed[:, :, :T + 1].cpu(), packed_o)
    assert torch.equal(scale[:, :, :T + 1].cpu(), scale_o)
    # nothing beyond the written rows was touched
    assert (packed[:, :, T + 1:] == 0xAB).all() and (scale[:, :, T + 1:] == -1.0).all()


def test_quantize_edge_values(cuda_device):
    """All-zero rows, a single huge outlier, exact .5 rounding ties."""
    T, D, C = 8, 128, 32
    key = torch.zeros(1, 1, T, D, dtype=torch.bfloat16, device=cuda_device)
    key[0, 0, 1, :32] = 1.0
    key[0, 0, 2, 0] = 3.0e38
    key[0, 0, 2, 1] = 1.0
    key[0, 0, 3, :32] = torch.tensor([7.0, 3.5, 2.5, 1.5, 0.5, -0.5, -1.5, -2.5] * 4, dtype=torch.bfloat16)
    key[0, 0, 4, 5] = -1.0e-30
    ch = torch.arange(C, dtype=torch.int32, device=cuda_device)[None]
    packed, scale = ops.quantize(key, ch)
    _, packed_o, scale_o = oracle.quantize_pack(key.cpu(), ch.cpu())
    assert torch.equal(packed.cpu(), packed_o)
    assert torch.equal(scale.cpu(), scale_o)


def test_every_bf16_magnitude_as_the_row_maximum(cuda_device):
    """The kernel forms scale = absmax / 7 and the codes without the division routine; the row maximum can only
    be a bf16 value, so all 32640 finite positive magnitudes are tried as the maximum of a row (with neighbours
    at fixed fractions of it, among them exact rounding boundaries) and every scale and code must equal the
    oracle's IEEE arithmetic."""
    mags = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)          # all finite positive bf16
    T = mags.numel()
    key = torch.zeros((1, 1, T, 128), dtype=torch.bfloat16)
    fr = torch.tensor([1.0, -1.0, 0.5, -0.5, 0.25, 0.75, 3 / 14, 5 / 14, 1 / 14, 13 / 14, 9 / 14, 11 / 14, 0.0, 1 / 7, 2 / 7, 6 / 7])
    key[0, 0, :, :16] = (mags.float()[:, None] * fr[None, :]).to(torch.bfloat16)
    key[0, 0, :, 16:64] = (mags.float()[:, None] * torch.linspace(-1, 1, 48)[None, :]).to(torch.bfloat16)
    ch = torch.arange(64, dtype=torch.int32).view(1, 64)
    packed, scale = ops.quantize(key.to(cuda_device), ch.to(cuda_device))
    _, packed_o, scale_o = oracle.quantize_pack(key, ch)
    assert torch.equal(scale.cpu(), scale_o)
    assert torch.equal(packed.cpu(), packed_o)


def test_every_pair_of_bf16_magnitudes(cuda_device):
    """The codes come from a reciprocal and two fused multiply-adds instead of the division routine; that is
    exact by Markstein's theorem, and this test checks it on every pair (row maximum, value) of finite positive
    bf16 magnitudes with value <= maximum (both signs of the value), against IEEE division, rint and clamp done
    by torch in fp32 on the same device. (The oracle's numpy division is tied to the same arithmetic by the
    other tests of this file.)"""
    dev = cuda_device
    mags = torch.arange(1, 0x7F80, dtype=torch.int32, device=dev).to(torch.int16).view(torch.bfloat16)   # 32639 values
    n = mags.numel()
    ch = torch.arange(64, dtype=torch.int32, device=dev).view(1, 64)
    per_row = 62                                            # channel 0: the maximum, channel 1: its negative
    rows_per_max = (n + per_row - 1) // per_row
    pad = rows_per_max * per_row - n
    xs = torch.cat([mags, mags[:1].expand(pad)]).view(rows_per_max, per_row)           # [rows_per_max, 62]
    block = 256                                             # maxima per launch: 256 * 527 rows
    for m0 in range(0, n, block):
        mx = mags[m0:m0 + block]                            # [m]
        m = mx.numel()
        vals = torch.minimum(xs[None].expand(m, -1, -1), mx[:, None, None])            # value <= maximum
        sign = torch.where((torch.arange(per_row, device=dev) & 1).bool(), -1.0, 1.0).to(torch.bfloat16)
        key = torch.zeros((1, 1, m * rows_per_max, 128), dtype=torch.bfloat16, device=dev)
        k3 = key.view(m, rows_per_max, 128)
        k3[:, :, 0] = mx[:, None]
        k3[:, :, 1] = -mx[:, None]
        k3[:, :, 2:64] = vals * sign
        packed, scale = ops.quantize(key, ch)
        sel = key[..., :64].float()
        amax = sel.abs().amax(-1).clamp_min(2.0 ** -24)
        s_ref = amax / torch.full_like(amax, 7.0)          # a tensor divisor: true division, not a multiplication by 1/7
        codes_ref = torch.round(sel / s_ref[..., None]).clamp(-7, 7).to(torch.int16)
        u = codes_ref & 0xF
        packed_ref = (u[..., 0::2] | (u[..., 1::2] << 4)).to(torch.uint8)
        assert torch.equal(scale, s_ref), f"scales differ for maxima {m0}..{m0 + m}"
        assert torch.equal(packed, packed_ref), f"codes differ for maxima {m0}..{m0 + m}"
