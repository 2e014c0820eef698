"""Weight encoders: fp32 ``[N, K]`` -> canonical GGUF-style blocks (uint8 ``[N, bytes_per_row]``).

Load-side utility, not on the per-token path.  Written with torch ops so that it runs wherever the
tensor lives (a B200 quantizes a 7B-parameter model in a fraction of a second).  Any encoder that
emits valid blocks is acceptable to the kernels; these use round-to-nearest for Q8_0 (d = amax/127)
and a direct min/max affine fit per sub-block for Q4_K / Q6_K.
"""
from __future__ import annotations

import torch

from ._lib import FMT_Q4_K, FMT_Q6_K, FMT_Q8_0


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """fp32 [...] -> little-endian fp16 bytes [..., 2] (uint8)."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    n, k = w.shape
    b = w.float().reshape(n, k // 32, 32)
    amax = b.abs().amax(dim=-1)
    d = amax / 127.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    v = b * inv.unsqueeze(-1)
    q = (torch.sign(v) * torch.floor(v.abs() + 0.5)).to(torch.int8)  # roundf: half away from zero
    out = torch.empty((n, k // 32, 34), dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = q.view(torch.uint8)
    return out.reshape(n, -1)


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    n, k = w.shape
    nb = k // 256
    x = w.float().reshape(n, nb, 8, 32)
    lo = x.amin(dim=-1).clamp(max=0.0)
    hi = x.amax(dim=-1).clamp(min=0.0)
    mn = -lo
    scale = (hi - lo) / 15.0
    d16 = (scale.amax(dim=-1) / 63.0).to(torch.float16)
    m16 = (mn.amax(dim=-1) / 63.0).to(torch.float16)
    d, dmin = d16.float().unsqueeze(-1), m16.float().unsqueeze(-1)
    sc = torch.where(d > 0, torch.round(scale / d), torch.zeros_like(scale)).clamp(0, 63)
    m = torch.where(dmin > 0, torch.round(mn / dmin), torch.zeros_like(mn)).clamp(0, 63)
    ds, dm = (d * sc).unsqueeze(-1), (dmin * m).unsqueeze(-1)
    q = torch.where(ds > 0, torch.round((x + dm) / ds), torch.zeros_like(x)).clamp(0, 15).to(torch.uint8)
    sc, m = sc.to(torch.uint8), m.to(torch.uint8)
    out = torch.empty((n, nb, 144), dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d16.float())
    out[..., 2:4] = _f16_bytes(m16.float())
    out[..., 4:8] = (sc[..., :4] & 63) | ((sc[..., 4:] >> 4) << 6)
    out[..., 8:12] = (m[..., :4] & 63) | ((m[..., 4:] >> 4) << 6)
    out[..., 12:16] = (sc[..., 4:] & 15) | ((m[..., 4:] & 15) << 4)
    qp = q.reshape(n, nb, 4, 2, 32)  # pair p holds sub-blocks 2p (low nibble) and 2p+1 (high nibble)
    out[..., 16:] = (qp[:, :, :, 0, :] | (qp[:, :, :, 1, :] << 4)).reshape(n, nb, 128)
    return out.reshape(n, -1)


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    n, k = w.shape
    nb = k // 256
    x = w.float().reshape(n, nb, 16, 16)
    s = x.abs().amax(dim=-1) / 31.0
    d16 = (s.amax(dim=-1) / 127.0).to(torch.float16)
    d = d16.float().unsqueeze(-1)
    isc = torch.where(d > 0, torch.round(s / d), torch.zeros_like(s)).clamp(0, 127)
    ds = (d * isc).unsqueeze(-1)
    q = torch.where(ds > 0, torch.round(x / ds), torch.zeros_like(x)).clamp(-32, 31) + 32
    q = q.to(torch.uint8).reshape(n, nb, 2, 4, 32)  # [half][group of 32][l]
    out = torch.empty((n, nb, 210), dtype=torch.uint8, device=w.device)
    ql = torch.empty((n, nb, 2, 64), dtype=torch.uint8, device=w.device)
    ql[..., 0:32] = (q[:, :, :, 0] & 15) | ((q[:, :, :, 2] & 15) << 4)
    ql[..., 32:64] = (q[:, :, :, 1] & 15) | ((q[:, :, :, 3] & 15) << 4)
    qh = (q[:, :, :, 0] >> 4) | ((q[:, :, :, 1] >> 4) << 2) | ((q[:, :, :, 2] >> 4) << 4) | ((q[:, :, :, 3] >> 4) << 6)
    out[..., 0:128] = ql.reshape(n, nb, 128)
    out[..., 128:192] = qh.reshape(n, nb, 64)
    out[..., 192:208] = isc.to(torch.int8).view(torch.uint8)
    out[..., 208:210] = _f16_bytes(d16.float())
    return out.reshape(n, -1)


_QUANTIZERS = {FMT_Q8_0: quantize_q8_0, FMT_Q4_K: quantize_q4_k, FMT_Q6_K: quantize_q6_k}


def quantize(fmt: int, w: torch.Tensor) -> torch.Tensor:
    """Encode an fp32 ``[N, K]`` weight (K a multiple of the block length) into canonical blocks."""
    return _QUANTIZERS[fmt](w)
