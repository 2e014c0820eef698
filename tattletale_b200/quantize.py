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


# ---- trellis-coded 3-bit format (include/ttq.h, TTQ_FMT_TQ3) -----------------------------------------
_TQ3_UNIT = 1.0 / 147.8


def _tq3_values(states: torch.Tensor) -> torch.Tensor:
    """Decoded value of 16-bit trellis states (int64 tensor)."""
    h = (states * 2654435761) & 0xFFFFFFFF
    s = (h & 0xFF) + ((h >> 8) & 0xFF) + ((h >> 16) & 0xFF) + (h >> 24)
    return (s - 510).to(torch.float32) * _TQ3_UNIT


def _hadamard128(t: torch.Tensor) -> torch.Tensor:
    """Orthonormal Sylvester-Hadamard transform of the last dimension in blocks of 128."""
    shape = t.shape
    v = t.reshape(-1, 128)
    h = 1
    while h < 128:
        v = v.reshape(-1, 128 // (2 * h), 2, h)
        a, b = v[:, :, 0, :], v[:, :, 1, :]
        v = torch.stack((a + b, a - b), dim=2).reshape(-1, 128)
        h *= 2
    return (v * (1.0 / 128 ** 0.5)).reshape(shape)


def quantize_tq3(w: torch.Tensor, seed: int = 1, beam: int = 64, tile_chunk: int = 1 << 13) -> torch.Tensor:
    """fp32 [N, K] -> the flat uint8 buffer of TTQ_FMT_TQ3 (tiles | out_scale fp16 | in_sign bits).

    out_scale[n] = +-rms of row n, in_sign random (seeded torch generator); the rotated, normalised target is
    coded tile by tile with a beam search over the sliding-window trellis, run from weight 255 of a tile down
    to weight 0 (the CPU checker holds the exact Viterbi search of the same code; the beam trades a little
    error for a search that vectorises over all tiles).
    """
    n, k = w.shape
    if n % 128 or k % 128:
        raise ValueError("the trellis format needs N and K in multiples of 128")
    dev = w.device
    g = torch.Generator(device="cpu").manual_seed(seed)
    in_neg = torch.randint(0, 2, (k,), generator=g).to(dev)
    out_neg = torch.randint(0, 2, (n,), generator=g).to(dev)
    w = w.float()
    rms = w.pow(2).mean(dim=1).sqrt()
    rms = torch.where(rms > 0, rms, torch.ones_like(rms))
    scale16 = torch.where(out_neg.bool(), -rms, rms).to(torch.float16)
    tiny = torch.tensor(2.0 ** -24, dtype=torch.float16, device=dev)
    scale16 = torch.where(scale16 == 0, tiny, scale16)
    t = w / scale16.float().unsqueeze(1) * torch.where(in_neg.bool(), -1.0, 1.0).unsqueeze(0)
    t = _hadamard128(t)                                   # along K
    t = _hadamard128(t.t().contiguous()).t().contiguous()  # along N
    # tiles [N/16, K/16, 16, 16] -> [tiles, 256] in weight order t = 16 r + c
    tiles = t.reshape(n // 16, 16, k // 16, 16).permute(0, 2, 1, 3).reshape(-1, 256)
    n_tiles = tiles.shape[0]
    syms = torch.empty((n_tiles, 256), dtype=torch.uint8, device=dev)
    sym_range = torch.arange(8, device=dev, dtype=torch.int64)
    for c0 in range(0, n_tiles, tile_chunk):
        tg = tiles[c0:c0 + tile_chunk]
        nt = tg.shape[0]
        ctx = torch.zeros((nt, 1), dtype=torch.int64, device=dev)       # 13-bit context of each survivor
        cost = torch.zeros((nt, 1), dtype=torch.float32, device=dev)
        back = []                                                       # per step: (parent survivor, symbol)
        for step in range(255, -1, -1):
            states = (ctx.unsqueeze(2) << 3) | sym_range                # [nt, B, 8]
            e = cost.unsqueeze(2) + (_tq3_values(states) - tg[:, step].reshape(nt, 1, 1)) ** 2
            e = e.reshape(nt, -1)
            keep = min(beam, e.shape[1])
            cost, idx = torch.topk(e, keep, dim=1, largest=False)
            back.append(idx.to(torch.int16))
            ctx = states.reshape(nt, -1).gather(1, idx) & 0x1FFF
        cur = torch.zeros((nt,), dtype=torch.int64, device=dev)         # best survivor after the last step
        for i, step in enumerate(range(0, 256)):
            idx = back[255 - step].to(torch.int64).gather(1, cur.unsqueeze(1)).squeeze(1)
            syms[c0:c0 + nt, step] = (idx & 7).to(torch.uint8)
            cur = idx >> 3
    # pack 256 x 3 bits little-endian: 8 symbols -> 3 bytes
    s = syms.to(torch.int64).reshape(n_tiles, 32, 8)
    word = sum(s[:, :, i] << (3 * i) for i in range(8))                 # 24 bits
    tile_bytes = torch.stack((word & 0xFF, (word >> 8) & 0xFF, (word >> 16) & 0xFF), dim=2).to(torch.uint8).reshape(n_tiles, 96)
    bits = in_neg.reshape(k // 8, 8).to(torch.int64)
    sign_bytes = sum(bits[:, i] << i for i in range(8)).to(torch.uint8)
    return torch.cat((tile_bytes.reshape(-1), scale16.view(torch.uint8).reshape(-1), sign_bytes))
