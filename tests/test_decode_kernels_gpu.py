"""Decode-step kernels around the linears (residual + RMSNorm, RoPE + KV append, single-query attention) against
plain fp32 torch references of the same operations.  Floating-point kernels: tolerances are the 16-bit
storage rounding (bf16 8 bits, f16 11 bits of mantissa)."""
import math

import pytest
import torch

import tattletale_b200 as ttq

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 6e-3), (torch.float16, 8e-4)])
@pytest.mark.parametrize("m,hid", [(1, 4096), (5, 1024), (32, 4096), (3, 264)])
def test_add_rmsnorm(ctx, dtype, tol, m, hid):
    g = torch.Generator(device="cuda").manual_seed(m + hid)
    h = torch.randn(m, hid, generator=g, device="cuda").to(dtype)
    d = torch.randn(m, hid, generator=g, device="cuda").to(dtype)
    w = (1 + 0.1 * torch.randn(hid, generator=g, device="cuda")).to(dtype)
    h_ref = (h.float() + d.float()).to(dtype)                      # the residual stream is stored in 16 bits
    want = torch.nn.functional.rms_norm(h_ref.float(), (hid,), w.float(), 1e-5)
    h2 = h.clone()
    out = ttq.add_rmsnorm(ctx, h2, d, w, 1e-5)
    assert torch.equal(h2, h_ref)
    assert rel(out, want) < tol
    # without a residual the stream is untouched
    h3 = h.clone()
    out = ttq.add_rmsnorm(ctx, h3, None, w, 1e-5)
    assert torch.equal(h3, h)
    assert rel(out, torch.nn.functional.rms_norm(h.float(), (hid,), w.float(), 1e-5)) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 6e-3), (torch.float16, 8e-4)])
def test_rope_kv_append(ctx, dtype, tol):
    b, hq, hkv, d, ctx_len, pos = 3, 8, 2, 128, 64, 17
    g = torch.Generator(device="cuda").manual_seed(5)
    qkv = torch.randn(b, (hq + 2 * hkv) * d, generator=g, device="cuda").to(dtype)
    inv = 1.0 / (500000.0 ** (torch.arange(0, d, 2, device="cuda", dtype=torch.float64) / d))
    ang = pos * inv
    cos = torch.cat([ang.cos(), ang.cos()]).to(dtype)
    sin = torch.cat([ang.sin(), ang.sin()]).to(dtype)
    kc = torch.zeros(b, hkv, ctx_len, d, device="cuda", dtype=dtype)
    vc = torch.zeros_like(kc)
    q = ttq.rope_kv_append(ctx, qkv, hq, hkv, d, cos, sin, kc, vc, pos)

    def rope(t):
        t = t.float()
        rot = torch.cat([-t[..., d // 2:], t[..., :d // 2]], dim=-1)
        return t * cos.float() + rot * sin.float()

    q_ref = rope(qkv[:, :hq * d].view(b, hq, d))
    k_ref = rope(qkv[:, hq * d:(hq + hkv) * d].view(b, hkv, d))
    v_ref = qkv[:, (hq + hkv) * d:].view(b, hkv, d)
    assert rel(q, q_ref) < tol
    assert rel(kc[:, :, pos], k_ref) < tol
    assert torch.equal(vc[:, :, pos], v_ref)
    kc[:, :, pos] = 0
    vc[:, :, pos] = 0
    assert not kc.any() and not vc.any()  # nothing else was written


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 6e-3), (torch.float16, 1e-3)])
@pytest.mark.parametrize("b,hq,hkv,n_ctx", [(1, 32, 8, 2048), (2, 8, 8, 130), (3, 16, 2, 1), (2, 4, 2, 128), (1, 8, 4, 777)])
def test_decode_attention(ctx, dtype, tol, b, hq, hkv, n_ctx):
    d, ctx_len = 128, max(n_ctx, 256)
    g = torch.Generator(device="cuda").manual_seed(b * 100 + n_ctx)
    q = torch.randn(b, hq, d, generator=g, device="cuda").to(dtype)
    kc = torch.randn(b, hkv, ctx_len, d, generator=g, device="cuda").to(dtype)
    vc = torch.randn(b, hkv, ctx_len, d, generator=g, device="cuda").to(dtype)
    out = ttq.decode_attention(ctx, q, kc, vc, n_ctx)
    grp = hq // hkv
    k = kc[:, :, :n_ctx].float().repeat_interleave(grp, dim=1)
    v = vc[:, :, :n_ctx].float().repeat_interleave(grp, dim=1)
    s = torch.einsum("bhd,bhpd->bhp", q.float(), k) / math.sqrt(d)
    want = torch.einsum("bhp,bhpd->bhd", torch.softmax(s, dim=-1), v)
    assert rel(out, want) < tol
    # positions beyond n_ctx are never read: poison them
    if n_ctx < ctx_len:
        kc[:, :, n_ctx:] = float("nan")
        vc[:, :, n_ctx:] = float("nan")
        assert torch.equal(ttq.decode_attention(ctx, q, kc, vc, n_ctx), out)


def test_argument_errors(ctx):
    q = torch.zeros(1, 6, 128, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(1, 4, 16, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ttq.TtqError):
        ttq.decode_attention(ctx, q, kc, kc, 8)       # 6 query heads over 4 kv heads
    q = torch.zeros(1, 4, 64, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(1, 4, 16, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ttq.TtqError):
        ttq.decode_attention(ctx, q, kc, kc, 8)       # head dimension other than 128
    h = torch.zeros(2, 100, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ttq.TtqError):
        ttq.add_rmsnorm(ctx, h, None, torch.ones(100, device="cuda", dtype=torch.bfloat16), 1e-5)  # H % 8
    # a V cache that is an 8-byte-offset view of a larger buffer: refused on the host, before any launch (the kernel
    # reads V rows as 16-byte vectors)
    q = torch.zeros(1, 4, 128, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(1, 4, 16, 128, device="cuda", dtype=torch.bfloat16)
    big = torch.zeros(4 * 16 * 128 + 8, device="cuda", dtype=torch.bfloat16)
    v_off = big[4:4 + 4 * 16 * 128].view(1, 4, 16, 128)
    assert v_off.data_ptr() % 16 == 8
    with pytest.raises(ttq.TtqError) as ei:
        ttq.decode_attention(ctx, q, kc, v_off, 8)
    assert ei.value.status == 1  # TTQ_ERR_INVALID_ARG


@pytest.mark.parametrize("fmt", [ttq.FMT_Q4_K, ttq.FMT_Q6_K, ttq.FMT_Q8_0])
@pytest.mark.parametrize("m", [1, 2])
def test_norm_prepares_the_linear_input(ctx, fmt, m):
    """add_rmsnorm(prepare=True) + forward_prepared gives, bit for bit, what add_rmsnorm + forward gives: the norm
    kernel writes the same fixed-point planes the linear's own conversion pass would make of its (rounded) output."""
    from tattletale_b200 import quantize as Q

    hid, n = 4096, 1536
    g = torch.Generator(device="cuda").manual_seed(31 + m)
    lin = ttq.QuantLinear(ctx, fmt, Q.quantize(fmt, torch.randn(n, hid, generator=g, device="cuda") * 0.02), hid,
                          bias=torch.randn(n, generator=g, device="cuda"))
    w = (1 + 0.1 * torch.randn(hid, generator=g, device="cuda")).to(torch.bfloat16)
    h0 = torch.randn(m, hid, generator=g, device="cuda").to(torch.bfloat16)
    delta = torch.randn(m, hid, generator=g, device="cuda").to(torch.bfloat16)
    h1, h2 = h0.clone(), h0.clone()
    x1 = ttq.add_rmsnorm(ctx, h1, delta, w, 1e-5)
    y1 = lin.forward(x1, out_dtype=torch.float32)
    x2 = ttq.add_rmsnorm(ctx, h2, delta, w, 1e-5, prepare=True)
    y2 = lin.forward_prepared(m, torch.float32)
    y2b = lin.forward_prepared(m, torch.float32)  # the prepared rows may be consumed more than once
    ctx.check_device_status()
    assert torch.equal(x1, x2) and torch.equal(h1, h2) and torch.equal(y2, y2b)
    assert torch.equal(y1, y2)
    lin.close()


def test_prepared_form_errors(ctx):
    from tattletale_b200 import quantize as Q

    hid = 512
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, Q.quantize(ttq.FMT_Q4_K, torch.randn(64, hid, device="cuda") * 0.02), hid)
    w = torch.ones(hid, dtype=torch.bfloat16, device="cuda")
    h = torch.randn(2, hid, device="cuda").to(torch.bfloat16)
    x = ttq.add_rmsnorm(ctx, h, None, w, 1e-5, prepare=True)
    with pytest.raises(ttq.TtqError):  # row count differs from the prepared rows
        lin.forward_prepared(1)
    lin.forward(x)  # rewrites the scratch: the prepared rows are gone
    with pytest.raises(ttq.TtqError):
        lin.forward_prepared(2)
    with pytest.raises(ttq.TtqError):  # hidden size not a multiple of 256
        ttq.add_rmsnorm(ctx, torch.zeros(1, 384, dtype=torch.bfloat16, device="cuda"), None,
                        torch.ones(384, dtype=torch.bfloat16, device="cuda"), 1e-5, prepare=True)
    with pytest.raises(ttq.TtqError):  # more rows than the prepared form serves
        ttq.add_rmsnorm(ctx, torch.zeros(3, hid, dtype=torch.bfloat16, device="cuda"), None, w, 1e-5, prepare=True)
    lin.close()
