"""Mixture-of-experts layer (grouped Q4_K GEMM with on-device routing) against the CPU checker, through the C ABI.

The checker rounds the two intermediates to fp16 where the device stores them; what is left is the fp16
expansion of weights and activations inside the tensor-core GEMM (bar 1e-3 relative L2, as for the dense
GEMM) plus the fp16 activation the down projection consumes (the device rounds silu(g)*u once, the checker
rounds the same fp32 product: identical up to the expf implementation)."""
import numpy as np
import pytest
import torch

import oracle
import tattletale_b200 as ttq
from conftest import rel_l2
from gpu_util import make_weight, make_x, x_bits

pytestmark = pytest.mark.gpu
TOL = 1e-3


def build(ctx, n_exp, hidden, inter, top_k, max_tokens, seed):
    gu = [make_weight(ttq.FMT_Q4_K, 2 * inter, hidden, seed + 2 * e, std=0.05) for e in range(n_exp)]
    dn = [make_weight(ttq.FMT_Q4_K, hidden, inter, seed + 2 * e + 1, std=0.05) for e in range(n_exp)]
    layer = ttq.MoELayer(ctx, ttq.FMT_Q4_K, [torch.from_numpy(b) for b in gu], [torch.from_numpy(b) for b in dn],
                         hidden, inter, top_k, max_tokens)
    return layer, gu, dn


def routing(t, n_exp, top_k, seed, skew=False):
    rng = np.random.default_rng(seed)
    logits = rng.normal(0, 1, (t, n_exp))
    if skew:
        logits[:, 0] += 3.0  # most tokens pick expert 0: very uneven groups
    ids = np.argsort(-logits, axis=1)[:, :top_k].astype(np.int32)
    w = np.take_along_axis(logits, ids, axis=1)
    w = np.exp(w - w.max(axis=1, keepdims=True))
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    return ids, w


def check(ctx, layer, gu, dn, t, hidden, ids, w, seed, x_dtype=torch.bfloat16, y_dtype=torch.float32, tol=TOL):
    x = make_x(t, hidden, seed, x_dtype)
    y = torch.empty((t, hidden), dtype=y_dtype, device="cuda")
    layer.forward(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), out=y)
    ctx.check_device_status()
    want = oracle.moe(oracle.Q4_K, gu, dn, x_bits(x), oracle.BF16 if x_dtype == torch.bfloat16 else oracle.F16, ids, w)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_l2(got, want) < tol
    return got


@pytest.mark.parametrize("t,n_exp,top_k", [(40, 4, 2), (300, 8, 2), (64, 16, 4), (1, 4, 2), (700, 4, 1)])
def test_moe_matches_checker(ctx, t, n_exp, top_k):
    hidden, inter = 512, 256
    layer, gu, dn = build(ctx, n_exp, hidden, inter, top_k, max_tokens=1024, seed=9000 + t)
    ids, w = routing(t, n_exp, top_k, seed=t)
    check(ctx, layer, gu, dn, t, hidden, ids, w, seed=100 + t)
    layer.close()


def test_uneven_groups_and_empty_experts(ctx):
    hidden, inter, n_exp, top_k, t = 256, 512, 8, 2, 500
    layer, gu, dn = build(ctx, n_exp, hidden, inter, top_k, max_tokens=512, seed=9100)
    ids, w = routing(t, n_exp, top_k, seed=5, skew=True)
    ids[ids == 7] = 6  # expert 7 gets no token
    # a token must not name the same expert twice: repair collisions made by the edit above
    for r in range(t):
        if ids[r, 0] == ids[r, 1]:
            ids[r, 1] = (ids[r, 0] + 1) % 6
    assert not (ids == 7).any()
    check(ctx, layer, gu, dn, t, hidden, ids, w, seed=77)
    layer.close()


def test_dropped_choices_and_repeat_calls(ctx):
    """ids outside 0..E-1 contribute nothing (expert-parallel ranks skip foreign experts); a second call with
    other routing reuses the workspace; the same call twice gives the same bits."""
    hidden, inter, n_exp, top_k, t = 512, 256, 4, 2, 130
    layer, gu, dn = build(ctx, n_exp, hidden, inter, top_k, max_tokens=256, seed=9200)
    ids, w = routing(t, n_exp, top_k, seed=9)
    ids2 = ids.copy()
    ids2[ids2 >= 2] = -1
    a = check(ctx, layer, gu, dn, t, hidden, ids2, w, seed=78)
    b = check(ctx, layer, gu, dn, t, hidden, ids, w, seed=78)
    a2 = check(ctx, layer, gu, dn, t, hidden, ids2, w, seed=78)
    assert np.array_equal(a, a2)
    assert not np.array_equal(a, b)
    layer.close()


def test_output_types_and_f16_input(ctx):
    hidden, inter, n_exp, top_k, t = 256, 256, 4, 2, 90
    layer, gu, dn = build(ctx, n_exp, hidden, inter, top_k, max_tokens=128, seed=9300)
    ids, w = routing(t, n_exp, top_k, seed=11)
    check(ctx, layer, gu, dn, t, hidden, ids, w, seed=79, x_dtype=torch.float16, y_dtype=torch.float16, tol=2e-3)
    check(ctx, layer, gu, dn, t, hidden, ids, w, seed=80, y_dtype=torch.bfloat16, tol=6e-3)
    layer.close()


def test_argument_errors(ctx):
    hidden, inter = 256, 256
    layer, gu, dn = build(ctx, 2, hidden, inter, 1, max_tokens=16, seed=9400)
    x = make_x(32, hidden, 1).cuda()
    ids = torch.zeros((32, 1), dtype=torch.int32, device="cuda")
    w = torch.ones((32, 1), dtype=torch.float32, device="cuda")
    with pytest.raises(ttq.TtqError) as ei:
        layer.forward(x, ids, w)
    assert ei.value.status == 7  # beyond max_tokens
    layer.close()
    q8 = make_weight(ttq.FMT_Q8_0, 2 * inter, hidden, 1)
    with pytest.raises(ttq.TtqError):
        ttq.MoELayer(ctx, ttq.FMT_Q8_0, [torch.from_numpy(q8)], [torch.from_numpy(make_weight(ttq.FMT_Q8_0, hidden, inter, 2))],
                     hidden, inter, 1, 16)
