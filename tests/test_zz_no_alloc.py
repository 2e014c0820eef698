"""ttq_linear_forward_static: the decode linear for hosts that may not allocate device memory.

Some hosts cannot call cudaMalloc -- a server whose own pool already owns all device memory, or a
plug-in that is forbidden to allocate after start-up -- and therefore cannot create a library context
(its creation allocates scratch).  The entry point tested here takes no context and keeps its scratch
in a fixed array inside the library.  It must give the same result as the regular entry point, also on
a second call in a row, because every call reuses that one array with the previous call's contents
still in it.  This file is collected last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
import tattletale_b200 as ttq
from conftest import rel_l2
from gpu_util import OFMT, make_weight, make_x, x_bits
from tattletale_b200 import _lib

pytestmark = pytest.mark.gpu
TOL = 1e-3  # same bar as the other linear tests


def static_forward(lin, x, bias=None):
    """Calls the allocation-free entry point through the C ABI (no context argument)."""
    lib = _lib.load()
    y = torch.empty((x.shape[0], lin.out_features), dtype=torch.float32, device=x.device)
    err = ctypes.create_string_buffer(256)
    st = lib.ttq_linear_forward_static(
        lin.handle, x.data_ptr(), _lib.DT_BF16, x.shape[0], x.stride(0), None if bias is None else bias.data_ptr(),
        _lib.DT_F32, y.data_ptr(), _lib.DT_F32, y.stride(0), torch.cuda.current_stream().cuda_stream, err, 256)
    return st, err.value.decode(), y


def static_status():
    """The allocation-free status check: 0, or 8 (TTQ_ERR_TIMEOUT) if a kernel of an earlier call gave up a wait."""
    err = ctypes.create_string_buffer(256)
    return _lib.load().ttq_static_status(torch.cuda.current_stream().cuda_stream, err, 256)


@pytest.mark.parametrize("fmt", [ttq.FMT_Q4_K, ttq.FMT_Q8_0, ttq.FMT_Q6_K], ids=["q4_k", "q8_0", "q6_k"])
def test_two_calls_in_a_row_match_the_regular_entry_point(ctx, fmt):
    n, k = 192, 2048
    blocks = make_weight(fmt, n, k, seed=600)
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), k)
    bias = torch.from_numpy(np.random.default_rng(601).normal(0, 0.1, n).astype(np.float32)).cuda()
    # second call: fewer rows and other values, so stale planes of the first call are still in the array
    for m, seed, b in ((4, 610, None), (1, 611, bias)):
        x = make_x(m, k, seed).cuda()
        lin.bias = b
        want = lin.forward(x, out_dtype=torch.float32)
        st, msg, got = static_forward(lin, x, b)
        assert st == 0, msg
        torch.cuda.synchronize()
        assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < TOL
        if fmt != ttq.FMT_Q4_K or m <= 2:
            assert torch.equal(got, want)  # same kernels, same arithmetic: expected to agree exactly
        # and against the CPU checker, not only against the library's other entry point
        ref = oracle.linear(OFMT[fmt], blocks, x_bits(x.cpu()), oracle.BF16, None if b is None else b.cpu().numpy())
        assert rel_l2(got.cpu().numpy(), ref) < TOL
        assert static_status() == 0  # no kernel of the call gave up a bounded wait
    lin.bias = None
    lin.close()


def test_large_k_reads_planes_from_the_array(ctx):
    """K = 14336 with 4 rows does not fit shared memory: the kernel reads its fragments from the array."""
    n, k = 64, 14336
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, torch.from_numpy(make_weight(ttq.FMT_Q4_K, n, k, seed=620)), k)
    for m, seed in ((4, 621), (3, 622)):
        x = make_x(m, k, seed).cuda()
        want = lin.forward(x, out_dtype=torch.float32)
        st, msg, got = static_forward(lin, x)
        assert st == 0, msg
        torch.cuda.synchronize()
        assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < TOL
        assert static_status() == 0
    lin.close()


def test_sizes_beyond_the_fixed_array_are_rejected(ctx):
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, torch.from_numpy(make_weight(ttq.FMT_Q4_K, 16, 256, seed=630)), 256)
    st, msg, _ = static_forward(lin, torch.zeros(5, 256, dtype=torch.bfloat16, device="cuda"))
    assert st == 7 and "M <= 4" in msg  # TTQ_ERR_LIMIT
    lin.close()
    big = ttq.QuantLinear(ctx, ttq.FMT_Q8_0, torch.from_numpy(make_weight(ttq.FMT_Q8_0, 16, 16640, seed=631)), 16640)
    st, msg, _ = static_forward(big, torch.zeros(1, 16640, dtype=torch.bfloat16, device="cuda"))
    assert st == 7 and "16384" in msg
    big.close()
    lib = _lib.load()
    assert lib.ttq_linear_forward_static(None, None, 0, 1, 1, None, 0, None, 2, 1, None, None, 0) == 1
