"""A bounded device-side wait that runs out is reported, and the context stays usable (failure detection without
any GPU fault: the wait is on a counter that nothing sets).

A two-rank exchange is set up on ONE GPU: rank 0's communicator is connected, by plain device pointers, to a
second zeroed buffer that stands for a peer which never arrives.  The row-parallel linear pushes its partial
sums, polls the absent peer's counter for the configured number of polls (made short here), gives up, sets
status bit 2 and finishes; the host reads TTQ_ERR_TIMEOUT from ttq_device_status, and the next ordinary call
works.  No NVLink multicast, no second process, no trap, no endless loop."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
import tattletale_b200 as ttq
from conftest import rel_l2
from gpu_util import make_weight, make_x, x_bits
from tattletale_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [1, 5])  # integer decode kernel, fp16 tensor-core kernel
def test_absent_peer_times_out_and_context_recovers(ctx, m):
    lib = ctx._lib
    n, k = 256, 1024
    blocks = make_weight(ttq.FMT_Q4_K, n, k, seed=800)
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, torch.from_numpy(blocks), k)
    comm = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    _lib.check(ctx.handle, lib.ttq_comm_create(ctx.handle, 0, 2, n, 16, ctypes.byref(comm), handle))
    base, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
    _lib.check(ctx.handle, lib.ttq_comm_local_buffer(comm, ctypes.byref(base), ctypes.byref(nbytes)))
    fake_peer = torch.zeros(nbytes.value + 256, dtype=torch.uint8, device="cuda")
    fake_ptr = (fake_peer.data_ptr() + 255) & ~255
    bases = (ctypes.c_void_p * 2)(base.value, fake_ptr)
    _lib.check(ctx.handle, lib.ttq_comm_connect_pointers(comm, bases))
    _lib.check(ctx.handle, lib.ttq_comm_set_wait_limit(comm, 2000))
    x = make_x(m, k, 801).cuda()
    y = torch.empty(m, n, dtype=torch.float32, device="cuda")
    st = lib.ttq_linear_forward_allreduce(ctx.handle, lin.handle, x.data_ptr(), _lib.DT_BF16, m, k, None, _lib.DT_F32,
                                          y.data_ptr(), _lib.DT_F32, n, comm, torch.cuda.current_stream().cuda_stream)
    assert st == 0  # the launch itself succeeds; the give-up happens on the device
    with pytest.raises(ttq.TtqError) as ei:
        ctx.check_device_status()
    assert ei.value.status == 8  # TTQ_ERR_TIMEOUT
    ctx.check_device_status()  # the flag was cleared by the read
    # the kernel returned, the context works: an ordinary call gives the right answer
    got = lin.forward(x, out_dtype=torch.float32).cpu().numpy()
    ctx.check_device_status()
    assert rel_l2(got, oracle.linear(oracle.Q4_K, blocks, x_bits(x.cpu()), oracle.BF16)) < 1e-3
    lib.ttq_comm_destroy(comm)
    lin.close()


def test_wait_limit_argument_is_checked(ctx):
    lib = ctx._lib
    comm = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    _lib.check(ctx.handle, lib.ttq_comm_create(ctx.handle, 0, 2, 64, 4, ctypes.byref(comm), handle))
    assert lib.ttq_comm_set_wait_limit(comm, 0) == 1
    assert lib.ttq_comm_connect_pointers(comm, None) == 1
    lib.ttq_comm_destroy(comm)
