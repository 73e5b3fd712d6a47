"""GPU tests of the fused output-transform + all-reduce + residual kernel (rptc_peer_finish) that need
only one GPU: with a single rank it must equal the plain finish kernel, and a wait on a peer that never
shows up must run out after its time limit, raise the status word and leave the context usable."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_world1_equals_plain_finish():
    from rptc_b200 import ops
    from rptc_b200.linear import RPTCLinear
    from rptc_b200.tp import PeerAllReduce
    lin = RPTCLinear.random(2048, 4096, seed=1)
    g = torch.Generator(device="cuda").manual_seed(2)
    acc = torch.randn((2, 4096), device="cuda", generator=g) * 30
    h = torch.randn((2, 4096), device="cuda", generator=g).half()
    want = lin.finish(acc.clone(), residual=h.clone(), out=torch.empty_like(h))
    peer = PeerAllReduce(2, 4096, lin.block_out, 0, 1)
    for _ in range(3):                                  # epochs advance, buffers alternate
        a, hh = acc.clone(), h.clone()
        peer.finish(lin, a, hh)
        torch.cuda.synchronize()
        assert bool((a == 0).all())
        assert (hh.float() - want.float()).abs().max() <= 2e-3 * want.float().abs().max()
    ops.device_status()
    peer.close()


def test_wait_for_an_absent_peer_runs_out():
    from rptc_b200 import RPTCError, lib, ops
    from rptc_b200.linear import RPTCLinear
    from rptc_b200.tp import PeerAllReduce
    lin = RPTCLinear.random(2048, 1024, seed=3)
    # "world" of two whose second rank is a pair of buffers nobody ever writes
    peer = PeerAllReduce(1, 1024, lin.block_out, 0, 1, timeout_ms=50)
    # exchange buffers of [2 parities][2 ranks][1024 / 2] 64-bit (payload, epoch) words
    ghost_data = torch.zeros(2 * 2 * 512, dtype=torch.int64, device="cuda")
    own_data = torch.zeros(2 * 2 * 512, dtype=torch.int64, device="cuda")
    data = (ctypes.c_void_p * 2)(own_data.data_ptr(), ghost_data.data_ptr())
    flags = None                                         # the flags travel inside the data words
    acc = torch.ones((1, 1024), device="cuda")
    h = torch.zeros((1, 1024), dtype=torch.float16, device="cuda")
    st = lib().rptc_peer_finish(acc.data_ptr(), 1024, lin.signs_out.data_ptr(), 1.0, h.data_ptr(), 1024, data, flags,
                                peer.epochs.data_ptr(), 0, 2, 1, 1024, lin.block_out, 50, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    with pytest.raises(RPTCError) as e:
        ops.device_status()                              # synchronises; the kernel returned after ~50 ms
    assert e.value.status == -6
    ops.device_status()                                  # cleared; the context is still usable
    assert bool((h == 0).all())
    assert torch.ones(4, device="cuda").sum().item() == 4.0
    peer.close()
