"""The bounded peer-flag wait of the fused kernels, exercised alone: a flag that nothing sets
makes the wait run out after its (short) limit, the kernel returns with an error status that the
host reads, and the CUDA context keeps working."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_context_survives():
    from summa_b200 import ops
    from summa_b200.ops import native
    from summa_b200.parallel.health import device_wait_status
    native.register("sb_wait_probe", [native.P, ctypes.c_uint, native.L, native.P, native.P])
    device_wait_status()                                     # clear whatever earlier tests left
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    native.call("sb_wait_probe", flag.data_ptr(), 1, 300_000_000, gave_up.data_ptr(), native.stream())   # ~0.15 s of SM clock
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    st = device_wait_status()
    assert st["peer_wait_timeout"] and not st["mbarrier_timeout"] and int(gave_up.item()) == 1
    assert device_wait_status()["word"] == 0                 # reading clears the word
    # the context is intact: a tensor-core GEMM still runs and is correct
    x = torch.randn(256, 256, device="cuda").to(torch.bfloat16)
    w = torch.randn(256, 256, device="cuda").to(torch.bfloat16)
    torch.testing.assert_close(ops.linear(x, w, None).float(), x.float() @ w.float(), rtol=2e-2, atol=0.5)
    # a flag that is already there lets the wait through at once
    flag.fill_(1)
    native.call("sb_wait_probe", flag.data_ptr(), 1, 300_000_000, gave_up.data_ptr(), native.stream())
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 0 and device_wait_status()["word"] == 0
