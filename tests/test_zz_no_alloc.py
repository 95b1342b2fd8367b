"""The allocation-free attention-backward entry point, called through its exported C
symbol exactly as a host that cannot allocate device memory would call it (raw pointers
in, nothing allocated by the library), must reproduce the regular entry point. Two calls
in a row check that the built-in scratch carries nothing over from one call to the next.
Both entry points launch the same kernels, so the comparison is exact; agreement with the
fp32 PyTorch oracle follows from `test_gpu_attention.py`, which checks the regular entry
point against it. The test also reads the path's own status word (it must be 0) and checks
that the second call left the device's free memory untouched.
This file sorts last so a run that stops at the first failure has already run the rest."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _strides(t):
    return (ctypes.c_long * 3)(t.stride(0), t.stride(1), t.stride(2))


def test_noalloc_attention_backward_matches_regular_entry_twice():
    from summa_b200.ops import cuda_ops, native
    lib = native.lib()
    f = lib.sb_attention_bwd_noalloc
    P, I = ctypes.c_void_p, ctypes.c_int
    f.argtypes = [P] * 9 + [I] * 6 + [P] * 8 + [I, I, I, ctypes.c_float, P]
    f.restype = I
    lib.sb_set_device.argtypes = [I]
    lib.sb_set_device.restype = I
    assert lib.sb_set_device(torch.cuda.current_device()) == 0
    status = lib.sb_attention_bwd_noalloc_status
    status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
    status.restype = I
    for call, (B, S, Hq, Hkv, D, causal) in enumerate([(2, 384, 4, 2, 64, True), (1, 300, 2, 2, 128, True)]):
        torch.manual_seed(call)
        q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
        k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
        v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
        o, lse = cuda_ops.attention_fwd(q, k, v, causal)
        do = torch.randn_like(o)
        ref = [torch.empty_like(t) for t in (q, k, v)]
        cuda_ops.attention_bwd(q, k, v, o, do, lse, ref[0], ref[1], ref[2], causal, None, 0)
        got = [torch.full_like(t, float("nan")) for t in (q, k, v)]
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = f(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
               got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(), B, Hq, Hkv, S, S, D,
               _strides(q), _strides(k), _strides(v), _strides(o), _strides(do),
               _strides(got[0]), _strides(got[1]), _strides(got[2]), 1 if causal else 0, -1, 0,
               float(D) ** -0.5, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        word = ctypes.c_uint(123)
        assert status(ctypes.byref(word)) == 0          # synchronises
        assert word.value == 0, "a bounded wait inside the kernels gave up"
        if call > 0:        # the first call may load the kernels' module; after that nothing may change
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, (free_before, free_after)
        for a, b in zip(got, ref):
            assert torch.equal(a, b)
    # beyond the built-in capacity the call is refused, not attempted
    big = 1 << 21
    rc = f(None, None, None, None, None, None, None, None, None, 1, 1, 1, big, 128, 64,
           _strides(q), _strides(k), _strides(v), _strides(o), _strides(do), _strides(q), _strides(k), _strides(v),
           1, -1, 0, 0.125, torch.cuda.current_stream().cuda_stream)
    assert rc == -4
    # a head count that would wrap a 64-bit product is refused as well, not misjudged as small
    rc = f(None, None, None, None, None, None, None, None, None, 65535, 2 ** 31 - 1, 1, 2 ** 31 - 64, 128, 64,
           _strides(q), _strides(k), _strides(v), _strides(o), _strides(do), _strides(q), _strides(k), _strides(v),
           1, -1, 0, 0.125, torch.cuda.current_stream().cuda_stream)
    assert rc in (-4, -1)
