"""The allocation-free importance entry point against the regular one, through the C ABI.

`cafe_grad_importance_static` is for hosts that cannot allocate device memory while they run (their
own pool owns the device, or an allocation's device-wide stall is not acceptable mid-step): it keeps
its intermediates in a scratch array compiled into the library instead of a cudaMalloc'ed workspace.
The file sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _static_importance(lib, grad, F, B, D):
    import torch
    out = torch.empty(F * B, dtype=torch.float32, device=grad.device)
    rc = lib.cafe_grad_importance_static(grad.data_ptr(), D, F * D, F, B, D, out.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_static_scratch_matches_workspace_version_twice_in_a_row():
    import torch
    import cafe_b200
    lib = cafe_b200.load_library()
    F, B, D = 5, 777, 64
    sk = cafe_b200.HotSketch(1000, max_lookups=F * B)        # handle only for the regular entry point
    gen = torch.Generator(device="cuda").manual_seed(5)
    for call in range(2):                                     # second call reuses the scratch as the first left it
        grad = torch.randn(B, F, D, device="cuda", generator=gen) * (0.01 * (call + 1))
        want = torch.empty(F * B, dtype=torch.float32, device="cuda")
        rc = lib.cafe_grad_importance(sk.handle, grad.data_ptr(), D, F * D, F, B, D, want.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        rc, got = _static_importance(lib, grad, F, B, D)
        assert rc == 0
        torch.cuda.synchronize()
        np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), rtol=1e-5, atol=0)
        # and against the definition: norm * B / sum of the field's norms
        n = grad.permute(1, 0, 2).norm(dim=2)
        ref = (n * B / n.sum(dim=1, keepdim=True)).reshape(-1)
        np.testing.assert_allclose(got.cpu().numpy(), ref.cpu().numpy(), rtol=1e-5)


def test_static_scratch_rejects_what_does_not_fit():
    import torch
    import cafe_b200
    lib = cafe_b200.load_library()
    grad = torch.zeros(16, 1, 16, device="cuda")
    out = torch.zeros(16, device="cuda")
    too_many = (1 << 18) // 4 + 1
    rc = lib.cafe_grad_importance_static(grad.data_ptr(), 16, 16 * 4, 4, too_many, 16, out.data_ptr(), None)
    assert rc == 2                                            # CAFE_ERR_CAPACITY, nothing launched
    assert b"exceed" in lib.cafe_last_error()
    assert lib.cafe_grad_importance_static(grad.data_ptr(), 16, 16, 1, 16, 48, out.data_ptr(), None) == 6   # dim unsupported
    assert lib.cafe_grad_importance_static(None, 16, 16, 1, 16, 16, out.data_ptr(), None) == 1            # null input
    assert lib.cafe_grad_importance_static(grad.data_ptr(), 16, 16, 1, 0, 16, out.data_ptr(), None) == 0   # empty batch
