"""The fused dot interaction (cafe_dot_interaction_forward / _backward, through the C ABI) against the reference's
formulation in plain PyTorch fp32 (cat, bmm, lower-triangle gather, cat: dlrm_s_pytorch.py:779-812).
Tolerance: rtol 1e-5, atol 1e-5 (dot products of up to 128 fp32 terms added in a different order)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference(x, emb, itself):
    import torch
    T = emb if x is None else torch.cat([x.unsqueeze(1), emb], dim=1)
    Z = torch.bmm(T, T.transpose(1, 2))
    n = T.shape[1]
    li, lj = torch.tril_indices(n, n, offset=0 if itself else -1, device=emb.device)
    flat = Z[:, li, lj]
    return flat if x is None else torch.cat([x, flat], dim=1)


def _library(x, emb, itself, grad_out=None):
    import torch
    from cafe_b200 import _lib
    lib = _lib.load()
    B, F, D = emb.shape
    nv = F + (0 if x is None else 1)
    width = (0 if x is None else D) + nv * (nv - 1 + 2 * itself) // 2
    out = torch.empty(B, width, device=emb.device)
    st = torch.cuda.current_stream().cuda_stream
    xp = None if x is None else x.data_ptr()
    _lib.check(lib.cafe_dot_interaction_forward(xp, emb.data_ptr(), D, F * D, B, F, D, itself, out.data_ptr(), width, st), "forward")
    if grad_out is None:
        return out
    gx = None if x is None else torch.empty_like(x)
    ge = torch.empty_like(emb)
    _lib.check(lib.cafe_dot_interaction_backward(xp, emb.data_ptr(), D, F * D, B, F, D, itself, grad_out.data_ptr(), width,
                                                 None if gx is None else gx.data_ptr(), ge.data_ptr(), D, F * D, st), "backward")
    return out, gx, ge


@pytest.mark.parametrize("B,F,D,dense,itself", [(128, 26, 16, True, 0), (2048, 26, 128, True, 0), (64, 26, 128, True, 1),
                                                (300, 22, 16, False, 0), (7, 3, 64, True, 1), (1, 1, 32, True, 0)])
def test_forward_and_backward_match_the_reference_formulation(B, F, D, dense, itself):
    import torch
    g = torch.Generator(device="cuda").manual_seed(B * 131 + F)
    emb = torch.randn(B, F, D, device="cuda", generator=g)
    x = torch.randn(B, D, device="cuda", generator=g) if dense else None
    embr = emb.clone().requires_grad_(True)
    xr = None if x is None else x.clone().requires_grad_(True)
    want = _reference(xr, embr, itself)
    go = torch.randn(want.shape, device="cuda", generator=g)
    want.backward(go)
    out, gx, ge = _library(x, emb, itself, go)
    torch.testing.assert_close(out, want.detach(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ge, embr.grad, rtol=1e-5, atol=1e-5)
    if dense:
        torch.testing.assert_close(gx, xr.grad, rtol=1e-5, atol=1e-5)


def test_autograd_function_in_the_harness_and_argument_checks():
    import torch
    from cafe_b200 import _lib
    from cafe_b200.dlrm_harness import dot_interaction, fused_dot_interaction
    g = torch.Generator(device="cuda").manual_seed(5)
    emb = torch.randn(96, 26, 16, device="cuda", generator=g, requires_grad=True)
    x = torch.randn(96, 16, device="cuda", generator=g, requires_grad=True)
    a = fused_dot_interaction(x, emb)
    b = dot_interaction(x, emb)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
    w = torch.randn(a.shape, device="cuda", generator=g)
    ga = torch.autograd.grad((a * w).sum(), [x, emb])
    gb = torch.autograd.grad((b * w).sum(), [x, emb])
    for u, v in zip(ga, gb):
        torch.testing.assert_close(u, v, rtol=1e-5, atol=1e-5)
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    out = torch.empty(4, 4000, device="cuda")
    e = torch.zeros(4, 70, 16, device="cuda")
    assert lib.cafe_dot_interaction_forward(None, e.data_ptr(), 16, 70 * 16, 4, 70, 16, 0, out.data_ptr(), 4000, st) == 1   # F + 1 > 64
    e = torch.zeros(4, 26, 16, device="cuda")
    assert lib.cafe_dot_interaction_forward(None, e.data_ptr(), 16, 26 * 16, 4, 26, 16, 0, out.data_ptr(), 10, st) == 1     # row too short
    assert lib.cafe_dot_interaction_forward(None, e.data_ptr(), 16, 26 * 16, 0, 26, 16, 0, None, 0, st) == 0                # empty batch
