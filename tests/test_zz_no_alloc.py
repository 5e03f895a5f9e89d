"""GPU test of tnn_l2_loss_static, the L2 loss for callers that must not allocate device memory (a plug-in
whose host application owns all free device memory, or a loop that cannot afford an allocation's
device-wide synchronisation).  Its scratch is a fixed array inside the library, shared by all calls, so the
test runs it twice in a row and compares each result with the allocating entry point tnn_l2_loss.
Collected last on purpose: a failure here must not hide the other tests in a run that stops at the first
failure."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _reference(tnn_lib, pred, target):
    loss_sum, grads, values = tnn_lib.l2_loss(pred, target, 1.0, want_values=True)
    return loss_sum.clone(), grads.clone(), values.clone()


def test_static_scratch_l2_loss_matches_allocating_entry_point_twice(tnn_lib):
    gen = torch.Generator(device="cuda").manual_seed(11)
    # two different problems back to back: the second call finds the first call's partial sums in the array
    for batch, stride, n_targets in ((1 << 16, 64, 64), (8192 + 8, 32, 3)):
        pred = (torch.rand((batch, stride), device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
        target = torch.rand((batch, n_targets), device="cuda", generator=gen) * 2 - 1
        ref_sum, ref_grads, ref_values = _reference(tnn_lib, pred, target)
        # every output buffer is the caller's
        loss_sum = torch.zeros(1, dtype=torch.float32, device="cuda")
        grads = torch.empty_like(pred)
        values = torch.empty((batch, stride), dtype=torch.float32, device="cuda")
        tnn_lib.l2_loss_static(pred, target, loss_sum, grads, values)
        torch.cuda.synchronize()
        assert torch.equal(grads, ref_grads)      # element-wise results are the same kernel: same bits
        assert torch.equal(values, ref_values)
        # the sum is taken over a different number of partials, so only the order of additions differs
        assert abs(loss_sum.item() - ref_sum.item()) <= 1e-5 * abs(ref_sum.item())
        assert abs(loss_sum.item() - values.double().sum().item()) <= 1e-5 * abs(ref_sum.item())


def test_static_scratch_l2_loss_rejects_oversize_input(tnn_lib):
    import ctypes

    lib = tnn_lib.load()
    dummy = torch.zeros(16, device="cuda")
    p = ctypes.c_void_p(dummy.data_ptr())
    # 2^27 + 64 elements: beyond the fixed scratch capacity; rejected before anything is launched
    rc = lib.tnn_l2_loss_static(p, p, 64, None, None, (1 << 21) + 1, 64, 1.0, None, None)
    assert rc != 0
    assert b"exceeds the capacity" in lib.tnn_last_error()
