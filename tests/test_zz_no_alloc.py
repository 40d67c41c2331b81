"""The no-allocation triangle multiplication entry point (lf_triangle_multiplication_run_static).

Some hosts cannot let a library allocate device memory while they run (the GPU was handed to the
host's own pool at start-up, or cudaMalloc's device-wide synchronisation is not acceptable in
steady state).  For them the library has one entry point whose scratch is a fixed array in the
library's device image.  This file checks, through the C ABI, that it gives what the regular entry
point gives - on two calls in a row, since the calls share that array and it keeps the previous
call's contents - and that it refuses lengths beyond the array.  It is collected last so that a
run that stops at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _desc(nat, n, incoming, z, mask, out, weights, residual=0, dtype=None):
    dtype = nat.DTYPE_F32 if dtype is None else dtype
    return nat.TriangleDesc(n, 128, 128, 1 if incoming else 0, nat.VARIANCE_TWO_PASS, nat.PRECISION_BF16, residual, 0, 1e-5,
                            nat.SPACE_DEVICE, dtype, z.data_ptr(), mask.data_ptr(), out.data_ptr(), weights.handle)


@pytest.mark.parametrize("n,incoming", [(96, False), (128, True), (75, False)])
def test_static_entry_point_matches_regular_one_twice(n, incoming):
    import torch
    import localfold_b200 as lf
    from localfold_b200 import _native as nat, synthetic as syn
    from localfold_b200.operators import prepare_triangle_weights

    dev = lf.Device(0)
    d = syn.draw(900 + n)
    weights = prepare_triangle_weights(dev, syn.af2_triangle_weights(d, 128, 128), 128, 128)
    results = []
    for call in range(2):                      # fresh inputs per call: the scratch holds the previous call's data
        z = torch.from_numpy(d.normal(n, n, 128)).cuda()
        mask = torch.from_numpy(syn.residue_pair_mask(n, 0.1)).cuda()
        want = torch.empty_like(z)
        got = torch.empty_like(z)
        res = nat.Result()
        dev.check(dev.lib.lf_triangle_multiplication_run(dev.handle, ctypes.byref(_desc(nat, n, incoming, z, mask, want, weights)),
                                                         ctypes.byref(res)))
        dev.synchronize()
        dev.check(dev.lib.lf_triangle_multiplication_run_static(dev.handle, ctypes.byref(_desc(nat, n, incoming, z, mask, got, weights)),
                                                                ctypes.byref(res)))
        dev.synchronize()
        assert res.launches == 3
        a, b = got.cpu().numpy().astype(np.float64), want.cpu().numpy().astype(np.float64)
        assert np.isfinite(a).all()
        # same kernels on the same inputs: the tolerance is the 16-bit path's own, the results are in fact equal
        assert np.linalg.norm(a - b) / np.linalg.norm(b) <= 8e-3
        np.testing.assert_array_equal(a, b)
        results.append(a)
    assert not np.array_equal(results[0], results[1])
    weights.close()
    dev.close()


@pytest.mark.parametrize("bf16_pair", [False, True])
def test_static_entry_point_in_place_residual_form(bf16_pair):
    """The form the block runners use - the update added into z, which is also the output buffer - with a
    float32 and with a bf16 pair tensor, bit for bit against the regular entry point, twice in a row."""
    import torch
    import localfold_b200 as lf
    from localfold_b200 import _native as nat, synthetic as syn
    from localfold_b200.operators import prepare_triangle_weights

    dev = lf.Device(0)
    n = 112
    d = syn.draw(950)
    weights = prepare_triangle_weights(dev, syn.af2_triangle_weights(d, 128, 128), 128, 128)
    dtype = nat.DTYPE_BF16 if bf16_pair else nat.DTYPE_F32
    for call in range(2):
        z0 = torch.from_numpy(d.normal(n, n, 128)).cuda()
        if bf16_pair:
            z0 = z0.to(torch.bfloat16)
        mask = torch.from_numpy(syn.residue_pair_mask(n, 0.1)).cuda()
        want, got = z0.clone(), z0.clone()
        res = nat.Result()
        dev.check(dev.lib.lf_triangle_multiplication_run(dev.handle, ctypes.byref(_desc(nat, n, call == 1, want, mask, want, weights, 1, dtype)),
                                                         ctypes.byref(res)))
        dev.synchronize()
        dev.check(dev.lib.lf_triangle_multiplication_run_static(dev.handle, ctypes.byref(_desc(nat, n, call == 1, got, mask, got, weights, 1, dtype)),
                                                                ctypes.byref(res)))
        dev.synchronize()
        assert bool(torch.isfinite(got.float()).all())
        assert not torch.equal(got, z0)                 # the update was added
        assert torch.equal(got, want)
    weights.close()
    dev.close()


def test_static_entry_point_refuses_what_it_cannot_hold():
    import torch
    import localfold_b200 as lf
    from localfold_b200 import _native as nat, synthetic as syn
    from localfold_b200.operators import prepare_triangle_weights

    dev = lf.Device(0)
    d = syn.draw(7)
    weights = prepare_triangle_weights(dev, syn.af2_triangle_weights(d, 128, 128), 128, 128)
    n = 129
    z = torch.zeros((n, n, 128), device="cuda")
    mask = torch.ones((n, n), device="cuda")
    out = torch.empty_like(z)
    status = dev.lib.lf_triangle_multiplication_run_static(dev.handle, ctypes.byref(_desc(nat, n, False, z, mask, out, weights)), None)
    assert status == nat.LF_ERR_UNSUPPORTED
    assert b"exceeds the static scratch" in dev.lib.lf_last_error(dev.handle)
    host = nat.TriangleDesc(8, 128, 128, 0, nat.VARIANCE_TWO_PASS, nat.PRECISION_BF16, 0, 0, 1e-5, nat.SPACE_HOST,
                            nat.DTYPE_F32, z.data_ptr(), mask.data_ptr(), out.data_ptr(), weights.handle)
    assert dev.lib.lf_triangle_multiplication_run_static(dev.handle, ctypes.byref(host), None) == nat.LF_ERR_ARGUMENT
    weights.close()
    dev.close()
