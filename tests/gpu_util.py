"""Helpers shared by the GPU parity tests."""
import numpy as np

# Parity bar of the path (north star): against fp32-or-wider accumulated attention on the same fp16 inputs.
TOL_O_MAXABS = 2e-3
TOL_O_RELL2 = 1e-3
TOL_LSE = 1e-4


def to_dev(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def assert_parity(got_o, got_lse, want_o, want_lse, what=""):
    got_o, got_lse = np.asarray(got_o, np.float32), np.asarray(got_lse, np.float32)
    assert not np.isnan(got_o).any(), f"{what}: NaN in O"
    fin = np.isfinite(want_lse)
    assert np.array_equal(np.isneginf(got_lse), np.isneginf(want_lse)), f"{what}: -inf LSE pattern differs"
    err_o = float(np.abs(got_o - want_o).max())
    rel = float(np.linalg.norm(got_o - want_o) / max(np.linalg.norm(want_o), 1e-30))
    err_l = float(np.abs(got_lse[fin] - want_lse[fin]).max()) if fin.any() else 0.0
    assert err_o <= TOL_O_MAXABS, f"{what}: max|dO| = {err_o:.3e}"
    assert rel <= TOL_O_RELL2, f"{what}: rel-L2(O) = {rel:.3e}"
    assert err_l <= TOL_LSE, f"{what}: max|dLSE| = {err_l:.3e}"
    return err_o, rel, err_l
