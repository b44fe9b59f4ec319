"""The allocation-free Q4_K matvec entry point (lq_q4k_matvec_static), through the C ABI.

It serves callers that must not allocate device memory while running (all HBM already in their
own pools, a framework allocator that forbids raw cudaMalloc, or no tolerance for cudaMalloc's
device-wide synchronisation): its scratch is a fixed array inside the library image.  The check
is against the regular entry point (lq_dev_q4k_matvec), which runs the same kernels over a
context-owned workspace: outputs must agree to the tolerance the other tests use (they are in
fact bit-identical), on two calls in a row that reuse the shared scratch with different sizes.

Collected last on purpose: a failure here cannot hide the results of the other GPU tests.
"""
import numpy as np
import pytest

import oracle
from conftest import bits, rel_l2, seeded_weights, seeded_x

pytestmark = pytest.mark.gpu


def test_static_matvec_matches_regular_entry_point_twice():
    import torch

    import larql_b200

    be = larql_b200.CudaBackend(0)
    dev = torch.device("cuda", 0)
    try:
        # second call is smaller than the first: stale scratch from call one must not leak in
        for rows, cols, seed in [(1000, 8192, 11), (333, 2560, 12)]:
            m = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(seed, rows, cols))
            x = seeded_x(seed + 100, cols)
            w_d = torch.from_numpy(m.data.copy()).to(dev)
            x_d = torch.from_numpy(x).to(dev)
            out_ref = torch.empty(rows, dtype=torch.float32, device=dev)
            out_new = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
            torch.cuda.synchronize()
            assert be.dev_q4k_matvec(w_d.data_ptr(), w_d.numel(), x_d.data_ptr(), rows, cols, out_ref.data_ptr())
            be.synchronize()
            rc, msg = larql_b200.q4k_matvec_static(w_d.data_ptr(), w_d.numel(), x_d.data_ptr(), rows, cols,
                                                   out_new.data_ptr())
            assert rc == 0, msg
            a, b = out_new.cpu().numpy(), out_ref.cpu().numpy()
            assert rel_l2(a, b) < 1e-4
            assert np.array_equal(bits(a), bits(b))
            # and both agree with the CPU oracle within the fast path's tolerance
            assert rel_l2(a, oracle.q4k_matvec(m.data, x, rows, cols)) < 1e-4
        # sizes beyond the static scratch are refused with a reason, not attempted
        rc, msg = larql_b200.q4k_matvec_static(w_d.data_ptr(), 1 << 40, x_d.data_ptr(), 4, 16384 + 256,
                                               out_new.data_ptr())
        assert rc == larql_b200.LQ_REFUSED_UNSUPPORTED and "16384" in msg
        rc, msg = larql_b200.q4k_matvec_static(w_d.data_ptr(), w_d.numel(), x_d.data_ptr(), 4, 200, out_new.data_ptr())
        assert rc == larql_b200.LQ_REFUSED_SHAPE
    finally:
        be.close()
