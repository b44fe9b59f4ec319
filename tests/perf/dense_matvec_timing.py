"""Dense quantised matvec sweep (the walk with K = all): Q4_K and Q8_0, shapes [1024 x 3072],
[2560 x 10240], [3840 x 15360] (hidden x rows), batch 1 / 8 / 32, through the host-pointer C-ABI
calls (activations up, outputs down, one synchronisation per call; weights resident after the first
call).  Weights are seeded N(0, 0.02) quantised by the CPU oracle's encoders (test infrastructure).
Prints microseconds per call and the weight bytes per second the call sustains."""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import larql_b200  # noqa: E402
import oracle  # noqa: E402

be = larql_b200.CudaBackend(0)
rng = np.random.Generator(np.random.PCG64(2))


def best(fn, reps=20):
    fn()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return min(ts)


for hidden, rows in [(1024, 3072), (2560, 10240), (3840, 15360)]:
    w = rng.standard_normal((rows, hidden), dtype=np.float32) * np.float32(0.02)
    q4 = oracle.quantize_matrix(oracle.FMT_Q4_K, w)
    q8 = oracle.quantize_matrix(oracle.FMT_Q8_0, w)
    for batch in (1, 8, 32):
        x = rng.standard_normal((batch, hidden), dtype=np.float32)
        if batch == 1:
            t4 = best(lambda: be.q4k_matvec(q4.data, x[0], rows, hidden))
            t8 = best(lambda: be.q8_0_gemv(q8.data, x[0], rows, hidden))
        else:
            t4 = best(lambda: be.q4k_matmul(q4.data, x, rows, hidden, batch))
            t8 = best(lambda: [be.q8_0_gemv(q8.data, x[b], rows, hidden) for b in range(batch)])  # gemv only, as the trait
        print(f"[{hidden} x {rows}] batch {batch:2d}: Q4_K {t4 * 1e6:8.1f} us ({q4.nbytes / t4 / 1e9:7.1f} GB/s weights)   "
              f"Q8_0 {t8 * 1e6:8.1f} us ({q8.nbytes * (1 if batch == 1 else batch) / t8 / 1e9:7.1f} GB/s)")
    be.drop_weight_regions()
