"""Times one layer's walk per weight format at the Llama-3-70B shape (hidden 8192, 28672 features,
K = 4096, batch 1) through the host-pointer C-ABI call.  Weights are seeded N(0, 0.02), quantised by
the CPU oracle's encoders (test infrastructure); gate, up and down share one matrix, which does not
change the timing.  Usage: python tests/perf/format_walk_timing.py [features]"""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import larql_b200  # noqa: E402
import oracle  # noqa: E402

H, N, K = 8192, 28672, 4096
if len(sys.argv) > 1:
    N = int(sys.argv[1])
be = larql_b200.CudaBackend(0)
rng = np.random.Generator(np.random.PCG64(1))
w = rng.standard_normal((N, H), dtype=np.float32) * np.float32(0.02)
x = oracle.rms_norm(rng.standard_normal(H, dtype=np.float32))
names = {oracle.FMT_Q4_K: "q4_k", oracle.FMT_Q8_0: "q8_0", oracle.FMT_MXFP4: "mxfp4", oracle.FMT_NVFP4: "nvfp4"}
for fmt in (oracle.FMT_Q4_K, oracle.FMT_Q8_0, oracle.FMT_MXFP4, oracle.FMT_NVFP4):
    m = oracle.quantize_matrix(fmt, w)
    hm = larql_b200.HostMatrix(m.fmt, m.rows, m.cols, m.data, m.scales, float(m.tensor_scale))
    be.walk_ffn(hm, hm, hm, x, K, larql_b200.WALK_FORCE_SPARSE)  # upload + warm-up
    ts = []
    for _ in range(5):
        t0 = time.perf_counter()
        be.walk_ffn(hm, hm, hm, x, K, larql_b200.WALK_FORCE_SPARSE)
        ts.append(time.perf_counter() - t0)
    st = be.last_walk_stats()
    print(f"{names[fmt]:6s} lq_walk_ffn host call {min(ts) * 1e6:7.1f} us   band rows {st.n_band}")
    be.drop_weight_regions()
