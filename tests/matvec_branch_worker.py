"""Worker of tests/test_matvec_gpu.py::test_matvec_forced_branches: the decode matvec with its dispatcher pinned by the
environment of this process (SM100_Q4K_RING, SM100_Q4K_IMMA, SM100_Q4K_MMA, SM100_B32_IMMA, SM100_Q6K_IMMA, SM100_MV_WIDE = 0 switch the
respective kernel family off, so the next one in the chain serves the call), checked against the CPU oracle on ragged
and benchmark-like shapes.  The library reports the kernel family that served each call
(sm100_matvec_last_kernel); the worker prints one JSON line {"worst": NMSE, "kernels": {name: calls}}."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import sgref  # noqa: E402
from scrapgpulibrary_b200 import capi  # noqa: E402
from tests import util as U  # noqa: E402

# (dtype, K, N, M): whole tiles and leftover rows, short and long rows, one and several columns
CASES = [(U.Q4_K, 4096, 272, 1), (U.Q4_K, 4096, 264, 2), (U.Q4_K, 2048, 40, 4), (U.Q4_K, 12288, 48, 1), (U.Q4_K, 512, 33, 8),
         (U.Q4_K, 1024, 40, 1), (U.Q4_K, 4096, 64, 2), (U.Q4_K, 6144, 4112, 1), (U.Q4_K, 768, 9616, 1), (U.Q4_K, 16384, 32, 1), (U.Q4_K, 4096, 24016, 1),
         (U.Q6_K, 4096, 272, 1), (U.Q6_K, 2048, 40, 1), (U.Q6_K, 12288, 528, 1), (U.Q6_K, 4096, 64, 4), (U.Q6_K, 768, 24, 1), (U.Q6_K, 768, 8, 2),
         (U.Q4_0, 4096, 272, 1), (U.Q4_0, 2048, 33, 1), (U.Q4_0, 4096, 64, 3), (U.Q4_0, 96, 24, 1),
         (U.Q8_0, 4096, 272, 1), (U.Q8_0, 1024, 40, 1), (U.Q8_0, 4096, 64, 8), (U.Q8_0, 160, 17, 1), (U.Q8_0, 160, 17, 3)]


def main():
    capi.require_device()
    L = capi.lib()
    stream = capi.Stream(0)
    worst, kernels = 0.0, {}
    for dtype, k, n, m in CASES:
        wq = U.quantize(dtype, U.seeded_weights(5000 + dtype + k + n, n, k))
        x = U.seeded_acts(13 * m + k + n, m, k)
        want = sgref.mul_mat(dtype, wq, k, x)
        got = U.device_mul_mat(capi, stream, dtype, U.PACKED, wq, k, x)
        name = (L.sm100_matvec_last_kernel() or b"").decode()
        key = f"{U.NAMES[dtype]}:{name}"
        kernels[key] = kernels.get(key, 0) + 1
        e = float(sgref.nmse(got, want)) if np.isfinite(got).all() else float("inf")
        rows = max(float(sgref.nmse(got[:, r], want[:, r])) for r in (0, n // 2, n - 1))   # first, middle and last row on their own
        worst = max(worst, e, rows / 4)
    stream.close()
    print(json.dumps({"worst": worst, "kernels": kernels}))


if __name__ == "__main__":
    main()
