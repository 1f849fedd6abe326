"""Worker of tests/test_gemm_gpu.py::test_gemm_forced_tiles: the tensor-core GEMM with its tile shape pinned by the
environment of this process (SM100_GEMM_TN tokens per tile, SM100_GEMM_RT row tiles of 128 weight rows per CTA,
SM100_GEMM_TMEM_A = 1 / 0 for dequantized weights staged in tensor memory / shared memory),
checked against the CPU oracle on ragged shapes.  Prints one JSON line {"worst": NMSE, "cases": n}."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import sgref  # noqa: E402
from scrapgpulibrary_b200 import capi  # noqa: E402
from tests import util as U  # noqa: E402


def main():
    capi.require_device()
    stream = capi.Stream(0)
    worst, cases = 0.0, 0
    # (dtype, layout, K, N, M): N below, at and above one and two row tiles; M across token tiles; K with a half chunk
    for dtype, layout, k, n, m in [(U.Q8_0, U.PACKED, 96, 130, 100), (U.Q8_0, U.NATURAL, 512, 300, 260), (U.Q4_0, U.PACKED, 160, 256, 129),
                                   (U.Q4_K, U.PACKED, 512, 257, 300), (U.F16, U.NATURAL, 64, 513, 33), (U.Q8_0, U.PACKED, 2048, 640, 64)]:
        wq = U.quantize(dtype, U.seeded_weights(3000 + dtype + k, n, k))
        x = U.seeded_acts(17 * m + k, m, k)
        want = sgref.mul_mat(dtype, wq, k, x)
        got = U.device_mul_mat(capi, stream, dtype, layout, wq, k, x)
        if not np.isfinite(got).all():
            worst = float("inf")
        worst = max(worst, float(sgref.nmse(got, want)), max(float(sgref.nmse(got[t], want[t])) / 4 for t in range(m)))
        cases += 1
    stream.close()
    print(json.dumps({"worst": worst, "cases": cases, "tn": os.environ.get("SM100_GEMM_TN"), "rt": os.environ.get("SM100_GEMM_RT")}))


if __name__ == "__main__":
    main()
