"""Child process of tests/test_plugin_gpu.py::test_profile_table: a few ops and a plan on cuda_sm100 with
SCRAPGPU_SM100_PROFILE=1 set before the plugin loads; prints the per-op-key table the backend collected."""
import ctypes as C
import sys

import numpy as np

from scrapgpulibrary_b200 import abi
from tests import refsession
from tests import util as U


def main() -> int:
    gpu = refsession.Session("cuda_sm100")
    k, n = 1024, 512
    w = gpu.tensor(abi.Q4_K, [k, n], layout=abi.LAYOUT_R32).upload(U.quantize(U.Q4_K, U.seeded_weights(1, n, k)))
    x = gpu.tensor(abi.F32, [k]).upload(np.random.default_rng(2).standard_normal(k).astype(np.float32))
    y = gpu.tensor(abi.F32, [n]).upload(np.zeros(n, np.float32))
    z = gpu.tensor(abi.F32, [n]).upload(np.zeros(n, np.float32))
    for _ in range(3):
        gpu.execute(abi.OP_MUL_MAT, [w, x], [y], abi.MulMatParams())
    gpu.execute(abi.OP_ADD, [y, y], [z])
    gpu.sync()
    plug = refsession.plugin()
    plug.scrapgpu_cuda_sm100_profile_report.restype = C.c_size_t
    plug.scrapgpu_cuda_sm100_profile_report.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
    need = plug.scrapgpu_cuda_sm100_profile_report(gpu.stream, None, 0)
    buf = C.create_string_buffer(max(1, need))
    plug.scrapgpu_cuda_sm100_profile_report(gpu.stream, buf, need)
    sys.stdout.write(buf.value.decode())
    got = y.download(np.float32, n)
    print("RESULT_SUM", float(np.abs(got).sum()) > 0.0)
    gpu.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
