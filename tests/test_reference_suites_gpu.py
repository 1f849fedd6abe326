"""The reference's OWN device test programs, compiled byte-for-byte unchanged, run against the cuda_sm100 plugin.

tests/ops/ops_tests.cpp of the reference runs every op its backend reports as supported on the device and compares it
with scrapgpu_ref_execute (NMSE 1e-7, 1e-6 for quantized MUL_MAT, exact for GET_ROWS / SET_ROWS / CPY:
ops_tests.cpp:411-412,725,588-603); tests/attention/attention_tests.cpp checks the core's SDPA composition on the
device against a double-precision oracle (3e-4 absolute, attention_tests.cpp:40).  Both select their GPU backend by
the literal name "opencl11" under -DSCRAPGPU_*_TEST_WITH_OPENCL11 (ops_tests.cpp:1222-1236,
attention_tests.cpp:433-459); oracle/Makefile (`device_tests`) compiles them where they lie and links the one-function
shim backend/opencl11_register_shim.c, so that name registers cuda_sm100.  The programs print PASS / SKIP per case and
exit 0 only if nothing failed; SKIP lines are ops this backend reports UNSUPPORTED (outside the decode hot path)."""
import os
import re
import subprocess

import pytest

from oracle import refapi

pytestmark = pytest.mark.gpu

# ops of the decode hot path: none of their cases may be skipped
HOT_PATH = ("ADD", "SUB", "MUL", "DIV", "SCALE", "CLAMP", "SQR", "SQRT", "GLU", "RMS_NORM", "RMS_NORM_MUL", "ADD_RMS_NORM_MUL", "SOFT_MAX", "ROPE",
            "GET_ROWS", "SET_ROWS", "SET_ROWS_PAIR", "CPY", "DUP", "CONT", "MUL_MAT", "MUL_MAT_MULTI", "CONT_MUL_MAT")
# what this backend leaves UNSUPPORTED on purpose: the mixture-of-experts, state-space and shape-juggling ops that a
# dense decode step never issues, and full sorts (greedy decoding needs TOP_K with k = 1 only)
OUTSIDE = ("MUL_MAT_ID", "ADD_ID", "SSM_CONV", "CONCAT", "PAD", "SUM_ROWS", "ARGSORT", "TOP_K", "tensor_copy")


def run(binary, backend="opencl11"):
    if not os.path.exists(binary):
        pytest.fail(f"{binary} is missing on the GPU box: run `make -C oracle device_tests remote_tests` where the reference is checked out")
    env = dict(os.environ, SCRAPGPU_TEST_BACKEND=backend)
    r = subprocess.run([binary], capture_output=True, text=True, timeout=600, env=env)
    print(r.stdout)
    print(r.stderr)
    assert r.returncode == 0, f"exit {r.returncode} (77 = no device)\n" + r.stdout[-4000:] + r.stderr[-2000:]
    return r.stdout


def test_reference_ops_tests_pass_on_cuda_sm100():
    out = run(refapi.OPS_TESTS)
    assert "(NVIDIA, b200)" in out, out[:400]
    assert "FAIL" not in out
    m = re.search(r"(\d+) op runs, (\d+) skipped", out)
    assert m, out[-400:]
    runs, skipped = int(m.group(1)), int(m.group(2))
    assert runs >= 69, out[-400:]
    skipped_names = [ln.split()[1].split("/")[0] for ln in out.splitlines() if ln.startswith("SKIP ")]
    for name in skipped_names:
        assert name not in HOT_PATH, f"a decode hot-path op was skipped as unsupported: {name}\n" + "\n".join(ln for ln in out.splitlines() if ln.startswith("SKIP "))
        assert name in OUTSIDE, f"unexpected skip: {name}"
    assert "PASS  CONT_MUL_MAT" in out and "CONT_MUL_MAT V n_kv=520" in out
    print(f"ops_tests: {runs} op runs, {skipped} skipped: {sorted(set(skipped_names))}")


def test_reference_attention_tests_pass_on_cuda_sm100():
    out = run(refapi.ATTENTION_TESTS)
    assert "(cuda_sm100)" in out, out[:400]
    assert "4 attention runs" in out, out[-400:]


def test_reference_ops_tests_pass_through_the_reference_device_server():
    """The reference's scrapgpu-device-server (src/backends/remote/server.cpp) and the client side of its remote backend
    (client.cpp), both compiled unchanged (`make -C oracle remote_tests`): the ops suite spawns the server, which registers
    "opencl11" - answered by cuda_sm100 through the shim - and runs every case through the socket and shared-memory transport
    (ops_tests.cpp:1249-1287).  The same pass / skip picture as in process."""
    if not os.path.exists(refapi.DEVICE_SERVER):
        pytest.fail(f"{refapi.DEVICE_SERVER} is missing on the GPU box: run `make -C oracle remote_tests` where the reference is checked out")
    out = run(refapi.OPS_TESTS_REMOTE, backend="remote")
    assert "FAIL" not in out
    m = re.search(r"(\d+) op runs, (\d+) skipped", out)
    assert m, out[-400:]
    assert int(m.group(1)) >= 60, out[-400:]
    skipped_names = [ln.split()[1].split("/")[0] for ln in out.splitlines() if ln.startswith("SKIP ")]
    for name in skipped_names:
        assert name not in HOT_PATH, f"a decode hot-path op was skipped through the device server: {name}"
    print(f"ops_tests through scrapgpu-device-server: {m.group(1)} op runs, {m.group(2)} skipped")
