"""Plans on cuda_sm100: the node list of a decode layer handed to scrapgpu_plan_build as plain, unfused ops.

The reference's contract for plans is "select once at build, launch cheaply" (docs/API_CONTRACT.md:79-92 of the
reference); the fusions a backend is expected to find between neighbouring nodes are the ones its ggml adapter does per
graph (adapters/ggml/ggml-cl11.cpp:904-1031): RMS_NORM + MUL, ADD + RMS_NORM + MUL, MUL_MATs sharing src1, SET_ROWS
pairs.  Checked here through the reference's own public API (the unmodified core of oracle/_ref driving the plugin):

  * the plan's results equal the results of the same nodes executed one by one with scrapgpu_op_execute -- bit for bit
    where fusion keeps the arithmetic (MUL_MAT_MULTI, SET_ROWS_PAIR, RMS_NORM_MUL, ADD_RMS_NORM_MUL), within the
    reference's device bar of NMSE 1e-6 (tests/ops/ops_tests.cpp:725) where the normalisation moves into the matvec
    launch (its sum of squares is added in another order: the row may differ by one ulp);
  * the first execution (step by step), the second (recorded into a CUDA graph) and later ones (graph replay) agree
    bit for bit, and replays need fewer launches than nodes;
  * the same node list on the reference's CPU backend agrees within NMSE 1e-6;
  * an intermediate result is left unwritten only if output_use_count says the next node is its only reader."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import refapi, sgref
from scrapgpulibrary_b200 import _build, abi
from tests import util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def both():
    if not refapi.available() or not os.path.exists(_build.PLUGIN_SO):
        pytest.fail("oracle/_ref or the prebuilt plugin is missing on the GPU box: build them where the reference is checked out")
    from tests import refsession
    cpu, gpu = refsession.Session("cpu"), refsession.Session("cuda_sm100")
    yield cpu, gpu
    cpu.close()
    gpu.close()


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


HIDDEN, QN, KVN, FFN, CACHE_ROWS = 1024, 512, 128, 2048, 16


class Layer:
    """The tensors and the unfused node list of one decode layer on a session (cpu or cuda_sm100)."""

    def __init__(self, sess, packed: bool):
        lay = abi.LAYOUT_R32 if packed else abi.LAYOUT_NATURAL
        t = self.t = {}
        self.sess = sess

        def weight(name, seed, n, k):
            w = U.quantize(U.Q4_K, U.seeded_weights(seed, n, k))
            t[name] = sess.tensor(abi.Q4_K, [k, n], layout=lay).upload(w)

        weight("wq", 1, QN, HIDDEN)
        weight("wk", 2, KVN, HIDDEN)
        weight("wv", 3, KVN, HIDDEN)
        weight("wo", 4, HIDDEN, QN)
        weight("wgate", 5, FFN, HIDDEN)
        weight("wup", 6, FFN, HIDDEN)
        weight("wdown", 7, HIDDEN, FFN)
        for name, seed, n in (("x", 10, HIDDEN), ("prev", 11, HIDDEN), ("norm1", 12, HIDDEN), ("norm2", 13, HIDDEN)):
            t[name] = sess.tensor(abi.F32, [n]).upload(rnd(seed, n) if "norm" not in name else 1.0 + 0.1 * rnd(seed, n))
        for name, n in (("x1", HIDDEN), ("t1", HIDDEN), ("xn1", HIDDEN), ("q", QN), ("k", KVN), ("v", KVN), ("o", HIDDEN), ("x2", HIDDEN), ("xn2", HIDDEN),
                        ("gate", FFN), ("up", FFN), ("act", FFN), ("down", HIDDEN)):
            t[name] = sess.tensor(abi.F32, [n]).upload(np.full(n, -7.0, np.float32))
        t["ids"] = sess.tensor(abi.I32, [1]).upload(np.array([5], np.int32))
        for name in ("kcache", "vcache"):
            t[name] = sess.tensor(abi.F32, [KVN, CACHE_ROWS]).upload(np.zeros(KVN * CACHE_ROWS, np.float32))
        eps = lambda: abi.RmsNormParams(0, 1e-6)
        mm = lambda: abi.MulMatParams(0, 0)
        T = lambda *names: [t[n] for n in names]
        # (op, inputs, outputs, params, output_use_count)
        self.nodes = [
            (abi.OP_ADD, T("x", "prev"), T("x1"), None, 2),
            (abi.OP_RMS_NORM, T("x1"), T("t1"), eps(), 1),
            (abi.OP_MUL, T("t1", "norm1"), T("xn1"), None, 3),
            (abi.OP_MUL_MAT, T("wq", "xn1"), T("q"), mm(), 1),
            (abi.OP_MUL_MAT, T("wk", "xn1"), T("k"), mm(), 1),
            (abi.OP_MUL_MAT, T("wv", "xn1"), T("v"), mm(), 1),
            (abi.OP_SET_ROWS, T("k", "ids"), T("kcache"), abi.SetRowsParams(0, 0), 0),
            (abi.OP_SET_ROWS, T("v", "ids"), T("vcache"), abi.SetRowsParams(0, 0), 0),
            (abi.OP_MUL_MAT, T("wo", "q"), T("o"), mm(), 1),
            (abi.OP_ADD, T("x1", "o"), T("x2"), None, 2),
            (abi.OP_RMS_NORM_MUL, T("x2", "norm2"), T("xn2"), eps(), 2),
            (abi.OP_MUL_MAT, T("wgate", "xn2"), T("gate"), mm(), 1),
            (abi.OP_MUL_MAT, T("wup", "xn2"), T("up"), mm(), 1),
            (abi.OP_GLU, T("gate", "up"), T("act"), abi.GluParams(0, abi.GLU_SWIGLU, 1, 0), 1),
            (abi.OP_MUL_MAT, T("wdown", "act"), T("down"), mm(), 1),
        ]
        self.outputs = ["x1", "q", "k", "v", "kcache", "vcache", "o", "x2", "gate", "up", "act", "down"]
        # intermediates whose only readers are the following nodes (act is not among them: the launch that makes gate and up
        # also makes the SwiGLU activation and writes it out for the down projection)
        self.elidable = ["t1", "xn1", "xn2"]

    def run_nodes(self):
        for op, ins, outs, params, _ in self.nodes:
            self.sess.execute(op, ins, outs, params)
        self.sess.sync()

    def reset_outputs(self):
        t = self.t
        for name in self.outputs + self.elidable:
            n = int(np.prod([t[name].desc.ne[i] for i in range(4)]))
            t[name].upload(np.zeros(n, np.float32) if "cache" in name else np.full(n, -7.0, np.float32))

    def read(self, names):
        out = {}
        for name in names:
            n = int(np.prod([self.t[name].desc.ne[i] for i in range(4)]))
            out[name] = self.t[name].download(np.float32, n)
        return out

    def build_plan(self, use_counts=True):
        L = refapi.lib()
        self.ops = [abi.Op(op, [x.desc for x in ins], [x.desc for x in outs], params) for op, ins, outs, params, _ in self.nodes]
        arr = (abi.PlanNode * len(self.ops))()
        for i, o in enumerate(self.ops):
            arr[i].struct_size = C.sizeof(abi.PlanNode)
            arr[i].op = o.desc
            arr[i].output_use_count = self.nodes[i][4] if use_counts else 0
        pd = abi.PlanDesc(C.sizeof(abi.PlanDesc), arr, len(self.ops))
        plan = C.c_void_p()
        refapi.check(L.scrapgpu_plan_build(self.sess.device, C.byref(pd), C.byref(plan)), "plan_build")
        return plan


def test_plan_matches_node_by_node_execution_and_replays_as_a_graph(both):
    from tests import refsession
    L = refapi.lib()
    P = refsession.plugin()
    cpu, gpu = both
    glayer, clayer = Layer(gpu, packed=True), Layer(cpu, packed=False)
    clayer.run_nodes()
    want_cpu = clayer.read(clayer.outputs)
    glayer.run_nodes()
    per_op = glayer.read(glayer.outputs + glayer.elidable)
    for name in glayer.outputs:
        assert sgref.nmse(per_op[name], want_cpu[name]) <= 1e-6, name

    plan = glayer.build_plan()
    results, launches = [], []
    for _ in range(4):
        glayer.reset_outputs()
        gpu.sync()
        before = P.scrapgpu_cuda_sm100_launch_count()
        refapi.check(L.scrapgpu_plan_execute(gpu.stream, plan), "plan_execute")
        gpu.sync()
        launches.append(P.scrapgpu_cuda_sm100_launch_count() - before)
        results.append(glayer.read(glayer.outputs + glayer.elidable))
    # 15 nodes: ADD+RMS_NORM+MUL+3 MUL_MAT -> 1 launch, 2 SET_ROWS -> 2 (one op), o -> 1, ADD+RMS_NORM_MUL+2 MUL_MAT+GLU -> 1, down -> 1
    assert launches[0] <= 7, launches          # the step-by-step run counts its launches; replays launch a graph
    assert launches[2] == 0 and launches[3] == 0, launches
    for r in results[1:]:
        for name in glayer.outputs:
            assert np.array_equal(r[name].view(np.uint32), results[0][name].view(np.uint32)), f"{name}: graph replay differs from the first execution"
    first = results[0]
    for name in ("x1", "x2"):    # adds keep their arithmetic under fusion
        assert np.array_equal(first[name].view(np.uint32), per_op[name].view(np.uint32)), name
    # the scattered rows are the k / v projections: node by node the second and third of three consecutive MUL_MATs are
    # served by the ring kernel, in the plan all three by one fused launch of matvec_q4k_imma; the two add the same
    # integer block sums in different orders, every other element of the caches must be untouched
    for name in ("kcache", "vcache"):
        assert sgref.nmse(first[name], per_op[name]) <= 1e-10, name
        assert np.array_equal(first[name] == 0, per_op[name] == 0), name
    for name in glayer.outputs:
        assert sgref.nmse(first[name], per_op[name]) <= 1e-6, name
        assert sgref.nmse(first[name], want_cpu[name]) <= 1e-6, name
    # the caller said that t1, xn1 and xn2 have no other reader: they were not written
    for name in glayer.elidable:
        assert np.all(first[name] == -7.0), f"{name} was written although its only readers were fused with it"
    refapi.check(L.scrapgpu_plan_free(plan), "plan_free")


def test_plan_without_use_counts_keeps_every_intermediate(both):
    """output_use_count = 0 means "not stated": the plan may still fuse launches, but every tensor a node names as
    its output must hold that node's result afterwards."""
    L = refapi.lib()
    cpu, gpu = both
    glayer = Layer(gpu, packed=True)
    glayer.run_nodes()
    per_op = glayer.read(glayer.outputs + glayer.elidable)
    plan = glayer.build_plan(use_counts=False)
    for _ in range(3):
        glayer.reset_outputs()
        refapi.check(L.scrapgpu_plan_execute(gpu.stream, plan), "plan_execute")
        gpu.sync()
        got = glayer.read(glayer.outputs + glayer.elidable)
        for name in glayer.outputs + glayer.elidable:
            assert sgref.nmse(got[name], per_op[name]) <= 1e-6, name
        for name in ("t1", "x1", "x2"):
            assert np.array_equal(got[name].view(np.uint32), per_op[name].view(np.uint32)), name
        # (act = SwiGLU(gate, up): node by node `up` is the second of two consecutive MUL_MATs and comes from the ring
        # kernel, in the plan gate, up and act are one launch of matvec_q4k_imma: same block sums, other order of addition)
        assert sgref.nmse(got["act"], per_op["act"]) <= 1e-10
    refapi.check(L.scrapgpu_plan_free(plan), "plan_free")
